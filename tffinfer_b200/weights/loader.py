"""Weights by tensor name, with one error that says everything that is wrong.

The reference looks tensors up by name in ``weight_map`` and dereferences an
unknown tensor type unchecked (src/core/runtime/InferRuntime.cu:546-585, :553); a
missing weight silently yields a null graph node.  Here every tensor the parts ask
for is checked against the files first, and a single :class:`WeightError` lists the
missing tensors, the unexpected ones and the wrong shapes.

Dtype policy.  A tensor stored in 16 bits (bfloat16/float16) is held in bfloat16
when the engine computes in bfloat16, and widened (exactly) to float32 when the
engine computes in float32.  A tensor stored in 32 bits stays in 32 bits in either
mode.  Small per-channel vectors (norm weights) are always widened to float32, which
changes no value.  Integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.base import WeightSpec, VECTOR, INT_TABLE
from .safetensors_io import SafetensorsFile, open_model_files


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, duplicates=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        self.duplicates = list(duplicates)
        lines = ["model weights do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unusable dtypes ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n}: {d}" for n, d in self.wrong_dtype))
        if self.duplicates:
            lines.append(f"  stored in more than one file ({len(self.duplicates)}): " + ", ".join(self.duplicates))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def held_dtype(stored: torch.dtype, role: str, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is held in on the device (see the module docstring)."""
    if role == INT_TABLE:
        return torch.int32
    if role == VECTOR:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return compute  # stored in 16 bits: bfloat16 when serving, float32 in the 32-bit mode


def check_and_load(files: List[SafetensorsFile], expected: Dict[str, WeightSpec],
                   compute_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    where: Dict[str, SafetensorsFile] = {}
    duplicates = []
    for f in files:
        for n in f.names():
            if n in where:
                duplicates.append(n)
            where[n] = f
    missing = [n for n in expected if n not in where]
    unexpected = [n for n in where if n not in expected]
    wrong_shape, wrong_dtype = [], []
    for n, spec in expected.items():
        if n not in where:
            continue
        dt, shape = where[n].info(n)
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((n, spec.shape, shape))
        if spec.role == INT_TABLE and dt not in _INTS:
            wrong_dtype.append((n, f"{dt} stored where an integer table is expected"))
        if spec.role != INT_TABLE and dt not in _FLOATS:
            wrong_dtype.append((n, f"{dt} stored where floating point is expected"))
    if missing or unexpected or wrong_shape or wrong_dtype or duplicates:
        raise WeightError(sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype, sorted(set(duplicates)))
    out: Dict[str, torch.Tensor] = {}
    for n, spec in expected.items():
        t = where[n].tensor(n)
        out[n] = t.to(device=device, dtype=held_dtype(t.dtype, spec.role, compute_dtype)).contiguous()
    return out


def load_model_weights(model_dir: str, expected: Dict[str, WeightSpec],
                       compute_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    files = open_model_files(model_dir)
    try:
        return check_and_load(files, expected, compute_dtype, device)
    finally:
        for f in files:
            f.close()


def check_tensors(tensors: Dict[str, torch.Tensor], expected: Dict[str, WeightSpec],
                  compute_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """The same checks and dtype policy for tensors that are already in memory."""
    missing = sorted(n for n in expected if n not in tensors)
    unexpected = sorted(n for n in tensors if n not in expected)
    wrong_shape = [(n, expected[n].shape, tuple(tensors[n].shape)) for n in expected
                   if n in tensors and tuple(tensors[n].shape) != tuple(expected[n].shape)]
    wrong_dtype = []
    for n, spec in expected.items():
        if n in tensors:
            dt = tensors[n].dtype
            if spec.role == INT_TABLE and dt not in _INTS:
                wrong_dtype.append((n, f"{dt} given where an integer table is expected"))
            if spec.role != INT_TABLE and dt not in _FLOATS:
                wrong_dtype.append((n, f"{dt} given where floating point is expected"))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)
    return {n: tensors[n].to(device=device, dtype=held_dtype(tensors[n].dtype, spec.role, compute_dtype)).contiguous()
            for n, spec in expected.items()}
