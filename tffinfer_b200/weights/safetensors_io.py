"""Reader and writer of the safetensors container, written from the format's
description: 8 bytes little-endian header length N, N bytes of JSON mapping each
tensor name to {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to
the end of the header), then the raw little-endian data.  The file is memory-mapped
and tensors are handed out by name, as the reference hands out GGUF tensors from an
mmap by name (src/core/model/gguf/GGUFLoader.cpp:187-217; src/core/model/FileLoader.h:179-210).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file.  ``entries[name] = (dtype_name, shape, begin, end)``."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {}) if isinstance(header, dict) else {}
        self.data_start = 8 + n
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if e - b != count * _DTYPES[dt][1] or b < 0 or self.data_start + e > size:
                raise SafetensorsError(f"{path}: tensor '{name}' data_offsets [{b}, {e}) do not match "
                                       f"shape {list(shape)} dtype {dt} or the file size")
            self.entries[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str):
        dt, shape, _, _ = self.entries[name]
        return _DTYPES[dt][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapping (read-only memory: copy before writing)."""
        dt, shape, b, e = self.entries[name]
        tdt = _DTYPES[dt][0]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self.data_start + b:self.data_start + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # non-writable buffer: tensors are only read
            t = torch.frombuffer(buf, dtype=tdt)
        return t.reshape(shape)

    def close(self):
        # views handed out keep the mapping alive; only the file handle is closed here
        try:
            self._f.close()
        except Exception:
            pass


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """``model.safetensors``, or the shards named by ``model.safetensors.index.json``."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        files = sorted(set(wm.values()))
        if not files:
            raise SafetensorsError(f"{index}: empty weight_map")
        return [SafetensorsFile(os.path.join(model_dir, fn)) for fn in files]
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
