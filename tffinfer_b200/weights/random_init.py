"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
typed configuration and a seed.  The reference has no such mode; its only weights
are GGUF files.  Every tensor has a random stream of its own, derived from the seed
and the tensor's name, so values do not depend on the order tensors are visited in.
Matrices are N(0, init_std); norm weights are 1 + N(0, scale) (scale 0 gives ones).
"""
from __future__ import annotations

import hashlib
import os
from typing import Dict

import torch

from ..config.model_config import ModelConfig, write_config_json
from ..parts.base import WeightSpec, INT_TABLE
from ..parts.model import Model
from ..registry import get_architecture
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _stream(seed: int, name: str) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensor(seed: int, name: str, spec: WeightSpec, init_std: float, norm_noise: float,
                  store_dtype: torch.dtype) -> torch.Tensor:
    g = _stream(seed, name)
    if spec.role == INT_TABLE:
        return torch.zeros(spec.shape, dtype=torch.int32)
    if spec.init == "zeros":
        t = torch.zeros(spec.shape, dtype=torch.float32)
    elif spec.init == "one_plus_normal":
        s = norm_noise if spec.init_scale is None else spec.init_scale
        t = 1.0 + s * torch.randn(spec.shape, generator=g, dtype=torch.float32)
    else:
        s = init_std if spec.init_scale is None else spec.init_scale
        t = s * torch.randn(spec.shape, generator=g, dtype=torch.float32)
    return t.to(store_dtype)


def random_state_dict(cfg: ModelConfig, seed: int, store_dtype: str = "bfloat16",
                      norm_noise: float = 0.1) -> Dict[str, torch.Tensor]:
    arch = get_architecture(cfg.architecture)
    desc = arch.describe(cfg)
    model = Model(desc)
    sd = _STORE[store_dtype]
    return {name: random_tensor(seed, name, spec, desc.init_std, norm_noise, sd)
            for name, spec in model.expected_tensors().items()}


def write_random_model(model_dir: str, cfg: ModelConfig, seed: int, store_dtype: str = "bfloat16",
                       norm_noise: float = 0.1) -> str:
    """Create ``model_dir`` with config.json and model.safetensors.  Returns the folder."""
    os.makedirs(model_dir, exist_ok=True)
    write_config_json(model_dir, cfg)
    tensors = random_state_dict(cfg, seed, store_dtype, norm_noise)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir


def random_tensors_on_device(cfg: ModelConfig, seed: int, device, store_dtype: str = "bfloat16",
                             norm_noise: float = 0.0) -> Dict[str, torch.Tensor]:
    """Random weights made on the device, for shapes too large to go through a file
    quickly (benchmarks).  Matrices are N(0, init_std); norm weights 1 + N(0, norm_noise)."""
    arch = get_architecture(cfg.architecture)
    desc = arch.describe(cfg)
    model = Model(desc)
    sd = _STORE[store_dtype]
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = {}
    for name, spec in model.expected_tensors().items():
        if spec.role == INT_TABLE:
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.init == "one_plus_normal":
            s = norm_noise if spec.init_scale is None else spec.init_scale
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
            if s:
                t += s * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
            out[name] = t.to(sd)
        elif spec.init == "zeros":
            out[name] = torch.zeros(spec.shape, dtype=sd, device=device)
        else:
            s = desc.init_std if spec.init_scale is None else spec.init_scale
            t = torch.empty(spec.shape, dtype=sd, device=device)
            t.normal_(0.0, s, generator=gen)
            out[name] = t
    return out
