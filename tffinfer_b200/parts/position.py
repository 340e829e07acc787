"""Rotary position encoding, rotate-half ("NEOX") pairing, as the reference applies it
inside its attention kernel (src/kernel/cuda/paged_flash_attention.cu:300-384 for K,
:390-481 for Q) from a table of (cos, sin) of ``pos * exp(-(2i/d) * ln(base))``
(src/kernel/cuda/rope_table.cu:33-36).  The whole head is rotated unless
``rotary_dim`` says otherwise.  The table is float32 and is built by a kernel once."""
from __future__ import annotations

import torch

from ..registry import register_part
from .base import PositionEncoding


@register_part("position", "rotary")
class RotaryPosition(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int = 0, prefix: str = ""):
        super().__init__(prefix)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim) if rotary_dim else int(head_dim)
        self.theta = float(theta)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim {self.head_dim}")
        self.table = None

    def prepare(self, ops, device, max_position: int) -> None:
        self.table = torch.empty((max_position, self.rotary_dim // 2, 2), dtype=torch.float32, device=device)
        ops.rope_table(self.table, self.theta, self.rotary_dim)

    def rotary(self):
        return self.table, self.rotary_dim


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, prefix: str = ""):
        super().__init__(prefix)
