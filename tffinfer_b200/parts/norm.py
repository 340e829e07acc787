"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` computed in float32, multiplication
order ``(x * r) * w``, the weight a plain multiplier (no ``1 + w``), as the reference
computes it (src/kernel/cuda/norm.cu:31-48; built by ModelCreatorBase::build_norm,
src/core/model/base/ModelCreatorBase.cpp:198-221)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import Norm, WeightSpec, VECTOR


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    def __init__(self, dim: int, eps: float, prefix: str = ""):
        super().__init__(prefix)
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.dim,), VECTOR, init="one_plus_normal")}

    def load(self, tensors, ops, act_dtype) -> None:
        self.weight = tensors["weight"]

    def deferred(self, x, ops, out_dtype):
        """The norm of ``x`` as an object that the kernel library's products can fold in, or None when the
        library cannot (then ``forward`` runs the norm kernel)."""
        can = getattr(ops, "can_fold_norm", None)
        if can is None or not can(x, self.weight, out_dtype):
            return None
        from ..kernels.library import DeferredNorm
        return DeferredNorm(x, self.weight, self.eps, out_dtype, ops)

    def forward(self, x, ops, out_dtype, row_index=None):
        rows = x.shape[0] if row_index is None else row_index.shape[0]
        out = torch.empty((rows, self.dim), dtype=out_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out, row_index)
        return out
