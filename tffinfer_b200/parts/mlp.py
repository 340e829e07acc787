"""Dense gated feed-forward: ``down( silu(gate(h)) * up(h) )`` without biases, with
``silu(g) = g / (1 + exp(-g))`` as the reference computes it
(src/kernel/cuda/unary.cu:10-27; built by ModelCreatorBase::build_ffn,
src/core/model/base/ModelCreatorBase.cpp:51-94), followed by the residual add
(src/core/model/qwen3/QWen3Creator.cpp:148-151)."""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import FeedForward, WeightSpec, MATRIX


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    takes_deferred_norm = True        # the input only feeds the gate/up product

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            "gate_proj.weight": WeightSpec((self.intermediate_size, self.hidden_size), MATRIX),
            "up_proj.weight": WeightSpec((self.intermediate_size, self.hidden_size), MATRIX),
            "down_proj.weight": WeightSpec((self.hidden_size, self.intermediate_size), MATRIX),
        }

    def load(self, tensors, ops, act_dtype) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        # one projection instead of two; the kernel library chooses how gate and up rows are laid out
        self.w_gate_up = ops.merge_gate_up(g.to(dt), u.to(dt))
        self.w_down = tensors["down_proj.weight"]

    def forward(self, h, ctx, residual):
        ctx.ops.gated_mlp(h, self.w_gate_up, self.w_down, residual, self.intermediate_size)
        return residual
