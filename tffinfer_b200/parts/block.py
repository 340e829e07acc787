"""Arrangements of the parts around the residual stream.  ``pre_norm`` is the
reference's Qwen3 block (src/core/model/qwen3/QWen3Creator.cpp:62-151):
``x = x + mixer(norm(x)); x = x + ffn(norm(x))``, the stream kept in float32."""
from __future__ import annotations

from ..registry import register_part
from .base import Block, LayerContext


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, mixer, feed_forward, mixer_norm=None, ffn_norm=None, extra_norms=None):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, extra_norms)
        if mixer_norm is None or ffn_norm is None:
            raise ValueError("the pre_norm arrangement needs mixer_norm and ffn_norm")

    def forward(self, x, ctx: LayerContext, act_dtype):
        h = self.mixer_norm.forward(x, ctx.ops, act_dtype)
        x = self.mixer.forward(h, ctx, residual=x)
        h = self.ffn_norm.forward(x, ctx.ops, act_dtype)
        x = self.feed_forward.forward(h, ctx, residual=x)
        return x
