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

    @staticmethod
    def _normed(norm, consumer, x, ctx: LayerContext, act_dtype):
        """The norm's output for ``consumer``.  A part that does nothing with its input but hand it to the kernel
        library's products says so (``takes_deferred_norm``); it may then get the norm not yet run, which the
        library folds into the product where that saves a kernel."""
        if getattr(consumer, "takes_deferred_norm", False) and hasattr(norm, "deferred"):
            d = norm.deferred(x, ctx.ops, act_dtype)
            if d is not None:
                return d
        return norm.forward(x, ctx.ops, act_dtype)

    def forward(self, x, ctx: LayerContext, act_dtype):
        h = self._normed(self.mixer_norm, self.mixer, x, ctx, act_dtype)
        x = self.mixer.forward(h, ctx, residual=x)
        h = self._normed(self.ffn_norm, self.feed_forward, x, ctx, act_dtype)
        x = self.feed_forward.forward(h, ctx, residual=x)
        return x
