"""Grouped-query attention over the paged cache, with optional per-head RMSNorm of
queries and keys and optional rotary encoding.

Order of operations, as the reference's Qwen3 graph states it
(src/core/model/qwen3/QWen3Creator.cpp:66-140): q,k,v projections without bias ->
reshape to heads -> RMSNorm over head_dim of q and of k with one weight vector each
(:93-101) -> K and V into the cache (:104-108) -> RoPE on q and k -> causal softmax
attention with scale 1/sqrt(head_dim), query head h reading kv head h // (heads/kv_heads)
(src/kernel/cuda/paged_flash_attention.cu:891-892, :1158) -> output projection ->
residual add.  The reference caches un-rotated keys and rotates them on every read;
here keys are rotated once, before they are written, which is algebraically the same.
A ``window`` > 0 lets a query at position p see keys p-window+1 .. p only.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import Mixer, WeightSpec, MATRIX, VECTOR, KVNeed, LayerContext


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm: bool = True, qk_norm_eps: float = 0.0, window: int = 0,
                 softmax_scale: Optional[float] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.qk_norm = bool(qk_norm)
        self.qk_norm_eps = float(qk_norm_eps)
        self.window = int(window)
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.head_dim)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.qk_norm and not self.qk_norm_eps > 0:
            raise ValueError("qk_norm needs qk_norm_eps > 0")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {
            "q_proj.weight": WeightSpec((self.q_width, self.hidden_size), MATRIX),
            "k_proj.weight": WeightSpec((self.kv_width, self.hidden_size), MATRIX),
            "v_proj.weight": WeightSpec((self.kv_width, self.hidden_size), MATRIX),
            "o_proj.weight": WeightSpec((self.hidden_size, self.q_width), MATRIX),
        }
        if self.qk_norm:
            s["q_norm.weight"] = WeightSpec((self.head_dim,), VECTOR, init="one_plus_normal")
            s["k_norm.weight"] = WeightSpec((self.head_dim,), VECTOR, init="one_plus_normal")
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        q, k, v = tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]
        dt = q.dtype if (q.dtype == k.dtype == v.dtype) else torch.float32
        # one projection instead of three: rows [q heads | k heads | v heads]
        self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        if self.qk_norm:
            self.q_norm_w = tensors["q_norm.weight"]
            self.k_norm_w = tensors["k_norm.weight"]

    def forward(self, h, ctx: LayerContext, residual):
        ops, batch = ctx.ops, ctx.batch
        T = h.shape[0]
        # projection, q/k norm, rotation, cache write and attention: how many kernels that is, is the kernel
        # library's business; the projection's accumulators stay in float32 until q and k have been normalised
        rot = ctx.position.rotary() if ctx.position is not None else None
        attn = torch.empty((T, self.q_width), dtype=h.dtype, device=h.device)
        ops.attend(h, self.w_qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
                   rot[0] if rot else None, rot[1] if rot else 0,
                   batch, ctx.block_table, ctx.kv_cache, ctx.kv_layer, ctx.page_size, attn,
                   self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window, ctx.write_cache)
        ops.gemm(attn, self.w_o, residual, residual=residual)
        return residual
