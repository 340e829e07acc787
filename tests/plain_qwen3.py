"""A plain, slow implementation of Qwen3 dense: whole sequences, no cache, no batch,
one function for each part.  It shares no code with ``tffinfer_b200``: it parses
config.json itself, reads the weights with the ``safetensors`` library, and works in
one floating type (float64 by default, so that it is an oracle for the 32-bit engine).

It rests on the formulas of NKKdev/TFFinfer, cited at each function by the file's path
inside that project.  The reference as a whole cannot be built or imported offline (glog,
Taskflow and libdivide are fetched from the network by its CMakeLists.txt:28-78) and it has no
CPU implementation of the model, but its device code for the norm, the rotation table, the
SiLU product and the rotating causal attention of 32 heads on 8 of 128 depends on nothing of
the project: tests/golden/make_reference_golden.py cut those kernels out of a checkout at run
time and ran them on a B200, tests/golden/reference_outputs.npz keeps what they computed, and
tests/test_reference_golden.py holds ``rms_norm``, ``rope_angles``, ``rope_rotate_half``,
``silu`` and ``causal_attention`` of this file against it.  The embedding, the projections,
the order of the parts in a layer and the sampling rest on the cited formulas alone.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Sequence

import torch


# ----------------------------------------------------------------------------- config
def read_plain_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    L = c["num_hidden_layers"]
    if c.get("layer_types"):
        windows = [c["sliding_window"] if t == "sliding_attention" else 0 for t in c["layer_types"]]
    elif c.get("use_sliding_window") and c.get("sliding_window"):
        windows = [c["sliding_window"] if i >= c.get("max_window_layers", 0) else 0 for i in range(L)]
    else:
        windows = [0] * L
    return dict(
        hidden=c["hidden_size"], layers=L, heads=c["num_attention_heads"], kv_heads=c["num_key_value_heads"],
        head_dim=c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"],
        inter=c["intermediate_size"], vocab=c["vocab_size"], eps=c["rms_norm_eps"], theta=c["rope_theta"],
        max_pos=c["max_position_embeddings"], tied=bool(c.get("tie_word_embeddings", False)), windows=windows)


def read_plain_weights(model_dir: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return {k: v.to(dtype) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


# ------------------------------------------------------------------------------ parts
def embedding(tokens: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """x[t] = E[token[t]], no scale factor (src/core/model/qwen3/QWen3Creator.cpp:283-321;
    src/kernel/cpu/embedding.cpp:35-49)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x * rsqrt(mean(x^2) + eps)) * w over the last axis; the weight multiplies as it is
    (src/kernel/cuda/norm.cu:31-48; src/core/model/base/ModelCreatorBase.cpp:198-221)."""
    r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (x * r) * w


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x . W^T with W stored [out, in], no bias (src/core/model/base/ModelCreatorBase.cpp:121-175;
    weight rows are outputs: src/kernel/cuda/quant/quant_q_8_0_mat_mul.cu:481-484)."""
    return x @ w.t()


def rope_angles(positions: Sequence[int], dim: int, theta: float) -> torch.Tensor:
    """angle[p, i] = p * exp(-(2i/dim) * ln(theta)), i < dim/2 (src/kernel/cuda/rope_table.cu:33-34).
    The frequency is rounded to float32 and the product is one float32 multiplication, as on
    the device; cos and sin are then taken in the working type."""
    i = torch.arange(dim // 2, dtype=torch.float64)
    inv_freq = torch.exp(-(2.0 * i / dim) * math.log(theta)).to(torch.float32)
    p = torch.as_tensor(list(positions), dtype=torch.float32)
    return p[:, None] * inv_freq[None, :]            # float32 [T, dim/2]


def rope_rotate_half(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """Rotate-half ("NEOX") pairing over the whole head: (a, b) = (x[i], x[i + d/2]) ->
    (a cos - b sin, a sin + b cos) (src/kernel/cuda/paged_flash_attention.cu:300-384 for keys,
    :390-481 for queries).  x: [T, heads, d]; angles: [T, d/2]."""
    half = x.shape[-1] // 2
    angles = angles.to(x.device)
    cos = torch.cos(angles.to(torch.float64)).to(x.dtype)[:, None, :]
    sin = torch.sin(angles.to(torch.float64)).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """q: [T, heads, d]; k, v: [T, kv_heads, d].  Query head h reads kv head h // (heads/kv_heads)
    (src/kernel/cuda/paged_flash_attention.cu:891-892); scores (q.k) / sqrt(d) (:1158), keys at
    positions <= the query's (mask 0 / -inf, src/kernel/cuda/mask_op.cu:39), softmax, times v
    (:696-792).  window > 0: only the last ``window`` keys, the query's own included."""
    T, H, d = q.shape
    G = H // k.shape[1]
    out = torch.empty_like(q)
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= pos[None, :] > pos[:, None] - window
    for h in range(H):
        g = h // G
        s = (q[:, h, :] @ k[:, g, :].t()) / math.sqrt(d)
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    positions: Sequence[int], window: int) -> torch.Tensor:
    """Projections -> per-head RMSNorm of q and k (one weight vector of length d each, same
    eps as the block norms, before RoPE; src/core/model/qwen3/QWen3Creator.cpp:66-101) -> RoPE
    -> attention -> output projection (ModelCreatorBase.cpp:242-283)."""
    T = h.shape[0]
    H, KV, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    q = linear(h, w[f"{prefix}.q_proj.weight"]).view(T, H, d)
    k = linear(h, w[f"{prefix}.k_proj.weight"]).view(T, KV, d)
    v = linear(h, w[f"{prefix}.v_proj.weight"]).view(T, KV, d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["eps"])
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["eps"])
    ang = rope_angles(positions, d, cfg["theta"])
    q, k = rope_rotate_half(q, ang), rope_rotate_half(k, ang)
    o = causal_attention(q, k, v, window)
    return linear(o.reshape(T, H * d), w[f"{prefix}.o_proj.weight"])


def silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x)) (src/kernel/cuda/unary.cu:10-12)."""
    return x / (1.0 + torch.exp(-x))


def swiglu_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)) (src/core/model/base/ModelCreatorBase.cpp:51-94;
    src/kernel/cuda/unary.cu:26: op(x1) * x2 with x1 = gate, x2 = up)."""
    return linear(silu(linear(h, w[f"{prefix}.gate_proj.weight"])) * linear(h, w[f"{prefix}.up_proj.weight"]),
                  w[f"{prefix}.down_proj.weight"])


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict,
                  positions: Sequence[int]) -> torch.Tensor:
    """x1 = x + attn(norm(x)); x2 = x1 + mlp(norm(x1)) (src/core/model/qwen3/QWen3Creator.cpp:62-151)."""
    p = f"model.layers.{i}"
    h = rms_norm(x, w[f"{p}.input_layernorm.weight"], cfg["eps"])
    x = x + attention_block(h, w, f"{p}.self_attn", cfg, positions, cfg["windows"][i])
    h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["eps"])
    return x + swiglu_mlp(h, w, f"{p}.mlp")


def forward_logits(tokens: Sequence[int], w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence: embedding, the layers in order, final norm,
    output projection with the embedding table when tied
    (src/core/model/qwen3/QWen3Creator.cpp:49-165)."""
    positions = list(range(len(tokens)))
    x = embedding(tokens, w["model.embed_tokens.weight"])
    for i in range(cfg["layers"]):
        x = decoder_layer(x, w, i, cfg, positions)
    y = rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return linear(y, head)


class PlainModel:
    """``device``: where the plain arithmetic runs; the large test shapes use the GPU's float64
    units for it, the formulas are the same."""

    def __init__(self, model_dir: str, dtype=torch.float64, device: str = "cpu"):
        self.cfg = read_plain_config(model_dir)
        self.w = {k: v.to(device) for k, v in read_plain_weights(model_dir, dtype).items()}

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        return forward_logits(tokens, self.w, self.cfg).cpu()


# --------------------------------------------------------------------------- sampling
def sample_greedy(logits: torch.Tensor) -> int:
    """First maximum (std::max_element, src/core/sampler/LLMSampler.cpp:43-45)."""
    return int((logits == logits.max()).nonzero()[0].item())


def repetition_penalty(logits: torch.Tensor, seen: Sequence[int], penalty: float) -> torch.Tensor:
    """Once for every distinct token of the prompt and the output so far: a positive logit is divided by
    the penalty, any other multiplied by it (src/core/sampler/LLMSampler.cpp:21-34)."""
    out = logits.clone()
    for t in set(int(x) for x in seen):
        if 0 <= t < out.numel():
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def sample_temperature(logits: torch.Tensor, temperature: float, u: float, top_k: int = 0,
                       top_p: float = 1.0, min_p: float = 0.0) -> int:
    """logits / T (LLMSampler.cpp:36-41), softmax, optional filters named by SamplingConfig
    (LLMSampler.h:55-63), then the first index whose cumulative probability exceeds u * total."""
    if temperature <= 0:
        return sample_greedy(logits)
    z = (logits.to(torch.float64) - logits.max().to(torch.float64)) / temperature
    p = torch.exp(z)
    keep = torch.ones_like(p, dtype=torch.bool)
    if min_p > 0:
        keep &= p >= min_p * p.max()
    if 0 < top_k < p.numel():
        kth = torch.topk(p, top_k).values[-1]
        keep &= p >= kth
    if top_p < 1.0:
        sp, _ = torch.sort(p, descending=True)
        c = torch.cumsum(sp, 0)
        n = int((c < top_p * p.sum()).sum().item()) + 1
        keep &= p >= sp[min(n, p.numel()) - 1]
    p = torch.where(keep, p, torch.zeros_like(p))
    c = torch.cumsum(p, 0)
    idx = int((c > u * c[-1]).nonzero()[0].item())
    return idx
