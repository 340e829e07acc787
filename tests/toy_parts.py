"""Toy parts defined outside the framework: a mixer with state of its own, a routed
feed-forward, an absolute position encoding, an arrangement with norms after the mixer and
after the feed-forward as well as before them, a scaled embedding and capped logits, and an
architecture made of them.  They
exist to show that parts and architectures can be registered, built and stepped
without a change to the framework's files.  They are not a model of anyone's."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from tffinfer_b200 import register_part, register_architecture
from tffinfer_b200.config import ModelConfig
from tffinfer_b200.parts import (Mixer, FeedForward, PositionEncoding, Block, WeightSpec, MATRIX, VECTOR, StateNeed,
                                 ModelDescription, LayerSpec, PartSpec, ScheduleEntry)

LOGIT_SCALE, LOGIT_SOFTCAP = 0.5, 5.0


@register_part("mixer", "toy_running_mean", replace=True)
class RunningMeanMixer(Mixer):
    """out_t = W . mean(h_0 .. h_t).  The state is the running sum and the count."""
    def __init__(self, hidden_size: int, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size = hidden_size

    def cache_need(self):
        return StateNeed((self.hidden_size + 1,), "float32")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"mix.weight": WeightSpec((self.hidden_size, self.hidden_size), MATRIX)}

    def load(self, tensors, ops, act_dtype):
        self.w = tensors["mix.weight"]

    def forward(self, h, ctx, residual):
        # Everything stays on the device and no shape depends on the batch's values, so that a decode
        # step with this mixer can be captured in a CUDA graph: the running sum of each request's rows is
        # the running sum over all rows minus what the rows ahead of the request add up to.
        b = ctx.batch
        H = self.hidden_size
        D = torch.float64
        req = b.tok_req.long()
        first = b.q_start[:-1].long()                    # first row of each request
        last = b.q_start[1:].long() - 1                  # last row of each request
        slots = b.slots.long()
        st = ctx.state.index_select(0, slots).to(D)      # [B, H + 1]: running sum, count
        total = torch.cumsum(h.to(D), 0)
        ahead = total.index_select(0, first) - h.to(D).index_select(0, first)
        csum = total - ahead.index_select(0, req) + st[:, :H].index_select(0, req)
        rows = torch.arange(h.shape[0], device=h.device)
        cnt = st[:, H].index_select(0, req) + (rows - first.index_select(0, req) + 1).to(D)
        mean = (csum / cnt[:, None]).to(torch.float32)
        new_state = torch.cat([csum.index_select(0, last), cnt.index_select(0, last)[:, None]], dim=1)
        ctx.state.index_copy_(0, slots, new_state.to(ctx.state.dtype))
        out = torch.empty_like(residual)
        ctx.ops.gemm(mean.to(h.dtype), self.w, out)
        residual += out
        return residual


@register_part("feed_forward", "toy_top1_experts", replace=True)
class Top1Experts(FeedForward):
    """Router logits in float32, one expert per token, each expert a single matrix."""
    def __init__(self, hidden_size: int, num_experts: int, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.num_experts = hidden_size, num_experts

    def weight_specs(self):
        s = {"router.weight": WeightSpec((self.num_experts, self.hidden_size), VECTOR, init="normal", init_scale=0.5)}
        for e in range(self.num_experts):
            s[f"experts.{e}.weight"] = WeightSpec((self.hidden_size, self.hidden_size), MATRIX)
        return s

    def load(self, tensors, ops, act_dtype):
        self.router = tensors["router.weight"]
        self.experts = [tensors[f"experts.{e}.weight"] for e in range(self.num_experts)]

    def forward(self, h, ctx, residual):
        # every expert runs on every row and the router's choice picks one result: wasteful, and free of
        # shapes that depend on the data (a toy, and a decode step with it can be captured in a CUDA graph)
        choice = (h.float() @ self.router.t()).argmax(-1)
        for e in range(self.num_experts):
            out = torch.empty((h.shape[0], self.hidden_size), dtype=torch.float32, device=h.device)
            ctx.ops.gemm(h, self.experts[e], out)
            residual += torch.where((choice == e)[:, None], out, torch.zeros_like(out))
        return residual


@register_part("position", "toy_learned_absolute", replace=True)
class LearnedAbsolute(PositionEncoding):
    """A learned vector per position, added to the residual stream after the embedding."""
    def __init__(self, hidden_size: int, max_position: int, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.max_position = hidden_size, max_position

    def weight_specs(self):
        return {"weight": WeightSpec((self.max_position, self.hidden_size), VECTOR, init="normal", init_scale=0.02)}

    def load(self, tensors, ops, act_dtype):
        self.table = tensors["weight"]

    def embed(self, x, batch, ops):
        return x + self.table[batch.positions.long()]


@register_part("block", "toy_sandwich", replace=True)
class SandwichBlock(Block):
    """x + norm(mixer(norm(x))), then x + norm(ffn(norm(x))): the two norms behind the parts come from the
    layer's ``extra_norms``."""
    def forward(self, x, ctx, act_dtype):
        h = self.mixer_norm.forward(x, ctx.ops, act_dtype)
        m = self.mixer.forward(h, ctx, residual=torch.zeros_like(x))
        x = x + self.extra_norms["post_mixer"].forward(m, ctx.ops, torch.float32)
        h = self.ffn_norm.forward(x, ctx.ops, act_dtype)
        f = self.feed_forward.forward(h, ctx, residual=torch.zeros_like(x))
        return x + self.extra_norms["post_ffn"].forward(f, ctx.ops, torch.float32)


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    hidden_size: int = 48
    vocab_size: int = 97
    num_layers: int = 3
    num_experts: int = 3
    max_position: int = 128
    eps: float = 1e-5

    @staticmethod
    def from_json_dict(d):
        return ToyConfig(architecture=d["architectures"][0], hidden_size=d["hidden_size"], vocab_size=d["vocab_size"],
                         num_layers=d["num_layers"], num_experts=d["num_experts"],
                         max_position=d["max_position"], eps=d["eps"])

    def to_json_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "num_layers": self.num_layers, "num_experts": self.num_experts, "max_position": self.max_position,
                "eps": self.eps}


def describe_toy(cfg: ToyConfig) -> ModelDescription:
    H = cfg.hidden_size
    layers = []
    for i in range(cfg.num_layers):
        p = f"blocks.{i}"
        if i % 2 == 0:
            mixer = PartSpec("toy_running_mean", dict(hidden_size=H), prefix=f"{p}.mixer")
        else:
            mixer = PartSpec("gqa_attention", dict(hidden_size=H, num_heads=3, num_kv_heads=1, head_dim=16,
                                                   qk_norm=False, window=0), prefix=f"{p}.mixer")
        ffn = (PartSpec("toy_top1_experts", dict(hidden_size=H, num_experts=cfg.num_experts), prefix=f"{p}.ffn")
               if i % 2 == 0 else PartSpec("swiglu", dict(hidden_size=H, intermediate_size=2 * H), prefix=f"{p}.ffn"))
        norm = lambda name: PartSpec("rms_norm", dict(dim=H, eps=cfg.eps), prefix=f"{p}.{name}")
        layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"), ffn_norm=norm("norm2"),
                                block="pre_norm" if i % 2 == 0 else "toy_sandwich",
                                extra_norms={} if i % 2 == 0 else {"post_mixer": norm("norm3"), "post_ffn": norm("norm4")},
                                position=None))
    # layer 0 runs twice (each run with a state of its own); the last run of the attention
    # layer reads the cache of its first run instead of keeping one
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)]
    return ModelDescription(
        hidden_size=H, vocab_size=cfg.vocab_size, max_position=cfg.max_position,
        embed_name="embed.weight", lm_head_name="head.weight",
        final_norm=PartSpec("rms_norm", dict(dim=H, eps=cfg.eps), prefix="final_norm"),
        layers=layers, schedule=schedule,
        positions={"abs": PartSpec("toy_learned_absolute", dict(hidden_size=H, max_position=cfg.max_position),
                                   prefix="positions")},
        embed_scale=float(H) ** 0.5, logit_scale=LOGIT_SCALE, logit_softcap=LOGIT_SOFTCAP)


def register_toy():
    register_architecture("ToyStateLM", ToyConfig.from_json_dict, describe_toy, replace=True)


# ------------------------------------------------------------------ plain whole-sequence twin
def toy_plain_logits(tokens, w: Dict[str, torch.Tensor], cfg: ToyConfig) -> torch.Tensor:
    import math
    D = torch.float64
    w = {k: v.to(D) for k, v in w.items()}
    H = cfg.hidden_size
    T = len(tokens)

    def norm(x, name):
        return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + cfg.eps)) * w[name]

    x = w["embed.weight"][torch.tensor(tokens)] * float(H) ** 0.5 + w["positions.weight"][:T]
    kv_of_layer1 = None
    for e, li in enumerate([0, 1, 2, 0, 1]):
        p = f"blocks.{li}"
        h = norm(x, f"{p}.norm1.weight")
        if li % 2 == 0:
            mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=D)[:, None]
            x = x + mean @ w[f"{p}.mixer.mix.weight"].t()
        else:
            q = (h @ w[f"{p}.mixer.q_proj.weight"].t()).view(T, 3, 16)
            if e == 1:
                k = (h @ w[f"{p}.mixer.k_proj.weight"].t()).view(T, 1, 16)
                v = (h @ w[f"{p}.mixer.v_proj.weight"].t()).view(T, 1, 16)
                kv_of_layer1 = (k, v)
            else:
                k, v = kv_of_layer1                      # the borrowed cache
            o = torch.empty(T, 3, 16, dtype=D)
            mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
            for hh in range(3):
                s = (q[:, hh] @ k[:, 0].t()) / math.sqrt(16)
                o[:, hh] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, 0]
            x = x + norm(o.reshape(T, 48) @ w[f"{p}.mixer.o_proj.weight"].t(), f"{p}.norm3.weight")
        h = norm(x, f"{p}.norm2.weight")
        if li % 2 == 0:
            choice = (h @ w[f"{p}.ffn.router.weight"].t()).argmax(-1)
            out = torch.zeros_like(x)
            for ex in range(cfg.num_experts):
                sel = choice == ex
                out[sel] = h[sel] @ w[f"{p}.ffn.experts.{ex}.weight"].t()
            x = x + out
        else:
            g = h @ w[f"{p}.ffn.gate_proj.weight"].t()
            u = h @ w[f"{p}.ffn.up_proj.weight"].t()
            x = x + norm(((g / (1 + torch.exp(-g))) * u) @ w[f"{p}.ffn.down_proj.weight"].t(), f"{p}.norm4.weight")
    logits = norm(x, "final_norm.weight") @ w["head.weight"].t()
    return LOGIT_SOFTCAP * torch.tanh(logits * LOGIT_SCALE / LOGIT_SOFTCAP)
