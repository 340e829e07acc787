"""Turns the logits of a step into one token per row, on the device.

The uniform number of a draw is a function of (seed, request key, index of the token
being generated) alone -- a counter-based generator, where the reference seeds a
thread-local mt19937 from random_device (src/core/runtime/InferRuntime.cu:240) -- so
a request's tokens do not depend on which other requests share its steps, and a
request that was preempted and recomputed continues with the same draws."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .params import SamplingParams

_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_for(seed: int, request_key: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32)."""
    h = _splitmix64(seed & _M64)
    h = _splitmix64(h ^ (request_key & _M64))
    h = _splitmix64(h ^ (index & _M64))
    return (h >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], request_keys: Sequence[int],
               indices: Sequence[int], seen_tokens: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """logits float32 [R, V]; row r belongs to a request with params[r], key request_keys[r],
        generating its token number indices[r]; seen_tokens[r] (prompt + generated) is needed only
        when a repetition penalty is set.  Returns int32 [R] on the device."""
        R = logits.shape[0]
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        if R == 0:
            return out
        if any(p.repetition_penalty != 1.0 for p in params):
            self._penalize(logits, params, seen_tokens)
        if all(p.is_greedy for p in params):
            self.ops.argmax(logits, out)
            return out
        host = np.zeros((5, R), dtype=np.float32)
        ks = np.zeros(R, dtype=np.int32)
        for r, p in enumerate(params):
            host[0, r] = 0.0 if p.is_greedy else p.temperature
            host[1, r] = uniform_for(p.seed, request_keys[r], indices[r])
            host[2, r] = p.top_p
            host[3, r] = p.min_p
            ks[r] = p.top_k
        use_filters = any((p.top_k > 0 or p.top_p < 1.0 or p.min_p > 0.0) and not p.is_greedy for p in params)
        dev = torch.from_numpy(host).to(logits.device)
        kd = torch.from_numpy(ks).to(logits.device) if use_filters else None
        self.ops.sample(logits, dev[0], dev[1], out,
                        top_k=kd, top_p=dev[2] if use_filters else None, min_p=dev[3] if use_filters else None)
        return out

    def _penalize(self, logits, params, seen_tokens) -> None:
        """logit > 0 -> logit / penalty, else logit * penalty, once per distinct seen token
        (src/core/sampler/LLMSampler.cpp:21-34)."""
        rows, toks, pens = [], [], []
        for r, p in enumerate(params):
            if p.repetition_penalty == 1.0 or not seen_tokens or not seen_tokens[r]:
                continue
            u = sorted(set(int(t) for t in seen_tokens[r]))
            rows.extend([r] * len(u))
            toks.extend(u)
            pens.extend([p.repetition_penalty] * len(u))
        if not rows:
            return
        dev = logits.device
        self.ops.repetition_penalty(logits,
                                    torch.tensor(rows, dtype=torch.int32, device=dev),
                                    torch.tensor(toks, dtype=torch.int32, device=dev),
                                    torch.tensor(pens, dtype=torch.float32, device=dev))
