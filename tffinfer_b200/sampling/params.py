"""Sampling options of one request, named after the reference's SamplingConfig
(src/core/sampler/LLMSampler.h:55-63: _type, _temperature, _top_k, _top_p, _min_p,
_repetition_penalty, _seed).  The reference's ``sample`` ignores all of them and
returns the first maximum (LLMSampler.cpp:13-19); its helpers for temperature,
repetition penalty and multinomial draws exist unused (LLMSampler.cpp:21-54).  Here
they are honoured."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

GREEDY = "greedy"
RANDOM = "random"
TOP_K = "top_k"
TOP_P = "top_p"
STRATEGIES = ("default", GREEDY, RANDOM, TOP_K, TOP_P)   # FOR_EACH_STRATEGY, LLMSampler.h:18-24


@dataclass(frozen=True)
class SamplingParams:
    type: str = GREEDY                 # "greedy": temperature and filters are ignored
    temperature: float = 1.0
    top_k: int = 0                     # 0 = off
    top_p: float = 1.0                 # 1 = off
    min_p: float = 0.0                 # 0 = off
    repetition_penalty: float = 1.0    # 1 = off
    seed: int = 0
    max_new_tokens: int = 16
    eos_token_ids: Tuple[int, ...] = ()

    def __post_init__(self):
        if self.type not in STRATEGIES:
            raise ValueError(f"sampling type must be one of {STRATEGIES}, got '{self.type}'")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0 or not (0 < self.top_p <= 1.0) or not (0 <= self.min_p < 1.0):
            raise ValueError("top_k >= 0, 0 < top_p <= 1 and 0 <= min_p < 1 are required")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")

    @property
    def is_greedy(self) -> bool:
        return self.type in (GREEDY, "default") or self.temperature == 0.0

    @staticmethod
    def make(temperature: float = 0.0, **kw) -> "SamplingParams":
        """temperature 0 -> greedy; otherwise random sampling with the given filters."""
        if temperature == 0.0:
            return SamplingParams(type=GREEDY, temperature=1.0, **kw)
        t = TOP_K if kw.get("top_k", 0) > 0 else TOP_P if kw.get("top_p", 1.0) < 1.0 else RANDOM
        return SamplingParams(type=t, temperature=temperature, **kw)
