"""Shared equipment of the tests: tiny configurations, model folders in temporary
places, the four ways of cutting the same requests into steps, and the comparison
with the plain implementation."""
from __future__ import annotations

import os
import random
from typing import Dict, List, Sequence

import torch

from tffinfer_b200.config import Qwen3Config
from tffinfer_b200.engine import ModelRunner, StepEntry
from tffinfer_b200.weights import write_random_model

FULL, SLIDE = "full_attention", "sliding_attention"


def tiny_config(name: str) -> Qwen3Config:
    """A, B: the two tiny shapes that differ in every size and option; C adds sliding
    windows on two of its layers, an odd vocabulary and a head size that is no power of two."""
    if name == "A":
        return Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=64, num_layers=2, num_heads=4,
                           num_kv_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
                           rms_norm_eps=1e-6, rope_theta=1e4, max_position=128, tie_word_embeddings=True,
                           layer_types=(FULL,) * 2).validate()
    if name == "B":
        return Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=96, num_layers=3, num_heads=8,
                           num_kv_heads=2, head_dim=32, intermediate_size=160, vocab_size=320,
                           rms_norm_eps=1e-5, rope_theta=1e6, max_position=256, tie_word_embeddings=False,
                           layer_types=(FULL,) * 3).validate()
    if name == "C":
        return Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=80, num_layers=4, num_heads=6,
                           num_kv_heads=3, head_dim=48, intermediate_size=112, vocab_size=311,
                           rms_norm_eps=3e-6, rope_theta=5e5, max_position=512, tie_word_embeddings=False,
                           sliding_window=24, layer_types=(FULL, SLIDE, FULL, SLIDE)).validate()
    if name == "D":   # head size 64, multiples of 8 everywhere: takes the tensor-core kernels in bfloat16
        return Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=128, num_layers=2, num_heads=4,
                           num_kv_heads=2, head_dim=64, intermediate_size=192, vocab_size=264,
                           rms_norm_eps=1e-6, rope_theta=1e5, max_position=1024, tie_word_embeddings=False,
                           sliding_window=40, layer_types=(FULL, SLIDE)).validate()
    raise KeyError(name)


PAGE_SIZE = {"A": 4, "B": 8, "C": 16, "D": 16}
PROMPT_LENS = {"A": [1, 7, 33], "B": [2, 13, 40, 64], "C": [3, 29, 70, 101], "D": [5, 90, 37, 600]}
DECODE_LENS = {"A": 16, "B": 24, "C": 40, "D": 36}


def make_model_dir(tmp_path, name: str, seed: int = 1234, store_dtype: str = "bfloat16") -> str:
    d = os.path.join(str(tmp_path), f"tiny_{name}_{store_dtype}")
    if not os.path.isdir(d):
        write_random_model(d, tiny_config(name), seed=seed, store_dtype=store_dtype)
    return d


def make_requests(name: str, seed: int = 7) -> Dict[str, List[int]]:
    """Full token sequences (prompt + the tokens that will be force-fed as decoded)."""
    rng = random.Random(seed)
    cfg = tiny_config(name)
    out = {}
    for i, n in enumerate(PROMPT_LENS[name]):
        total = n + DECODE_LENS[name]
        out[f"r{i}"] = [rng.randrange(cfg.vocab_size) for _ in range(total)]
    return out


# ------------------------------------------------------------------------------ traces
# A trace is a list of steps; a step is (entries, end) with entries = [(req, start, n)].
def trace_whole(reqs: Dict[str, List[int]]):
    return [([(r, 0, len(t))], [r]) for r, t in reqs.items()]


def trace_tail_decode(reqs: Dict[str, List[int]], tail: int = 32):
    steps = []
    for r, t in reqs.items():
        n = len(t)
        first = max(1, n - tail)
        steps.append(([(r, 0, first)], []))
        for p in range(first, n):
            steps.append(([(r, p, 1)], [r] if p == n - 1 else []))
        if first == n:
            steps[-1] = (steps[-1][0], [r])
    return steps


def trace_portions(reqs: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 5, 3, 11, 2, 4, 2)):
    steps = []
    k = 0
    for r, t in reqs.items():
        p = 0
        while p < len(t):
            n = min(sizes[k % len(sizes)], len(t) - p)
            k += 1
            if len(t) - p - n == 1:        # never leave a lone last token: portions go down to two tokens
                n += 1
            steps.append(([(r, p, n)], [r] if p + n == len(t) else []))
            p += n
    return steps


def trace_mixed(reqs: Dict[str, List[int]], prompt_lens: Sequence[int], max_live: int, page_size: int,
                pool_tokens: int, chunk: int, seed: int = 3):
    """Up to ``max_live`` live requests; portions of prompts beside single decoded tokens of
    others in the same step; a request is admitted only when the pool (in tokens, each
    request rounded up to a multiple of ``round_to``) has room for its whole length, so that
    with a small pool later requests reuse the pages of finished ones."""
    rng = random.Random(seed)
    names = list(reqs)
    plen = dict(zip(names, prompt_lens))
    waiting = list(names)
    live: List[str] = []
    done_at = {r: 0 for r in names}
    steps = []

    def held(r):
        return -(-len(reqs[r]) // page_size) * page_size

    while waiting or live:
        while waiting and len(live) < max_live and sum(held(x) for x in live) + held(waiting[0]) <= pool_tokens:
            live.append(waiting.pop(0))
        assert live, "pool too small for a single request"
        entries, end = [], []
        for r in list(live):
            p = done_at[r]
            total = len(reqs[r])
            if p < plen[r]:
                n = min(rng.choice([chunk, 2, chunk // 2 + 1, 3]), plen[r] - p)
                if plen[r] - p - n == 1 and plen[r] - p >= 2:
                    n += 1
            else:
                n = 1
            if rng.random() < 0.15 and len(live) > 1 and entries:
                continue                                 # a request may sit a step out
            entries.append((r, p, n))
            done_at[r] = p + n
            if p + n == total:
                end.append(r)
                live.remove(r)
        if entries:
            steps.append((entries, end))
    return steps


def run_trace(runner: ModelRunner, reqs: Dict[str, List[int]], steps, poison: bool = False,
              stats: Dict[str, int] = None) -> Dict[str, torch.Tensor]:
    """Feeds the steps through the runner's step function, asking for the logits of every
    token; returns per request a tensor [len, vocab] (float32, on the CPU).

    ``poison``: every page that a step or the end of a request gives back is filled with NaN before the
    next step runs, so that a read of a page the request no longer holds shows in the logits.
    ``stats``: receives ``pages_reused``, the number of times a page id was handed to a request after
    another request had held it."""
    got = {r: [None] * len(t) for r, t in reqs.items()}
    groups = range(len(runner.kv_caches))
    held = {}                                   # (request, group) -> pages it holds
    past_holders = [dict() for _ in groups]     # group -> page -> requests that held it
    reused = 0

    def account(r, released: bool):
        nonlocal reused
        for g in groups:
            now = set() if released else {p for p in runner.cache.block_table(r, g) if p >= 0}
            before = held.get((r, g), set())
            for p in now - before:
                holders = past_holders[g].setdefault(p, set())
                if holders - {r}:
                    reused += 1
                holders.add(r)
            gone = sorted(before - now)
            if poison and gone:
                runner.kv_caches[g][torch.tensor(gone, device=runner.kv_caches[g].device)] = float("nan")
            held[(r, g)] = now

    for entries, end in steps:
        ents = []
        for r, start, n in entries:
            if not runner.cache.is_live(r):
                assert start == 0
                assert runner.add_request(r)
            assert runner.num_tokens(r) == start, (r, runner.num_tokens(r), start)
            ents.append(StepEntry(r, reqs[r][start:start + n], list(range(n))))
        logits = runner.step(ents).float().cpu()
        row = 0
        for r, start, n in entries:
            for i in range(n):
                assert got[r][start + i] is None
                got[r][start + i] = logits[row]
                row += 1
            account(r, released=False)
        for r in end:
            runner.finish_request(r)
            account(r, released=True)
        runner.cache.check()
    if stats is not None:
        stats["pages_reused"] = reused
    return {r: torch.stack(v) for r, v in got.items()}


def steps_to_jsonl(reqs: Dict[str, List[int]], steps) -> List[str]:
    """The steps as the lines bin/trace_run reads, the logits of every token wanted."""
    import json
    return [json.dumps({"step": i, "entries": [{"id": r, "tokens": reqs[r][start:start + n], "want": list(range(n))}
                                               for r, start, n in entries], "end": list(end)})
            for i, (entries, end) in enumerate(steps)]


def max_rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest |got - want| over the largest |want| of the same row."""
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    return float(((got.double() - want.double()).abs() / scale).max())


def first_bad(got: torch.Tensor, want: torch.Tensor, tol: float):
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    err = ((got.double() - want.double()).abs() / scale).amax(dim=-1)
    err = torch.nan_to_num(err, nan=float("inf"))          # a row with a NaN in it is wrong, not within the bar
    bad = (err > tol).nonzero()
    return None if bad.numel() == 0 else (int(bad[0]), float(err[int(bad[0])]))
