"""Models whose attention is sharp: the q and k norm weights are scaled up, so that every
query gives most of its weight to a few keys, near or far.  With flat random weights a key
that is read from the wrong page, dropped at a window's edge or left out of a split moves
the logits by one part in hundreds; here it moves them by a large share of their size.
The test first shows that (one changed token far back changes later logits strongly in the
plain implementation) and then compares every way of cutting with the plain implementation.
The scale is the largest at which the rounding of the dtype itself (scores grow with the
square of the scale, and so does what a rounded q or k does to a weight) stays inside the
tolerance that all other tests use."""
import os

import pytest

from helpers import (tiny_config, make_requests, PAGE_SIZE, PROMPT_LENS, trace_tail_decode, trace_portions,
                     trace_mixed, run_trace, first_bad, max_rel_err)
from plain_qwen3 import PlainModel
from tffinfer_b200.config import EngineConfig, write_config_json
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights.random_init import random_state_dict
from tffinfer_b200.weights.safetensors_io import write_safetensors

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def sharp_model_dir(tmp_path, name: str, scale: float) -> str:
    cfg = tiny_config(name)
    tensors = random_state_dict(cfg, seed=99, store_dtype="bfloat16")
    for key, t in tensors.items():
        if key.endswith("q_norm.weight") or key.endswith("k_norm.weight"):
            tensors[key] = (t.float() * scale).to(t.dtype)
    d = os.path.join(str(tmp_path), f"sharp_{name}")
    os.makedirs(d, exist_ok=True)
    write_config_json(d, cfg)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


@pytest.mark.parametrize("name,dtype,scale", [("C", "float32", 2.0), ("D", "float32", 2.0),
                                              ("C", "bfloat16", 1.5), ("D", "bfloat16", 1.5)])
def test_sharp_attention_in_every_cut(tmp_path, name, dtype, scale):
    d = sharp_model_dir(tmp_path, name, scale)
    cfg = tiny_config(name)
    reqs = make_requests(name)
    pm = PlainModel(d)
    want = {r: pm.logits(t) for r, t in reqs.items()}

    # the fault would show: one other token far back moves later logits by far more than the tolerance
    longest = max(reqs.values(), key=len)
    changed = list(longest)
    changed[1] = (changed[1] + 1) % cfg.vocab_size
    moved = max_rel_err(pm.logits(changed)[64:], pm.logits(longest)[64:])
    assert moved > 10 * TOL[dtype], moved

    ps = PAGE_SIZE[name]
    most = max(-(-len(t) // ps) * ps for t in reqs.values())
    traces = {
        "tail": (most, trace_tail_decode(reqs)),
        "portions": (most, trace_portions(reqs)),
        "mixed": (most + most // 2, trace_mixed(reqs, PROMPT_LENS[name], max_live=4, page_size=ps,
                                                pool_tokens=most + most // 2, chunk=7)),
    }
    for mode, (pool, steps) in traces.items():
        runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=ps, max_cache_tokens=pool, max_live_requests=4,
                                             use_cuda_graphs=False))
        for c in runner.kv_caches:
            c.fill_(float("nan"))
        got = run_trace(runner, reqs, steps)
        for r in reqs:
            bad = first_bad(got[r], want[r], TOL[dtype])
            assert bad is None, (f"{name}/{mode}/{dtype}/{r}: first wrong position {bad[0]} "
                                 f"(rel err {bad[1]:.3e}) of {len(reqs[r])}")
