"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16,
for every way of cutting the same requests into steps."""
import pytest
import torch

from helpers import (make_model_dir, make_requests, PAGE_SIZE, PROMPT_LENS,
                     trace_whole, trace_tail_decode, trace_portions, trace_mixed, run_trace,
                     first_bad)
from plain_qwen3 import PlainModel
from tffinfer_b200.config import EngineConfig
from tffinfer_b200.engine import ModelRunner

pytestmark = pytest.mark.gpu

# largest |difference| over the row's largest |logit|
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


@pytest.fixture(scope="module")
def plain_logits(tmp_path_factory):
    out = {}
    tmp = tmp_path_factory.mktemp("models")
    for name in ("A", "B", "C", "D"):
        d = make_model_dir(tmp, name)
        reqs = make_requests(name)
        pm = PlainModel(d)
        out[name] = (d, reqs, {r: pm.logits(t) for r, t in reqs.items()})
    return out


def _steps(name, mode, reqs):
    ps = PAGE_SIZE[name]
    longest = max(-(-len(t) // ps) * ps for t in reqs.values())
    if mode == "mixed":
        pool = longest + longest // 2
        return pool, trace_mixed(reqs, PROMPT_LENS[name], max_live=4, page_size=ps, pool_tokens=pool,
                                 chunk=5 if name == "A" else 7)
    return longest, {"whole": trace_whole, "tail": trace_tail_decode, "portions": trace_portions}[mode](reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cut_modes_match_plain(plain_logits, name, mode, dtype):
    d, reqs, want = plain_logits[name]
    pool, steps = _steps(name, mode, reqs)
    ecfg = EngineConfig(dtype=dtype, page_size=PAGE_SIZE[name], max_cache_tokens=pool, max_live_requests=4,
                        use_cuda_graphs=False)
    runner = ModelRunner(d, ecfg)
    # poison the cache: a read of a slot that was never written shows up as NaN
    for c in runner.kv_caches:
        c.fill_(float("nan"))
    stats = {}
    got = run_trace(runner, reqs, steps, poison=True, stats=stats)
    for r in reqs:
        bad = first_bad(got[r], want[r], TOL[dtype])
        assert bad is None, (f"{name}/{mode}/{dtype}/{r}: first wrong position {bad[0]} "
                             f"(rel err {bad[1]:.3e}) of {len(reqs[r])}")
        assert torch.isfinite(got[r]).all()
    assert all(p.num_free == p.num_pages for p in runner.cache.pools)
    if mode == "mixed":
        assert stats["pages_reused"] > 0, "the pool was meant to be so small that pages are used again"


@pytest.mark.parametrize("name", ["B", "D"])
def test_weights_stored_in_32_bits_stay_so_when_serving_in_bfloat16(tmp_path, name):
    """A model folder whose tensors are float32: in the bfloat16 mode they are not narrowed (the products
    with them run on the FFMA kernel), activations and cache are bfloat16, and the logits still follow the
    plain implementation."""
    d = make_model_dir(tmp_path, name, store_dtype="float32")
    reqs = make_requests(name)
    pm = PlainModel(d)
    pool, steps = _steps(name, "portions", reqs)
    runner = ModelRunner(d, EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE[name], max_cache_tokens=pool,
                                         max_live_requests=4, use_cuda_graphs=False))
    assert runner.model.lm_head.dtype == torch.float32 and runner.kv_caches[0].dtype == torch.bfloat16
    got = run_trace(runner, reqs, steps)
    for r, t in reqs.items():
        bad = first_bad(got[r], pm.logits(t), TOL["bfloat16"])
        assert bad is None, (name, r, bad)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_first_tokens_of_a_sequence(plain_logits, name, dtype):
    """The very first tokens: a request that starts with single tokens from an empty cache (the decode
    kernels with one, two, three keys), one that starts with a two-token portion, and a third that
    arrives while the others are under way; every position against the plain implementation."""
    d, reqs, want = plain_logits[name]
    names = list(reqs)[:3]
    some = {r: reqs[r][:min(len(reqs[r]), 12)] for r in names}
    steps, done = [], {r: 0 for r in names}

    def feed(r, n):
        n = min(n, len(some[r]) - done[r])
        if n > 0:
            steps.append(([(r, done[r], n)], []))
            done[r] += n

    first, second = names[0], names[1 % len(names)]
    for _ in range(3):
        feed(first, 1)                      # one token at a time from position 0
    if second != first:
        feed(second, 2)                     # a two-token portion from position 0
    for r in names[2:]:
        feed(r, 1)
    while any(done[r] < len(some[r]) for r in names):
        entries = []
        for r in names:
            if done[r] < len(some[r]):
                entries.append((r, done[r], 1))
                done[r] += 1
        steps.append((entries, []))
    steps[-1] = (steps[-1][0], list(names))
    ecfg = EngineConfig(dtype=dtype, page_size=PAGE_SIZE[name], max_cache_tokens=3 * 16 * 4, max_live_requests=4,
                        use_cuda_graphs=False)
    runner = ModelRunner(d, ecfg)
    for c in runner.kv_caches:
        c.fill_(float("nan"))
    got = run_trace(runner, some, steps)
    for r in names:
        bad = first_bad(got[r], want[r][:len(some[r])], TOL[dtype])
        assert bad is None, f"{name}/{dtype}/{r}: first wrong position {bad[0]} (rel err {bad[1]:.3e})"


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_float32_logits_are_the_same_bits_however_the_requests_are_cut(plain_logits, name):
    """In the 32-bit mode every output element is summed in an order that depends on its own row alone
    (products in k order, norms and softmax per row, keys walked in blocks aligned to absolute positions),
    so the four cuts must agree to the last bit, not merely within rounding."""
    d, reqs, _ = plain_logits[name]
    got = {}
    for mode in ("whole", "tail", "portions", "mixed"):
        pool, steps = _steps(name, mode, reqs)
        runner = ModelRunner(d, EngineConfig(dtype="float32", page_size=PAGE_SIZE[name], max_cache_tokens=pool,
                                             max_live_requests=4, use_cuda_graphs=(mode == "tail")))
        got[mode] = run_trace(runner, reqs, steps)
    for mode in ("tail", "portions", "mixed"):
        for r in reqs:
            same = (got[mode][r] == got["whole"][r]).all(dim=-1)
            assert bool(same.all()), (f"{name}/{mode}/{r}: position {int((~same).nonzero()[0])} differs from the whole "
                                      f"prompt by {float((got[mode][r] - got['whole'][r]).abs().max()):.3e}")


def _trace_decode_together(reqs, prompt_lens, stagger: int = 5):
    """Each prompt in a step of its own, then all requests decode together, one token each a step; request i
    has ``stagger * i`` more of its tokens in its prompt step, so the requests end at different times and the
    batch shrinks from all of them to one."""
    steps, at = [], {}
    names = list(reqs)
    for i, (r, n) in enumerate(zip(names, prompt_lens)):
        first = min(len(reqs[r]) - 1, n + stagger * i)
        steps.append(([(r, 0, first)], []))
        at[r] = first
    while at:
        entries = [(r, p, 1) for r, p in at.items()]
        end = [r for r, p in at.items() if p + 1 == len(reqs[r])]
        steps.append((entries, end))
        at = {r: p + 1 for r, p in at.items() if r not in end}
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_decode_steps_replayed_as_cuda_graphs_match_plain(plain_logits, name, dtype):
    """The path generation takes by default: decode-only steps run from device arrays of fixed size (three
    requests in a bucket of four, the spare row writing to the spare page), captured once per bucket and
    class of how unequal the contexts are, and replayed.  Logits of every position against the plain
    implementation, as in the eager cuts."""
    d, reqs, want = plain_logits[name]
    ps = PAGE_SIZE[name]
    pool = sum(-(-len(t) // ps) * ps for t in reqs.values())
    runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=ps, max_cache_tokens=pool, max_live_requests=4,
                                         use_cuda_graphs=True))
    for c in runner.kv_caches:
        c.fill_(float("nan"))
    steps = _trace_decode_together(reqs, PROMPT_LENS[name])
    got = run_trace(runner, reqs, steps, poison=True)
    for r in reqs:
        bad = first_bad(got[r], want[r], TOL[dtype])
        assert bad is None, f"{name}/{dtype}/{r}: first wrong position {bad[0]} (rel err {bad[1]:.3e})"
    buckets = {b: sorted(st["graphs"]) for b, st in runner._graphs.items() if st["graphs"]}
    assert len(buckets) >= 2, f"the batch was meant to shrink through several buckets: {buckets}"
    assert 4 in buckets and 3 not in buckets, f"three requests run in the bucket of four, one row padded: {buckets}"
    # the tail cut again, each decoded token a replay of the one-request graph
    runner2 = ModelRunner(d, EngineConfig(dtype=dtype, page_size=ps, max_cache_tokens=pool, max_live_requests=4,
                                          use_cuda_graphs=True))
    got = run_trace(runner2, reqs, trace_tail_decode(reqs))
    for r in reqs:
        bad = first_bad(got[r], want[r], TOL[dtype])
        assert bad is None, f"{name}/{dtype}/{r} (tail): first wrong position {bad[0]} (rel err {bad[1]:.3e})"
