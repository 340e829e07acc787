"""The step function, the cache manager and the batch builder on the CPU, with the
kernels replaced by their plain twins (tests/cpu_ops.py): every way of cutting the
same requests into steps gives the logits of the plain whole-sequence implementation."""
import pytest

from cpu_ops import CpuOps
from helpers import (make_model_dir, make_requests, PAGE_SIZE, PROMPT_LENS,
                     trace_whole, trace_tail_decode, trace_portions, trace_mixed, run_trace, max_rel_err)
from plain_qwen3 import PlainModel
from tffinfer_b200.config import EngineConfig
from tffinfer_b200.engine import ModelRunner

TOL = 2e-5   # float32 activations against a float64 oracle


def _runner(model_dir, name, pool_tokens):
    ecfg = EngineConfig(dtype="float32", page_size=PAGE_SIZE[name], max_cache_tokens=pool_tokens,
                        max_live_requests=4, device="cpu")
    return ModelRunner(model_dir, ecfg, ops=CpuOps())


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


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cut_modes_match_plain(plain_logits, name, mode):
    d, reqs, want = plain_logits[name]
    ps = PAGE_SIZE[name]
    longest = max(-(-len(t) // ps) * ps for t in reqs.values())
    if mode == "mixed":
        pool = longest + longest // 2
        steps = trace_mixed(reqs, PROMPT_LENS[name], max_live=4, page_size=ps, pool_tokens=pool,
                            chunk=5 if name == "A" else 7)
    else:
        pool = longest
        steps = {"whole": trace_whole, "tail": trace_tail_decode, "portions": trace_portions}[mode](reqs)
    runner = _runner(d, name, pool)
    stats = {}
    got = run_trace(runner, reqs, steps, poison=True, stats=stats)
    for r in reqs:
        err = max_rel_err(got[r], want[r])
        assert err < TOL, f"{name}/{mode}/{r}: rel err {err:.3e}"
    if mode == "mixed":
        assert stats["pages_reused"] > 0, "the pool was meant to be so small that pages are used again"
    assert all(p.num_free == p.num_pages for p in runner.cache.pools)
    assert runner.cache.slots.num_free == 4
    if mode == "mixed":
        assert any(p.high_water == p.num_pages or p.high_water > p.num_pages // 2 for p in runner.cache.pools)


@pytest.mark.parametrize("native", [True, False], ids=["native", "python"])
def test_a_step_that_cannot_run_is_refused_without_side_effects(tmp_path, native):
    """What the step function refuses, with the C++ host runtime and with its Python twin: a request that
    is not live, one that comes twice, no tokens, beyond the longest sequence, a token id outside the
    vocabulary, and more pages than are free -- and in every case nothing has been taken."""
    from tffinfer_b200.engine import StepEntry, OutOfPages, RequestError
    d = make_model_dir(tmp_path, "A")
    ecfg = EngineConfig(dtype="float32", page_size=4, max_cache_tokens=24, max_live_requests=3, device="cpu",
                        max_model_len=20)
    from host_twin import TwinCacheManager
    runner = ModelRunner(d, ecfg, ops=CpuOps(), cache_factory=None if native else TwinCacheManager)
    runner.add_request("a"); runner.add_request("b")
    free = lambda: [p.num_free for p in runner.cache.pools]
    before = free()
    for entries, err, words in [
            ([StepEntry("nobody", [1], [0])], RequestError, "not live"),
            ([StepEntry("a", [1, 2], []), StepEntry("a", [3], [0])], RequestError, "twice"),
            ([StepEntry("a", [], [])], RequestError, "no tokens"),
            ([StepEntry("a", list(range(21)), [0])], RequestError, "maximum length"),
            ([StepEntry("a", [1, 256], [0])], RequestError, "token id outside"),
            ([StepEntry("a", [1, -2], [0])], RequestError, "token id outside"),
            ([StepEntry("a", [1], [0], token_src=[0])], RequestError, "previous step"),
            ([StepEntry("a", list(range(1, 17)), [0]), StepEntry("b", list(range(1, 14)), [0])], OutOfPages, "pages")]:
        with pytest.raises(err, match=words):
            runner.make_batch(entries)
        assert free() == before and runner.num_tokens("a") == 0 and runner.num_tokens("b") == 0
    # what fits still runs afterwards
    logits = runner.step([StepEntry("a", list(range(1, 17)), [15]), StepEntry("b", [5, 6], [1])])
    assert tuple(logits.shape) == (2, 256) and runner.num_tokens("a") == 16 and runner.num_tokens("b") == 2
