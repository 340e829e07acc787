"""The scheduler's decisions on the host (a cache manager, no model), and generation
through the entry point with the kernels' plain twins.  Every test runs with the cache manager
of the C++ host runtime and with its Python twin."""
import pytest

from cpu_ops import CpuOps
from helpers import make_model_dir, PAGE_SIZE
from plain_qwen3 import PlainModel, sample_temperature, sample_greedy
from host_twin import TwinCacheManager
from tffinfer_b200.cache import NativeCacheManager, GroupSpec
from tffinfer_b200.config import EngineConfig
from tffinfer_b200.engine import Scheduler, Request, Engine, ModelRunner
from tffinfer_b200.sampling import SamplingParams, uniform_for


NATIVE = True


@pytest.fixture(autouse=True, params=[True, False], ids=["native", "python"])
def _which_manager(request):
    global NATIVE
    NATIVE = request.param
    yield


def _sched(pages=16, page=4, live=4, budget=8, max_len=64):
    cache = (NativeCacheManager if NATIVE else TwinCacheManager)([GroupSpec(2, 2, 16, 0)], page, [pages], live)
    return Scheduler(cache, budget, max_len), cache


def _req(i, n, new=4):
    return Request(id=f"r{i}", prompt=list(range(1, n + 1)), params=SamplingParams(max_new_tokens=new), key=i)


def _run(s, plan, tok=9):
    return s.update(plan, {e.request.id: tok for e in plan.entries if e.samples})


def test_prompt_is_cut_under_the_budget_and_decodes_go_first():
    s, cache = _sched(budget=8)
    s.add(_req(0, 5)); s.add(_req(1, 11))
    p = s.schedule()
    assert [(e.request.id, e.start, len(e.tokens), e.samples) for e in p.entries] == \
        [("r0", 0, 5, True), ("r1", 0, 3, False)]
    _run(s, p)
    p = s.schedule()          # r0 decodes (1 token) first, r1 gets the other 7
    assert [(e.request.id, e.start, len(e.tokens), e.samples) for e in p.entries] == \
        [("r0", 5, 1, True), ("r1", 3, 7, False)]
    assert p.entries[0].tokens == [9]
    _run(s, p)
    p = s.schedule()
    assert [(e.request.id, e.start, len(e.tokens), e.samples) for e in p.entries] == \
        [("r0", 6, 1, True), ("r1", 10, 1, True)]
    _run(s, p)
    cache.check()


def test_admission_waits_for_a_slot_and_finish_frees_everything():
    s, cache = _sched(live=2, budget=32, pages=32)
    for i in range(3):
        s.add(_req(i, 3, new=2))
    p = s.schedule()
    assert [e.request.id for e in p.entries] == ["r0", "r1"]       # no slot for r2
    _run(s, p)
    p = s.schedule(); outs = _run(s, p)                            # second token: both finish
    assert sorted(o.request_id for o in outs if o.finished) == ["r0", "r1"]
    assert all(o.finish_reason == "length" for o in outs)
    p = s.schedule()
    assert [e.request.id for e in p.entries] == ["r2"]
    _run(s, p); _run(s, s.schedule())
    assert not s.has_work()
    assert cache.pools[0].num_free == 32 and cache.slots.num_free == 2


def test_eos_stops_and_too_long_is_refused():
    s, cache = _sched(max_len=10)
    r = Request(id="a", prompt=[1, 2, 3], params=SamplingParams(max_new_tokens=5, eos_token_ids=(7,)), key=0)
    s.add(r)
    s.add(_req(1, 11))                          # longer than the model allows
    p = s.schedule()
    assert [q.id for q in p.finished] == ["r1"] and p.finished[0].finish_reason == "too_long"
    outs = s.update(p, {"a": 7})
    assert any(o.request_id == "a" and o.finished and o.finish_reason == "stop" for o in outs)
    assert not s.has_work()


def test_when_pages_run_out_the_last_admitted_is_preempted_and_recomputed():
    s, cache = _sched(pages=4, page=4, budget=16)              # 16 tokens of cache in all
    a, b = _req(0, 7, new=6), _req(1, 7, new=6)
    s.add(a); s.add(b)
    p = s.schedule()
    assert [e.request.id for e in p.entries] == ["r0", "r1"]   # 2 pages each: pool is full
    _run(s, p)
    p = s.schedule()                                            # both decode at position 7: still fits
    assert not p.preempted
    _run(s, p)
    p = s.schedule()                                            # position 8 needs a third page each
    assert [q.id for q in p.preempted] == ["r1"]
    assert [e.request.id for e in p.entries] == ["r0"]
    assert b.status == "waiting" and s.waiting[0] is b and b.num_preemptions == 1
    assert len(b.generated) == 2                                # it keeps its tokens
    cache.check()
    _run(s, p)
    # r1 comes back only when r0 has finished and recomputes prompt + generated as one prompt
    seen_b = []
    while s.has_work():
        p = s.schedule()
        seen_b += [(e.start, len(e.tokens)) for e in p.entries if e.request is b]
        _run(s, p)
        cache.check()
    assert seen_b[0] == (0, 9)
    assert len(a.generated) == 6 and len(b.generated) == 6
    assert cache.pools[0].num_free == 4


def test_a_request_that_cannot_fit_alone_ends_with_out_of_memory():
    s, cache = _sched(pages=2, page=4, budget=16)
    s.add(_req(0, 9))                              # 9 tokens > 8 tokens of cache
    p = s.schedule()
    assert p.finished and p.finished[0].finish_reason == "out_of_memory" and not p.entries
    s.update(p, {})
    r = _req(1, 6, new=8)                          # fits at first, outgrows the pool while decoding
    s.add(r)
    reasons = []
    while s.has_work():
        p = s.schedule()
        reasons += [o.finish_reason for o in _run(s, p) if o.finished]
    assert reasons == ["out_of_memory"] and len(r.generated) == 3     # 6 + 2 generated fill the 8 slots
    assert cache.pools[0].num_free == 2 and cache.slots.num_free == 4


# ------------------------------------------------------------------ through the entry point
def _engine(tmp_path, name, **kw):
    d = make_model_dir(tmp_path, name)
    ecfg = EngineConfig(dtype="float32", page_size=PAGE_SIZE[name], device="cpu", **kw)
    return d, Engine(runner=ModelRunner(d, ecfg, ops=CpuOps(), cache_factory=None if NATIVE else TwinCacheManager))


def _plain_generate(pm, prompt, n, params=None, key=0):
    toks = list(prompt)
    out = []
    for i in range(n):
        logits = pm.logits(toks)[-1].float()
        if params is None or params.is_greedy:
            t = sample_greedy(logits)
        else:
            t = sample_temperature(logits, params.temperature, uniform_for(params.seed, key, i),
                                   params.top_k, params.top_p, params.min_p)
        out.append(t); toks.append(t)
    return out


def test_greedy_generation_equals_plain_and_survives_preemption(tmp_path):
    import random
    rng = random.Random(5)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (1, 7, 33)]
    d, eng = _engine(tmp_path, "A", max_cache_tokens=256, max_live_requests=4, max_tokens_per_step=5)
    pm = PlainModel(d)
    want = [_plain_generate(pm, p, 16) for p in prompts]
    got = eng.generate(prompts, max_new_tokens=16)
    assert got == want
    # a pool so small that requests are preempted and recomputed: same tokens
    d, small = _engine(tmp_path, "A", max_cache_tokens=64, max_live_requests=4, max_tokens_per_step=5)
    got = small.generate(prompts, max_new_tokens=16)
    assert got == want
    assert small.scheduler.counters["preemptions"] > 0
    small.runner.cache.check()
    assert small.runner.cache.pools[0].num_free == small.runner.cache.pools[0].num_pages


def test_temperature_sampling_equals_plain_whatever_the_batching(tmp_path):
    import random
    rng = random.Random(6)
    prompts = [[rng.randrange(320) for _ in range(n)] for n in (2, 13, 40)]
    sp = SamplingParams.make(temperature=0.7, seed=42, max_new_tokens=8)
    d, eng = _engine(tmp_path, "B", max_cache_tokens=512, max_live_requests=4, max_tokens_per_step=7)
    pm = PlainModel(d)
    want = [_plain_generate(pm, p, 8, sp, key=i) for i, p in enumerate(prompts)]
    assert eng.generate(prompts, sp) == want
    d, one = _engine(tmp_path, "B", max_cache_tokens=512, max_live_requests=1, max_tokens_per_step=64)
    assert one.generate(prompts, sp) == want
    assert len({tuple(w) for w in want}) == 3


def test_infer_runtime_has_the_reference_call_sequence(tmp_path):
    from tffinfer_b200 import InferRuntime
    d = make_model_dir(tmp_path, "A")
    rt = InferRuntime()
    assert rt.load_model([d], use_f16=False, n_ctx=64, page_size=4, device="cpu", max_cache_tokens=128)
    rt.engine = Engine(runner=ModelRunner(d, rt._ecfg, ops=CpuOps()))     # init_runtime_context without a GPU
    assert rt.encode([[1, 2, 3], [4, 5]]) == 3
    out = []
    rt.infer(4, out)
    assert [len(o) for o in out] == [4, 4]


def test_a_windowed_group_serves_requests_longer_than_its_pool():
    """A group whose mixers keep a window of keys gives the pages behind the window back at every commit, so a
    request needs the window and one step's tokens at a time, not its whole length: 60 tokens run through a
    pool of 32.  The same length is refused when a group that keeps all keys shares the model."""
    page, pages, budget = 4, 8, 8
    Manager = NativeCacheManager if NATIVE else TwinCacheManager
    cache = Manager([GroupSpec(2, 2, 16, 8)], page, [pages], 2)
    s = Scheduler(cache, budget, 128)
    r = _req(1, 60, new=4)
    s.add(r)
    steps, most = 0, 0
    while s.has_work():
        p = s.schedule()
        assert not p.finished, p.finished[0].finish_reason
        most = max(most, pages - cache.pools[0].num_free)
        _run(s, p)
        steps += 1
        assert steps < 100
    assert r.finish_reason == "length" and len(r.generated) == 4
    assert most <= 5                                   # the window's pages and the step's, never the whole length
    assert cache.pools[0].num_free == pages
    cache.check()
    both = Manager([GroupSpec(2, 2, 16, 8), GroupSpec(1, 2, 16, 0)], page, [pages, pages], 2)
    s = Scheduler(both, budget, 128)
    s.add(_req(2, 60))
    p = s.schedule()
    assert p.finished and p.finished[0].finish_reason == "out_of_memory" and not p.entries
