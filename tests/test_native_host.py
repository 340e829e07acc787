"""The C++ host runtime (page pools, block tables, state slots, step packing) against its Python twins:
the same random orders of requests through both, every answer compared, the packed arrays of every step
compared element by element."""
import random

import numpy as np
import pytest

from host_twin import TwinCacheManager as CacheManager, pack_step
from tffinfer_b200.cache import NativeCacheManager, GroupSpec
from tffinfer_b200.engine.batch import StepEntry


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_native_manager_and_packer_equal_the_python_twins(seed):
    rng = random.Random(seed)
    groups = [GroupSpec(2, 2, 16, 0), GroupSpec(1, 2, 16, rng.choice([5, 9, 30]))]
    page = rng.choice([2, 4, 16])
    sizes = [rng.randint(20, 60), rng.randint(8, 20)]
    a = CacheManager(groups, page, sizes, 5)
    b = NativeCacheManager(groups, page, sizes, 5)
    live, packed = [], 0
    for step in range(1500):
        op = rng.random()
        if op < 0.2:
            r = f"r{step}"
            sa, sb = a.admit(r), b.admit(r)
            assert sa == sb
            if sa is not None:
                live.append(r)
        elif op < 0.75 and live:
            r, n = rng.choice(live), rng.randint(1, 9)
            assert a.pages_needed(r, n) == b.pages_needed(r, n)
            ra, rb = a.reserve(r, n), b.reserve(r, n)
            assert ra == rb
            if ra:
                k = rng.randint(0, n)
                a.commit(r, k); b.commit(r, k)
        elif live:
            r = live.pop(rng.randrange(len(live)))
            a.release(r); b.release(r)
        for r in live:
            assert a.num_tokens(r) == b.num_tokens(r) and a.slot_of(r) == b.slot_of(r)
            for g in range(2):
                assert a.block_table(r, g) == b.block_table(r, g)        # the same pages in the same order
        assert a.stats() == b.stats()
        if step % 25 == 0:
            a.check(); b.check()
        if live and step % 5 == 0:
            ents = []
            for r in rng.sample(live, rng.randint(1, len(live))):
                n = rng.randint(1, 5)
                if not a.reserve(r, n):
                    assert not b.reserve(r, n)
                    continue
                assert b.reserve(r, n)
                src = [rng.choice([-1, 0, 2]) for _ in range(n)] if rng.random() < 0.3 else None
                ents.append(StepEntry(r, [rng.randrange(100) for _ in range(n)],
                                      sorted(rng.sample(range(n), rng.randint(0, n))), token_src=src))
            if not ents:
                continue
            pad = rng.choice([0, 0, len(ents) + 2])
            kw = dict(pad_requests=pad, dummy_pages=[sizes[0] - 1, sizes[1] - 1], dummy_slot=4) if pad else {}
            if rng.random() < 0.5:
                kw["widths"] = (40, 40)
            arr, lay, info = pack_step(ents, [a.num_tokens(e.req) for e in ents], [a.slot_of(e.req) for e in ents],
                                       [[a.block_table(e.req, g) for e in ents] for g in range(2)], **kw)
            buf = np.full(lay.total, -7, dtype=np.int32) if rng.random() < 0.5 else None   # a caller's buffer, or its own
            arr2, lay2, info2 = b.pack_step(ents, out=buf, **kw)
            assert lay == lay2 and np.array_equal(arr, arr2)
            assert set(info) == set(info2)
            for key, v in info.items():
                assert np.array_equal(v, info2[key]) if isinstance(v, np.ndarray) else v == info2[key], key
            for e in ents:
                a.commit(e.req, len(e.tokens)); b.commit(e.req, len(e.tokens))
            packed += 1
    assert packed > 50
    for r in live:
        a.release(r); b.release(r)
    a.check(); b.check()
    assert a.stats() == b.stats() and b.pools[0].num_free == sizes[0]


def test_native_packer_refuses_what_the_python_one_refuses():
    m = NativeCacheManager([GroupSpec(1, 1, 16, 0)], 4, [8], 2)
    m.admit("a")
    assert m.reserve("a", 6)
    with pytest.raises(ValueError, match="wanted place"):
        m.pack_step([StepEntry("a", [1, 2, 3], [3])])
    with pytest.raises(ValueError, match="wider"):
        m.pack_step([StepEntry("a", [1, 2, 3], [0])], widths=(1,))
    with pytest.raises(ValueError):
        m.pack_step([StepEntry("a", [], [])])
    with pytest.raises(KeyError):
        m.pack_step([StepEntry("nobody", [1], [0])])
    with pytest.raises(ValueError):
        m.pack_step([StepEntry("a", [1, 2], [1])], out=np.zeros(5, dtype=np.int32))
    arr, layout, info = m.pack_step([StepEntry("a", [1, 2], [1])])
    assert layout.T == 2 and layout.B == 1 and info["real_logit_rows"] == 1 and not info["all_decode"]


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_native_planning_equals_the_python_scheduler_in_lockstep(seed):
    """Two schedulers over two cache managers, one deciding in C++ and one in Python, fed the same requests
    and the same drawn tokens: every plan (who runs, from where, how many tokens, who is preempted, who ends
    and why) and the caches' accounts are the same step after step, through preemptions and refusals."""
    from tffinfer_b200.engine import Scheduler, Request
    from tffinfer_b200.sampling import SamplingParams
    rng = random.Random(50 + seed)
    page = rng.choice([2, 4, 8])
    pages = rng.randint(6, 24)
    live = rng.randint(1, 4)
    budget = rng.choice([3, 8, 20])
    max_len = rng.choice([40, 200])
    groups = [GroupSpec(2, 2, 16, 0)] + ([GroupSpec(1, 2, 16, 7)] if seed % 2 else [])
    sizes = [pages] + ([max(3, pages // 2)] if seed % 2 else [])
    sa = Scheduler(CacheManager(groups, page, sizes, live), budget, max_len)
    sb = Scheduler(NativeCacheManager(groups, page, sizes, live), budget, max_len)

    def both(i, n, new):
        for s in (sa, sb):
            s.add(Request(id=f"r{i}", prompt=list(range(1, n + 1)), params=SamplingParams(max_new_tokens=new), key=i))

    added = preempted = refused = 0
    for step in range(400):
        if rng.random() < 0.3:
            n = rng.choice([0, 1, 3, 9, 17, 30, 60, 150]) if rng.random() < 0.2 else rng.randint(1, 25)
            both(added, n, rng.randint(1, 6))
            added += 1
        pa, pb = sa.schedule(), sb.schedule()
        assert [(e.request.id, e.start, e.tokens, e.samples) for e in pa.entries] == \
               [(e.request.id, e.start, e.tokens, e.samples) for e in pb.entries], step
        assert [r.id for r in pa.preempted] == [r.id for r in pb.preempted]
        assert [(r.id, r.finish_reason) for r in pa.finished] == [(r.id, r.finish_reason) for r in pb.finished]
        assert [r.id for r in sa.running] == [r.id for r in sb.running]
        assert [r.id for r in sa.waiting] == [r.id for r in sb.waiting]
        preempted += len(pb.preempted)
        refused += len(pb.finished)
        drawn = {e.request.id: rng.randrange(50) for e in pa.entries if e.samples}
        oa, ob = sa.update(pa, drawn), sb.update(pb, drawn)
        assert [(o.request_id, o.token, o.finished, o.finish_reason) for o in oa] == \
               [(o.request_id, o.token, o.finished, o.finish_reason) for o in ob]
        assert sa.cache.stats() == sb.cache.stats()
        for r in sb.running:
            for g in range(len(groups)):
                assert sa.cache.block_table(r.id, g) == sb.cache.block_table(r.id, g)
        if step % 20 == 0:
            sa.cache.check(); sb.cache.check()
    assert added > 50 and sa.counters == sb.counters
    assert preempted + refused > 0
