"""The C++ host runtime (page pools, block tables, state slots, step packing) against its Python twins:
the same random orders of requests through both, every answer compared, the packed arrays of every step
compared element by element."""
import random

import numpy as np
import pytest

from tffinfer_b200.cache import CacheManager, NativeCacheManager, GroupSpec
from tffinfer_b200.engine.batch import StepEntry, pack_step


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
