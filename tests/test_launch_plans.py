"""Launch decisions taken on the host: how the tensor-core product cuts the tiles of a last, partial wave,
and how the decode attention shares out the key range."""
from tffinfer_b200.kernels.library import CudaKernels


def cost(tail, s, ctas):
    return -(-tail * s // ctas) / s


def test_full_waves_are_left_alone():
    assert CudaKernels.tail_slices(148, 64, 148) == 0
    assert CudaKernels.tail_slices(296, 64, 148) == 0


def test_slices_shorten_the_last_wave_and_never_lengthen_it():
    for tiles in range(1, 700):
        s = CudaKernels.tail_slices(tiles, 64, 148)
        tail = tiles % 148
        if tail == 0:
            assert s == 0
            continue
        assert s == 0 or 2 <= s <= 8
        if s:
            assert cost(tail, s, 148) < 1.0
    # 256 tiles on 148 CTAs (a 2048 x 4096 output in 128 x 256 tiles): 108 left over, four slices make
    # three rounds of a quarter tile
    assert CudaKernels.tail_slices(256, 64, 148) == 4
    # few K blocks bound the number of slices
    assert CudaKernels.tail_slices(20, 2, 148) in (0, 2)


def test_key_split_follows_the_effective_number_of_requests():
    """sum / longest of the contexts decides the split of the key range, rounded to powers of two
    (the classes that decode graphs are captured for)."""
    from tffinfer_b200.kernels.library import CudaKernels, effective_requests
    assert effective_requests([2048] * 8) == 8.0
    assert effective_requests([]) == 1.0
    assert abs(effective_requests([4000, 10, 10, 10]) - 1.0075) < 1e-9
    from types import SimpleNamespace
    planner = SimpleNamespace(NUM_SMS=148)         # the planner reads the SM count from the device; a B200 has 148
    splits = lambda n: CudaKernels.attention_splits(planner, n, 1, 32, 8)
    assert [splits(n) for n in (1, 2, 4, 8, 16, 24, 32, 64)] == [16, 16, 9, 4, 2, 1, 1, 1]
    # 26 requests, one of them long: cut as 4 equal ones would be, not as 32
    assert splits(effective_requests([4000] + [500] * 25)) == splits(4.2) == splits(4) == 9
    assert splits(20) == splits(16) and splits(23) == splits(32)
    assert CudaKernels.key_split_class([600, 37, 580, 5, 610, 90]) == 4 and CudaKernels.key_split_class([9] * 24) == 32
    # many tokens a request (portions): never cut
    assert CudaKernels.attention_splits(planner, 1, 64, 32, 8) == 1
    # on a part with fewer SMs the same batch is cut into fewer shares
    assert CudaKernels.attention_splits(SimpleNamespace(NUM_SMS=74), 4, 1, 32, 8) == 4


def test_prompt_sized_products_take_the_configuration_with_the_fewest_waves():
    """Above the row count of the swapped orientation the product is planned by what its waves of tiles cost in
    each configuration (256 x 256 on pairs of SMs, 128 x 256, 128 x 128)."""
    p = CudaKernels.__new__(CudaKernels)               # the planner alone: no library is loaded
    p.NUM_SMS, p.USE_SM_PAIRS = 148, True
    plan = p.prompt_plan
    # 2048 rows of the 8B shape: pairs of SMs throughout; the added products cut their last wave in four
    assert plan(2048, 6144, 4096, False) == (0, 512, 0)
    assert plan(2048, 4096, 4096, True) == (0, 512, 4)
    assert plan(2048, 24576, 4096, False)[1] == 512
    # 544 rows of the 14B shape's q/k/v: 84 pair tiles are two waves on 74 pairs, 140 single tiles one wave on 148 SMs
    assert plan(544, 7168, 5120, False) == (0, 256, 0)
    # few rows and a narrow output: the small tile, whose wave is the cheapest
    assert plan(300, 6144, 4096, False) == (0, 128, 0)
    # a product that is stored is never cut along K; one that is added may be
    for M in (257, 300, 544, 1000, 4096):
        for N, K in ((6144, 4096), (4096, 12288), (34816, 5120)):
            assert plan(M, N, K, False)[2] == 0
            assert plan(M, N, K, True)[2] in (0, 2, 3, 4, 5, 6, 7, 8)
    # without pairs of SMs, or asked for one configuration, it plans within what it is given
    q = CudaKernels.__new__(CudaKernels)
    q.NUM_SMS, q.USE_SM_PAIRS = 148, False
    assert q.prompt_plan(2048, 6144, 4096, False)[1] in (256, 128)
    assert plan(2048, 6144, 4096, False, kinds=(256,)) == (0, 256, 0)
    # a narrow output has no pair tile
    assert plan(2048, 128, 4096, False)[1] in (256, 128)


def test_small_portions_behind_long_contexts_take_key_shares():
    """A portion of up to 256 packed rows (tokens times query heads a key/value head) behind 2,048 or more keys
    is cut along its keys so that every SM gets two CTAs of 64-row tiles; larger portions, short contexts
    and single decoded tokens are not its business."""
    from types import SimpleNamespace
    planner = SimpleNamespace(NUM_SMS=148)
    ps = lambda *a: CudaKernels.portion_splits(planner, *a)
    # one request: tokens, longest context, 32/8 heads
    assert ps(1, 16, 4016, 32, 8) == 16          # 64 rows: one tile a head, 8 CTAs a share
    assert ps(1, 32, 4032, 32, 8) == 16          # 128 rows: 16 CTAs a share
    assert ps(1, 64, 4064, 32, 8) == 8           # 256 rows: 32 CTAs a share
    assert ps(1, 65, 4065, 32, 8) == 1           # beyond 256 rows: the tensor-core tiles
    assert ps(1, 50, 2050, 40, 8) == 8           # 5 heads a group: 250 rows
    assert ps(1, 16, 300, 32, 8) == 1            # a short context is walked quickly
    assert ps(1, 16, 1500, 32, 8) == 1           # ... and so is one of 1,500 keys (measured: no gain below 2,048)
    assert ps(1, 4, 4004, 32, 8) == 1            # 16 rows: the decode kernel, which cuts its keys itself
    assert ps(4, 16, 4016, 32, 8) == 8           # several such portions in a step share the SMs (32 CTAs a share)
    assert CudaKernels.portion_splits(SimpleNamespace(NUM_SMS=74), 1, 64, 4064, 32, 8) == 4

