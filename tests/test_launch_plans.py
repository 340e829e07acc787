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
