"""How the tensor-core product cuts the tiles of a last, partial wave (host-side decision)."""
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
