"""The allocation-free attention entry point (tffinfer_b200/csrc/no_alloc_api.h).

Some users of the kernel library cannot allocate device memory when they call it: a host
that gave all memory to its own pool, a serving loop that must not pay the device-wide
synchronisation of cudaMalloc, a C program without PyTorch's allocator.  For them the
library keeps the split-key scratch in a fixed __device__ array.  This test calls that
entry point through its exported C symbol, twice in a row on the shared array with
different inputs, and checks each result against the ordinary entry point, which gets
its scratch from the caller, and against the plain attention of tests/cpu_ops.py (the two
entry points run the same kernel, so agreeing with each other would not be enough).  That
nothing is allocated is checked on the driver's own count of free device memory, which
sees a cudaMalloc from any library, not on PyTorch's allocator statistics.  It also checks
that a call too large for the array is refused, and that the size of a call is worked out
in 64 bits.  The file is named so that pytest collects it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

NQ, NKV, D, PAGE = 32, 8, 128, 16


def _case(seed, lens, splits, dev):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    blocks = [-(-(n + 1) // PAGE) for n in lens]
    n_pages = sum(blocks) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(blocks)
    table = torch.full((B, width), -1, dtype=torch.int32)
    k = 0
    for i, nb in enumerate(blocks):
        table[i, :nb] = torch.tensor(perm[k:k + nb], dtype=torch.int32)
        k += nb
    cache = torch.randn((n_pages, 1, 2, NKV, PAGE, D), generator=g).to(torch.bfloat16)
    q = torch.randn((B, NQ * D), generator=g).to(torch.bfloat16)
    q_start = torch.arange(B + 1, dtype=torch.int32)
    pos_start = torch.tensor(lens, dtype=torch.int32)          # one new token at position len
    return dict(q=q.to(dev), q_start=q_start.to(dev), pos_start=pos_start.to(dev), table=table.to(dev),
                cache=cache.to(dev), B=B, width=width, splits=splits)


def _call(lib, fn_name, c, out, workspace=None):
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    stream = vp(torch.cuda.current_stream().cuda_stream)
    head = [vp(c["q"].data_ptr()), vp(c["q_start"].data_ptr()), vp(c["pos_start"].data_ptr()),
            vp(c["table"].data_ptr()), ci(c["width"]), vp(c["cache"].data_ptr()), ci(1), ci(0), ci(PAGE),
            vp(out.data_ptr())]
    tail = [ci(c["B"]), ci(c["B"]), ci(1), ci(c["splits"]), ci(NQ), ci(NKV), ci(D), cf(1 / math.sqrt(D)), ci(0), stream]
    if workspace is not None:
        head.append(vp(workspace.data_ptr()))
    return getattr(lib, fn_name)(*(head + tail))


def _plain_attention(c):
    """The same attention by the plain twin of the kernels (float64 on the CPU)."""
    from types import SimpleNamespace
    from cpu_ops import CpuOps
    B = c["B"]
    batch = SimpleNamespace(positions=c["pos_start"].cpu(), tok_req=torch.arange(B, dtype=torch.int32))
    out = torch.empty((B, NQ * D), dtype=torch.float32)
    CpuOps().attention(c["q"].cpu().float(), batch, c["table"].cpu(), c["cache"].cpu().float(), 0, PAGE, out,
                       NQ, NKV, D, 1 / math.sqrt(D), 0)
    return out


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from tffinfer_b200.csrc import build
    lib = ctypes.CDLL(build.library_path(build=True, verbose=False))
    dev = "cuda"
    lib.tff_attention_bf16_workspace.restype = ctypes.c_longlong
    # two different calls, back to back, on the one shared scratch array
    cases = [_case(1, [300, 17, 2049, 64], 4, dev), _case(2, [5, 1000, 63], 7, dev)]
    # one call first that is not measured: the first use of a kernel makes the driver load its code
    warm = torch.empty((cases[0]["B"], NQ * D), dtype=torch.bfloat16, device=dev)
    assert _call(lib, "tff_attention_bf16_noalloc", cases[0], warm) == 0
    torch.cuda.synchronize()
    for c in cases:
        need = lib.tff_attention_bf16_workspace(ctypes.c_int(c["B"] * NQ), ctypes.c_int(c["splits"]), ctypes.c_int(D))
        ws = torch.empty(need // 4, dtype=torch.float32, device=dev)
        want = torch.full((c["B"], NQ * D), float("nan"), dtype=torch.bfloat16, device=dev)
        assert _call(lib, "tff_attention_bf16", c, want, ws) == 0
        got = torch.full((c["B"], NQ * D), float("nan"), dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        assert _call(lib, "tff_attention_bf16_noalloc", c, got) == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, f"the call changed the free device memory by {free_before - free_after} bytes"
        assert torch.isfinite(got).all()
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err < 1e-2, err          # the tolerance of the other bfloat16 attention tests
        plain = _plain_attention(c)
        err = float((got.float().cpu() - plain).abs().max() / plain.abs().max())
        assert err < 1e-2, err
    # a call that needs more scratch than the library holds is refused and launches nothing
    big = dict(cases[0])
    big["splits"] = 16
    rows_needed = 8 * 1024 * 1024 // (16 * (D + 2) * 4) + 1
    B = -(-rows_needed // NQ)
    big.update(B=B, q=torch.zeros((B, NQ * D), dtype=torch.bfloat16, device=dev),
               q_start=torch.arange(B + 1, dtype=torch.int32, device=dev),
               pos_start=torch.zeros(B, dtype=torch.int32, device=dev),
               table=torch.zeros((B, 1), dtype=torch.int32, device=dev), width=1)
    out = torch.zeros((B, NQ * D), dtype=torch.bfloat16, device=dev)
    assert _call(lib, "tff_attention_bf16_noalloc", big, out) == -6
    torch.cuda.synchronize()
    # arguments that are wrong are refused before the size is looked at, and launch nothing
    bad = dict(cases[1])
    bad["width"] = 0
    assert _call(lib, "tff_attention_bf16_noalloc", bad, torch.zeros_like(warm)) == -1


def test_the_size_of_a_call_is_worked_out_in_64_bits():
    """tokens * nq of a large batch is beyond an int: 2**27 tokens of 32 heads multiply to 2**32, which a
    32-bit product turns into 0 -- a call that 'needs nothing' and would then write far outside the array.
    The size function is pure host arithmetic, so asking it launches nothing."""
    from tffinfer_b200.csrc import build
    lib = ctypes.CDLL(build.library_path(build=True, verbose=False))
    f = lib.tff_attention_bf16_noalloc_bytes
    f.restype = ctypes.c_longlong
    f.argtypes = [ctypes.c_longlong] * 4
    limit = 8 * 1024 * 1024
    assert f(4, NQ, 4, D) == 4 * NQ * 4 * (D + 2) * 4 <= limit
    assert f(4, NQ, 1, D) == 0
    assert f(2 ** 27, 32, 2, D) == 2 ** 27 * 32 * 2 * (D + 2) * 4 > limit
    assert f(2 ** 31 - 1, 2 ** 20, 16, 512) == -1            # beyond 62 bits: refused, not wrapped
    assert f(0, NQ, 2, D) == f(4, 0, 2, D) == f(4, NQ, 0, D) == f(4, NQ, 2, 0) == f(-4, NQ, 2, D) == -1
