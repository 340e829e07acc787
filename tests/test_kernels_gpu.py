"""Each kernel alone against its plain twin (tests/cpu_ops.py), at sizes other than the
engine's: odd widths, vocabularies that are no power of two, head sizes in steps of 16,
any number of heads and groups, single rows, page edges."""
import math
import random

import numpy as np
import pytest
import torch

from cpu_ops import CpuOps
from tffinfer_b200.engine.batch import StepEntry
from host_twin import build_step_batch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from tffinfer_b200.kernels.library import CudaKernels
    k = CudaKernels()
    yield k
    k.check_errors()


def rel_err(got, want):
    want = want.double().cpu(); got = got.double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def g(shape, dtype, seed, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen) * scale).to(dtype)


@pytest.mark.parametrize("T,H,V", [(1, 64, 100), (5, 96, 311), (33, 4096, 1000)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_embed(ops, T, H, V, dt):
    table = g((V, H), dt, 1)
    tok = torch.randint(0, V, (T,), dtype=torch.int32)
    want = torch.empty(T, H); CpuOps().embed(tok, table, want)
    out = torch.empty(T, H, device=DEV)
    ops.embed(tok.to(DEV), table.to(DEV), out)
    assert torch.equal(out.cpu(), want)


def test_embed_with_a_scale_and_with_a_token_outside_the_table(ops):
    table = g((50, 96), torch.bfloat16, 1)
    tok = torch.tensor([3, 49, 0], dtype=torch.int32)
    want = torch.empty(3, 96); CpuOps().embed(tok, table, want, 96 ** 0.5)
    out = torch.empty(3, 96, device=DEV)
    ops.embed(tok.to(DEV), table.to(DEV), out, 96 ** 0.5)
    assert rel_err(out, want) < 1e-6
    bad = torch.tensor([3, 50, -1], dtype=torch.int32)          # never another token's row: poison instead
    ops.embed(bad.to(DEV), table.to(DEV), out)
    assert torch.isfinite(out[0]).all() and torch.isnan(out[1]).all() and torch.isnan(out[2]).all()


@pytest.mark.parametrize("R,V,scale,cap", [(1, 100, 0.5, 5.0), (7, 311, 1.0, 30.0), (3, 151936, 0.125, 0.0), (64, 4097, 2.0, 1.5)])
def test_logit_transform(ops, R, V, scale, cap):
    logits = g((R, V), torch.float32, 5, 20.0)
    want = logits.clone(); CpuOps().logit_transform(want, scale, cap)
    out = logits.clone().to(DEV)
    ops.logit_transform(out, scale, cap)
    assert rel_err(out, want) < 2e-6
    if cap > 0:
        assert float(out.abs().max()) <= cap


@pytest.mark.parametrize("shape,dt", [((7,), torch.float32), ((3, 5), torch.bfloat16), ((4096,), torch.float32),
                                      ((33,), torch.int32), ((1,), torch.bfloat16)])
def test_reset_state_slots_clears_exactly_the_slots_of_requests_at_position_zero(ops, shape, dt):
    slots_total = 6
    if dt == torch.int32:
        state = torch.arange(1, slots_total * 33 + 1, dtype=dt).view(slots_total, 33).to(DEV)
    else:
        state = (g((slots_total,) + shape, torch.float32, 6) + 3).to(dt).to(DEV)
    before = state.clone()
    slots = torch.tensor([4, 0, 2, 5], dtype=torch.int32)
    pos = torch.tensor([0, 17, 0, 1], dtype=torch.int32)
    want = before.cpu().clone(); CpuOps().reset_state_slots(want, slots, pos)
    ops.reset_state_slots(state, slots.to(DEV), pos.to(DEV))
    assert torch.equal(state.cpu(), want)
    assert float(state[4].float().abs().max()) == 0 and float(state[2].float().abs().max()) == 0
    assert torch.equal(state[[0, 1, 3, 5]].cpu(), before[[0, 1, 3, 5]].cpu())


@pytest.mark.parametrize("rows,dim", [(1, 48), (7, 80), (3, 4096), (2, 5120), (9, 1000)])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_rmsnorm_with_and_without_row_index(ops, rows, dim, odt):
    x = g((rows + 3, dim), torch.float32, 2, 3.0)
    w = 1 + 0.1 * g((dim,), torch.float32, 3)
    for idx in (None, torch.tensor([rows + 2] + list(range(rows - 1)), dtype=torch.int32)):
        n = rows + 3 if idx is None else rows
        want = torch.empty(n, dim, dtype=odt); CpuOps().rmsnorm(x, w, 1e-5, want, idx)
        out = torch.empty(n, dim, dtype=odt, device=DEV)
        ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out, None if idx is None else idx.to(DEV))
        assert rel_err(out, want) < (1e-6 if odt == torch.float32 else 8e-3)


@pytest.mark.parametrize("T,I", [(1, 16), (5, 112), (64, 12288), (3, 1001)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_swiglu(ops, T, I, dt):
    gu = g((T, 2 * I), dt, 4, 2.0)
    want = torch.empty(T, I, dtype=dt); CpuOps().swiglu(gu, want)
    out = torch.empty(T, I, dtype=dt, device=DEV)
    ops.swiglu(gu.to(DEV), out)
    assert rel_err(out, want) < (1e-6 if dt == torch.float32 else 8e-3)
    if dt == torch.bfloat16:                      # float32 accumulators in, bfloat16 out
        gu32 = g((T, 2 * I), torch.float32, 4, 2.0)
        CpuOps().swiglu(gu32, want)
        ops.swiglu(gu32.to(DEV), out)
        assert rel_err(out, want) < 8e-3
    if I % 16 == 0:                               # gate and up alternating in blocks
        CpuOps().swiglu(gu, want, 16)
        ops.swiglu(gu.to(DEV), out, 16)
        assert rel_err(out, want) < (1e-6 if dt == torch.float32 else 8e-3)


@pytest.mark.parametrize("T,I,K", [(1, 64, 64), (8, 12288, 4096), (300, 192, 264), (700, 1024, 520), (2048, 12288, 256),
                                   (257, 112, 80), (40, 160, 96)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_gemm_swiglu_merged_weights(ops, T, I, K, dt):
    """Every path of gemm_swiglu (fused tensor-core epilogue, split product + kernel, float32) from the
    library's own merged layout."""
    a = g((T, K), dt, 40)
    wg, wu = g((I, K), dt, 41, 0.06), g((I, K), dt, 42, 0.06)
    gate, up = a.double() @ wg.double().t(), a.double() @ wu.double().t()
    want = (gate / (1 + torch.exp(-gate))) * up
    merged = ops.merge_gate_up(wg.to(DEV), wu.to(DEV))
    assert merged.shape == (2 * I, K)
    out = torch.full((T, I), float("nan"), dtype=dt, device=DEV)
    ops.gemm_swiglu(a.to(DEV), merged, out)
    err = float((out.double().cpu() - want).abs().max() / want.abs().max())
    assert err < (1e-5 if dt == torch.float32 else 1.2e-2), err
    ops.check_errors()


@pytest.mark.parametrize("theta,rot,maxpos", [(1e4, 16, 128), (1e6, 128, 4096), (5e5, 48, 700)])
def test_rope_table(ops, theta, rot, maxpos):
    want = torch.empty(maxpos, rot // 2, 2); CpuOps().rope_table(want, theta, rot)
    out = torch.empty(maxpos, rot // 2, 2, device=DEV)
    ops.rope_table(out, theta, rot)
    assert float((out.cpu() - want).abs().max()) < 2e-6


SIMT_SHAPES = [(1, 64, 64), (7, 311, 80), (65, 130, 96), (3, 1000, 264), (130, 64, 17)]


@pytest.mark.parametrize("M,N,K", SIMT_SHAPES)
@pytest.mark.parametrize("adt,wdt,odt", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                         (torch.bfloat16, torch.float32, torch.bfloat16),
                                         (torch.bfloat16, torch.bfloat16, torch.float32)])
def test_gemm_simt(ops, M, N, K, adt, wdt, odt):
    a, w = g((M, K), adt, 5), g((N, K), wdt, 6, 0.05)
    for use_res in (False, True):
        if use_res and odt != torch.float32:
            continue
        res = g((M, N), torch.float32, 7) if use_res else None
        want = torch.empty(M, N, dtype=odt); CpuOps().gemm(a, w, want, res)
        out = res.clone().to(DEV) if use_res else torch.empty(M, N, dtype=odt, device=DEV)
        ops.gemm_simt(a.to(DEV), w.to(DEV), out, out if use_res else None)
        assert rel_err(out, want) < (2e-6 if odt == torch.float32 else 8e-3), (M, N, K, use_res)


def test_gemm_simt_rows_do_not_depend_on_the_batch(ops):
    a, w = g((70, 96), torch.float32, 8).to(DEV), g((130, 96), torch.float32, 9).to(DEV)
    full = torch.empty(70, 130, device=DEV); ops.gemm_simt(a, w, full)
    one = torch.empty(1, 130, device=DEV); ops.gemm_simt(a[37:38].contiguous(), w, one)
    assert torch.equal(full[37:38], one)


TC_SHAPES = [(1, 128, 64), (8, 6144, 4096), (5, 311, 80), (16, 256, 128), (17, 384, 200), (64, 4096, 1024),
             (100, 1000, 512), (256, 512, 4096), (257, 512, 256), (300, 311, 264), (1024, 768, 512),
             (2048, 4096, 4096), (128, 128, 8), (130, 6144, 4096), (300, 1000, 264), (513, 1256, 72)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tc_all_epilogues(ops, M, N, K):
    a, w = g((M, K), torch.bfloat16, 10), g((N, K), torch.bfloat16, 11, 0.05)
    ad, wd = a.to(DEV), w.to(DEV)
    ref = a.double() @ w.double().t()
    scale = float(ref.abs().max())
    for odt in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), dtype=odt, device=DEV)
        ops.gemm_tc(ad, wd, out)
        err = float((out.double().cpu() - ref).abs().max()) / scale
        assert err < (1e-5 if odt == torch.float32 else 8e-3), (M, N, K, odt, err)
    res = g((M, N), torch.float32, 12)
    out = res.clone().to(DEV)
    ops.gemm_tc(ad, wd, out, out)
    err = float((out.double().cpu() - (res.double() + ref)).abs().max()) / scale
    assert err < 1e-5, (M, N, K, "residual", err)
    ops.check_errors()


@pytest.mark.parametrize("M,N,K,swap,bn,splits", [(8, 512, 4096, 1, 16, 1), (8, 512, 4096, 1, 16, 0),
                                                  (40, 1000, 1000 // 8 * 8, 1, 64, 1), (64, 4096, 12288, 1, 64, 1),
                                                  (200, 300, 512, 1, 256, 1), (200, 300, 512, 0, 128, 0),
                                                  (200, 300, 512, 0, 256, 0), (16, 128, 64, 1, 32, 0),
                                                  (1, 24576, 4096, 1, 16, 1), (3, 40000, 256, 1, 16, 1),
                                                  (700, 1030, 520, 0, 128, 0), (700, 1030, 520, 0, 256, 0),
                                                  (130, 24576, 128, 0, 256, 0), (128, 64, 4096, 1, 128, 1),
                                                  (700, 1030, 520, 0, 256, 3), (2500, 2304, 264, 0, 256, 5),
                                                  (2500, 2304, 264, 0, 256, 8), (300, 311, 264, 0, 128, 8),
                                                  (2048, 4096, 1024, 0, 256, 4), (512, 4096, 4096, 0, 256, 2),
                                                  # bn = 512: 256 x 256 tiles on pairs of SMs (cta_group::2); 311 columns
                                                  # of float32 do not suit TMA: single CTAs take over
                                                  (700, 1030, 520, 0, 512, 0), (700, 1030, 520, 0, 512, 3),
                                                  (2500, 2304, 264, 0, 512, 5), (300, 311, 264, 0, 512, 2),
                                                  (2048, 4096, 1024, 0, 512, 4), (257, 512, 4096, 0, 512, 0),
                                                  (129, 256, 64, 0, 512, 0), (4096, 512, 128, 0, 512, 8)])
def test_gemm_tc_explicit_plans(ops, M, N, K, swap, bn, splits):
    """splits: 0 = whole tiles; 1 = stream-K shares with float32 adds; S >= 2 = the tiles of the last wave
    in S slices of their K range (more slices than K blocks leaves some empty)"""
    a, w = g((M, K), torch.bfloat16, 13), g((N, K), torch.bfloat16, 14, 0.05)
    ref = a.double() @ w.double().t()
    res = g((M, N), torch.float32, 15)
    out = res.clone().to(DEV)
    ops.gemm_tc(a.to(DEV), w.to(DEV), out, out, plan=(swap, bn, splits))
    err = float((out.double().cpu() - (res.double() + ref)).abs().max()) / float(ref.abs().max())
    assert err < 1e-5, err
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_tc(a.to(DEV), w.to(DEV), out, None, plan=(swap, bn, splits))
    err = float((out.double().cpu() - ref).abs().max()) / float(ref.abs().max())
    assert err < 1e-5, err
    ops.check_errors()


@pytest.mark.parametrize("M,H,I", [(1, 4096, 12288), (8, 4096, 12288), (16, 520, 192), (7, 264, 64), (4, 5120, 17408),
                                   (3, 64, 128)])
def test_norm_gate_up_product_and_swiglu_as_one_kernel(ops, M, H, I):
    """act = silu(gate) * up of RMSNorm(x) W^T for a decode step of at most 16 tokens: one kernel in which the
    CTAs of a cluster share a tile's K range and meet in the first one's shared memory; against the plain twins
    of the norm, the product and the SwiGLU kernel.  Then the whole feed-forward in two launches."""
    cpu = CpuOps()
    from tffinfer_b200.kernels.library import DeferredNorm
    x = g((M, H), torch.float32, 153, 2.0)
    nw = 1 + 0.1 * g((H,), torch.float32, 154)
    wg, wu = g((I, H), torch.bfloat16, 155, 0.05), g((I, H), torch.bfloat16, 156, 0.05)
    wd = g((H, I), torch.bfloat16, 151, 0.05)
    h = torch.empty(M, H, dtype=torch.bfloat16); cpu.rmsnorm(x, nw, 1e-5, h)
    want = x.clone(); cpu.gated_mlp(h, cpu.merge_gate_up(wg, wu), wd, want, I)
    xd = x.clone().to(DEV)
    assert ops.can_fold_norm(xd, nw.to(DEV), torch.bfloat16)
    launches = ops.launches
    ops.gated_mlp(DeferredNorm(xd, nw.to(DEV), 1e-5, torch.bfloat16, ops), ops.merge_gate_up(wg.to(DEV), wu.to(DEV)),
                  wd.to(DEV), xd, I)
    assert ops.launches == launches + 2
    ops.check_errors()
    # x * w is rounded to bfloat16 where the separate kernel rounds (x * r) * w: a bfloat16 rounding apart
    assert rel_err(xd - x.to(DEV), want - x) < 2e-2


def _paged_case(nq, nkv, d, page, lens_new, lens_old, window, dt, seed, layers=2, layer=1, rot=None):
    """Builds a batch of requests with ``lens_old`` tokens already cached and ``lens_new`` new ones,
    scattered pages, and returns everything both implementations need."""
    rng = random.Random(seed)
    B = len(lens_new)
    total = [o + n for o, n in zip(lens_old, lens_new)]
    blocks = [-(-t // page) for t in total]
    n_pages = sum(blocks) + 5
    ids = list(range(n_pages)); rng.shuffle(ids)
    tables, k = [], 0
    for b in blocks:
        tables.append(ids[k:k + b]); k += b
    entries = [StepEntry(i, [0] * n, []) for i, n in enumerate(lens_new)]
    cache = g((n_pages, layers, 2, nkv, page, d), dt, seed + 1)
    T = sum(lens_new)
    qkv = g((T, (nq + 2 * nkv) * d), dt, seed + 2)
    return entries, tables, cache, qkv


ATT_CASES = [
    # nq, nkv, d, page, new, old, window
    (4, 2, 16, 4, [1, 7, 33], [0, 0, 0], 0),
    (8, 2, 32, 8, [1, 1, 5], [40, 7, 16], 0),
    (6, 3, 48, 16, [3, 1, 20], [29, 100, 0], 24),
    (5, 5, 80, 16, [2, 9], [15, 16], 0),
    (32, 8, 128, 16, [1, 1, 64], [300, 17, 129], 0),
    (3, 1, 112, 32, [40], [31], 10),
]


@pytest.mark.parametrize("case", ATT_CASES)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_qk_norm_rope_write_then_attention(ops, case, dt):
    nq, nkv, d, page, new, old, window = case
    entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, new, old, window, dt, seed=20)
    cpu = CpuOps()
    table = torch.empty(512, d // 2, 2); cpu.rope_table(table, 1e4, d)
    qw, kw = 1 + 0.1 * g((d,), torch.float32, 30), 1 + 0.1 * g((d,), torch.float32, 31)
    bc = build_step_batch(entries, old, list(range(len(new))), [tables], "cpu")
    bg = build_step_batch(entries, old, list(range(len(new))), [tables], DEV)
    # plain
    T = qkv.shape[0]
    for in_dt in {torch.float32, dt}:
        qkv_in = qkv.to(in_dt)
        q_c, cache_c = torch.empty(T, nq * d, dtype=dt), cache.clone()
        cpu.qk_norm_rope_kv_write(qkv_in, q_c, qw, kw, 1e-6, table, d, bc, bc.block_tables[0], cache_c, 1, page,
                                  nq, nkv, d, True)
        q_g, cache_g = torch.empty(T, nq * d, dtype=dt, device=DEV), cache.clone().to(DEV)
        ops.qk_norm_rope_kv_write(qkv_in.to(DEV), q_g, qw.to(DEV), kw.to(DEV), 1e-6, table.to(DEV), d, bg,
                                  bg.block_tables[0], cache_g, 1, page, nq, nkv, d, True)
        tol = 2e-6 if dt == torch.float32 else 1e-2
        assert rel_err(q_g, q_c) < tol
        assert rel_err(cache_g, cache_c) < tol
    out_c = torch.empty(T, nq * d, dtype=dt)
    cpu.attention(q_c, bc, bc.block_tables[0], cache_c, 1, page, out_c, nq, nkv, d, 1 / math.sqrt(d), window)
    assert torch.equal(cache_g[:, 0].cpu(), cache[:, 0])            # the other layer is untouched
    out_g = torch.empty(T, nq * d, dtype=dt, device=DEV)
    # attention from the plain twin's cache, so that the two kernels are judged separately
    ops.attention(q_c.to(DEV), bg, bg.block_tables[0], cache_c.to(DEV), 1, page, out_g, nq, nkv, d,
                  1 / math.sqrt(d), window)
    assert rel_err(out_g, out_c) < (3e-6 if dt == torch.float32 else 1e-2)


@pytest.mark.parametrize("M,H,I", [(16, 4096, 12288), (5, 4096, 12288), (11, 520, 192), (16, 264, 64), (1, 64, 128)])
def test_gate_up_product_with_swiglu_in_the_cluster_for_normalised_rows(ops, M, H, I):
    """Decode steps whose norm was not deferred (another block arrangement): the rows come normalised in bfloat16,
    the clustered product applies SwiGLU itself; the feed-forward is two launches."""
    cpu = CpuOps()
    h = g((M, H), torch.bfloat16, 180)
    wg, wu = g((I, H), torch.bfloat16, 181, 0.05), g((I, H), torch.bfloat16, 182, 0.05)
    wd = g((H, I), torch.bfloat16, 183, 0.05)
    x = g((M, H), torch.float32, 184)
    want = x.clone(); cpu.gated_mlp(h, cpu.merge_gate_up(wg, wu), wd, want, I)
    xd = x.clone().to(DEV)
    launches = ops.launches
    ops.gated_mlp(h.to(DEV), ops.merge_gate_up(wg.to(DEV), wu.to(DEV)), wd.to(DEV), xd, I)
    assert ops.launches == launches + 2
    ops.check_errors()
    assert rel_err(xd - x.to(DEV), want - x) < 1.2e-2


@pytest.mark.parametrize("nq,nkv,page,new,old,K,norm,rope", [
    (32, 8, 16, [300, 450], [17, 0], 1024, True, True),      # two requests, the first with tokens cached
    (40, 8, 16, [777], [100], 512, True, True),              # 56 heads: 28 tiles of two heads
    (5, 2, 32, [600], [0], 256, True, True),                 # 9 heads: the last tile holds one head
    (8, 2, 8, [257], [3], 128, False, True),                 # no q/k norm
    (8, 2, 16, [300], [0], 128, True, False),                # no rotation
])
def test_qkv_projection_with_norm_rope_and_cache_write_in_the_epilogue(ops, nq, nkv, page, new, old, K, norm, rope):
    """Prompt-sized bfloat16 portions with heads of 128 run the projection, q/k RMSNorm, rotation and cache write
    as one kernel (the product on pairs of SMs with its q/k/v epilogue); against the plain twin of the two steps."""
    d, dt = 128, torch.bfloat16
    entries, tables, cache, _ = _paged_case(nq, nkv, d, page, new, old, 0, dt, seed=50)
    T = sum(new)
    cpu = CpuOps()
    table = torch.empty(2048, d // 2, 2); cpu.rope_table(table, 1e6, d)
    qw, kw = 1 + 0.1 * g((d,), torch.float32, 51), 1 + 0.1 * g((d,), torch.float32, 52)
    h = g((T, K), dt, 53)
    w = g(((nq + 2 * nkv) * d, K), dt, 54, 0.05)
    bc = build_step_batch(entries, old, list(range(len(new))), [tables], "cpu")
    bg = build_step_batch(entries, old, list(range(len(new))), [tables], DEV)
    q_c, cache_c = torch.empty(T, nq * d, dtype=dt), cache.clone()
    cpu.qkv_project(h, w, q_c, qw if norm else None, kw if norm else None, 1e-6, table if rope else None,
                    d if rope else 0, bc, bc.block_tables[0], cache_c, 1, page, nq, nkv, d, True)
    q_g, cache_g = torch.full((T, nq * d), float("nan"), dtype=dt, device=DEV), cache.clone().to(DEV)
    launches = ops.launches
    ops.qkv_project(h.to(DEV), w.to(DEV), q_g, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, 1e-6,
                    table.to(DEV) if rope else None, d if rope else 0, bg, bg.block_tables[0], cache_g, 1, page,
                    nq, nkv, d, True)
    assert ops.launches - launches == 1, "expected the one-kernel path"
    ops.check_errors()
    assert rel_err(q_g, q_c) < 1e-2
    assert rel_err(cache_g, cache_c) < 1e-2
    assert torch.equal(cache_g[:, 0].cpu(), cache[:, 0])            # the other layer is untouched
    # without the cache write only q is produced
    cache_g2 = cache.clone().to(DEV)
    ops.qkv_project(h.to(DEV), w.to(DEV), q_g, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None, 1e-6,
                    table.to(DEV) if rope else None, d if rope else 0, bg, bg.block_tables[0], cache_g2, 1, page,
                    nq, nkv, d, False)
    assert torch.equal(cache_g2.cpu(), cache)
    assert rel_err(q_g, q_c) < 1e-2


def test_qkv_projection_is_not_fused_where_another_plan_saves_a_wave(ops):
    """544 rows of a 7168-wide projection are 84 pair tiles on 74 pairs of SMs (two waves) and 140 single tiles on
    148 SMs (one): the projection then runs as the planned product and the separate kernel, with the same result."""
    nq, nkv, d, page, K, dt = 40, 8, 128, 16, 5120, torch.bfloat16
    new, old = [500, 44], [30, 0]
    assert ops.NUM_SMS == 148 and ops.prompt_plan(sum(new), (nq + 2 * nkv) * d, K, False)[1] != 512
    entries, tables, cache, _ = _paged_case(nq, nkv, d, page, new, old, 0, dt, seed=60)
    T = sum(new)
    cpu = CpuOps()
    table = torch.empty(2048, d // 2, 2); cpu.rope_table(table, 1e6, d)
    qw, kw = 1 + 0.1 * g((d,), torch.float32, 61), 1 + 0.1 * g((d,), torch.float32, 62)
    h = g((T, K), dt, 63)
    w = g(((nq + 2 * nkv) * d, K), dt, 64, 0.02)
    bc = build_step_batch(entries, old, list(range(len(new))), [tables], "cpu")
    bg = build_step_batch(entries, old, list(range(len(new))), [tables], DEV)
    q_c, cache_c = torch.empty(T, nq * d, dtype=dt), cache.clone()
    cpu.qkv_project(h, w, q_c, qw, kw, 1e-6, table, d, bc, bc.block_tables[0], cache_c, 1, page, nq, nkv, d, True)
    q_g, cache_g = torch.full((T, nq * d), float("nan"), dtype=dt, device=DEV), cache.clone().to(DEV)
    launches = ops.launches
    ops.qkv_project(h.to(DEV), w.to(DEV), q_g, qw.to(DEV), kw.to(DEV), 1e-6, table.to(DEV), d, bg, bg.block_tables[0],
                    cache_g, 1, page, nq, nkv, d, True)
    assert ops.launches - launches == 2, "expected the product and the separate kernel"
    ops.check_errors()
    assert rel_err(q_g, q_c) < 1e-2
    assert rel_err(cache_g, cache_c) < 1e-2


FLASH_CASES = [
    # nq, nkv, d, page, new, old, window, splits
    (32, 8, 128, 16, [1, 1, 1], [300, 17, 2049], 0, 1),        # decode, keys mode
    (32, 8, 128, 16, [1, 1, 1], [300, 17, 2049], 0, 4),        # decode, split keys (some splits empty)
    (32, 8, 128, 16, [1], [5], 0, 16),                         # more splits than key blocks
    (8, 8, 64, 8, [1, 2, 1], [63, 64, 65], 0, 3),              # no grouping, block edges
    (16, 2, 64, 32, [1, 1], [200, 31], 0, 2),                  # 8 heads a group: 8-row tiles
    (32, 8, 128, 16, [70, 1, 33], [0, 500, 129], 0, 1),        # portions beside a decode token (rows mode)
    (32, 8, 128, 16, [200], [0], 0, 1),                        # a whole prompt, several tiles
    (12, 4, 64, 16, [50, 3], [77, 10], 0, 1),                  # 3 heads a group: tiles cut through tokens
    (8, 2, 128, 16, [40, 1], [100, 150], 48, 1),               # sliding window, rows mode
    (8, 2, 128, 16, [1, 1], [100, 30], 48, 2),                 # sliding window, decode
    (4, 4, 128, 16, [130], [1], 0, 2),                         # rows mode with split keys
    (32, 8, 128, 16, [1] * 6, [3000, 10, 200, 50, 7, 129], 0, None),      # unequal contexts: the split follows sum / longest
    (32, 8, 128, 16, [70, 1, 1, 1], [40, 2500, 9, 300], 0, None),         # the same beside a portion (two launches)
    (32, 8, 128, 16, [16], [700], 0, 8),                       # a small portion behind a long context: 64-row tiles, split keys
    (12, 4, 64, 32, [50, 7], [1000, 30], 0, 4),                # the same with 3 heads a group and a second, short request
    (8, 2, 128, 16, [40, 9], [600, 150], 48, 4),               # ... and a sliding window (shares before the window are empty)
    (32, 8, 128, 16, [16], [2500], 0, None),                   # the share count chosen by the library (16)
    (40, 8, 128, 16, [50, 1, 1], [1500, 300, 2000], 0, None),  # beside decoded tokens the portion keeps one share (two launches)
    (32, 8, 128, 16, [20, 1, 1], [6500, 300, 2000], 0, None),  # ... unless its context is long: shares in both launches
]


@pytest.mark.parametrize("case", FLASH_CASES)
def test_flash_attention_bf16(ops, case):
    nq, nkv, d, page, new, old, window, splits = case
    dt = torch.bfloat16
    entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, new, old, window, dt, seed=70, layers=2)
    # slots beyond each request's tokens and unused pages hold NaN: reading them shows
    used = torch.zeros(cache.shape[0], page, dtype=torch.bool)
    for tb, n, o in zip(tables, new, old):
        for pos in range(n + o):
            used[tb[pos // page], pos % page] = True
    cache = cache.clone()
    cache.permute(0, 4, 1, 2, 3, 5)[~used] = float("nan")
    if window > 0:                                             # pages a window has passed are given back
        for i, (tb, n, o) in enumerate(zip(tables, new, old)):
            first_needed = max(0, o - window + 1) // page
            tables[i] = [-1] * first_needed + tb[first_needed:]
    T = sum(new)
    q = qkv[:, :nq * d].contiguous()
    bc = build_step_batch(entries, old, list(range(len(new))), [tables], "cpu")
    bg = build_step_batch(entries, old, list(range(len(new))), [tables], DEV)
    want = torch.empty(T, nq * d, dtype=dt)
    ctab = bc.block_tables[0].clone()
    CpuOps().attention(q, bc, ctab.clamp_min(0) if window > 0 else ctab, torch.nan_to_num(cache, nan=1e4),
                       1, page, want, nq, nkv, d, 1 / math.sqrt(d), window)
    out = torch.full((T, nq * d), float("nan"), dtype=dt, device=DEV)
    ops.attention_bf16(q.to(DEV), bg, bg.block_tables[0], cache.to(DEV), 1, page, out, nq, nkv, d, 1 / math.sqrt(d),
                       window, num_splits=splits)
    assert torch.isfinite(out).all()
    assert rel_err(out, want) < 1e-2
    gen = torch.empty(T, nq * d, dtype=dt, device=DEV)
    ops.attention_generic(q.to(DEV), bg, bg.block_tables[0], torch.nan_to_num(cache, nan=1e4).to(DEV), 1, page, gen,
                          nq, nkv, d, 1 / math.sqrt(d), window)
    assert rel_err(out, gen) < 1e-2


@pytest.mark.parametrize("nq,nkv,d,page,new,old", [(32, 8, 128, 16, [700], [300]), (8, 2, 64, 32, [333, 40], [0, 1000]),
                                                   (8, 8, 128, 8, [129, 2], [65, 3]),
                                                   # CTAs of two tiles whose tiles take turns at the exponentials: an odd
                                                   # number of tiles (the last CTA has one, and that one partial), heads
                                                   # of 64, and two requests of which the shorter leaves CTAs without rows
                                                   (32, 8, 128, 16, [650], [100]), (16, 4, 64, 16, [1300], [0]),
                                                   (32, 8, 128, 16, [300, 420], [0, 64])])
def test_prompt_attention_when_the_running_maximum_jumps_late(ops, nq, nkv, d, page, new, old):
    """Keys whose scores tower over everything before them, planted deep into the sequence: the
    running maximum grows by far more than the lazy-rescale threshold, so the output accumulated
    so far must be scaled down, more than once, and many key blocks go round the stage ring."""
    dt = torch.bfloat16
    entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, new, old, 0, dt, seed=90, layers=1)
    q = qkv[:, :nq * d].contiguous().view(-1, nq, d)
    q[:, :, 5] = 6.0
    G = nq // nkv
    for i, (tb, n, o) in enumerate(zip(tables, new, old)):
        total = n + o
        for frac, boost in ((0.35, 8.0), (0.6, 16.0), (0.9, 30.0)):
            pos = int(total * frac)
            cache[tb[pos // page], 0, 0, :, pos % page, 5] = boost          # score ~ 6 * boost / sqrt(d)
    q = q.view(-1, nq * d)
    T = q.shape[0]
    bc = build_step_batch(entries, old, list(range(len(new))), [tables], "cpu")
    bg = build_step_batch(entries, old, list(range(len(new))), [tables], DEV)
    want = torch.empty(T, nq * d, dtype=dt)
    CpuOps().attention(q, bc, bc.block_tables[0], cache, 0, page, want, nq, nkv, d, 1 / math.sqrt(d), 0)
    out = torch.full((T, nq * d), float("nan"), dtype=dt, device=DEV)
    ops.attention_bf16(q.to(DEV), bg, bg.block_tables[0], cache.to(DEV), 0, page, out, nq, nkv, d, 1 / math.sqrt(d), 0)
    assert torch.isfinite(out).all()
    assert rel_err(out, want) < 1e-2
    ops.check_errors()


@pytest.mark.parametrize("nq,nkv,new,old", [(40, 8, [300], [0]), (40, 8, [277], [0]), (40, 8, [300], [1500]),
                                            (24, 8, [150, 43], [700, 0]), (32, 8, [301], [900])])
def test_prompt_attention_with_a_warp_on_the_masked_path_beside_warps_on_the_short_one(ops, nq, nkv, new, old):
    """The last tile of packed rows ends inside a warp (5 or 3 query heads a key/value head, or a token count
    that leaves a remainder): that warp masks every key block, its neighbours take the short path and run
    ahead.  Launched several times back to back, as a model's layers are, and compared row by row: a
    product issued before the slow warp's probabilities were written shows in that warp's rows only."""
    dt, d, page = torch.bfloat16, 128, 16
    entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, new, old, 0, dt, seed=91, layers=1)
    q = qkv[:, :nq * d].contiguous()
    T = q.shape[0]
    bc = build_step_batch(entries, old, list(range(len(new))), [tables], "cpu")
    bg = build_step_batch(entries, old, list(range(len(new))), [tables], DEV)
    want = torch.empty(T, nq * d, dtype=dt)
    CpuOps().attention(q, bc, bc.block_tables[0], cache, 0, page, want, nq, nkv, d, 1 / math.sqrt(d), 0)
    qg, cg = q.to(DEV), cache.to(DEV)
    outs = [torch.full((T, nq * d), float("nan"), dtype=dt, device=DEV) for _ in range(8)]
    for out in outs:
        ops.attention_bf16(qg, bg, bg.block_tables[0], cg, 0, page, out, nq, nkv, d, 1 / math.sqrt(d), 0)
    ops.check_errors()
    w = want.double().view(T * nq, d)
    scale = w.abs().amax(dim=-1).clamp_min(1e-3)
    for k, out in enumerate(outs):
        assert torch.isfinite(out).all()
        err = (out.cpu().double().view(T * nq, d) - w).abs().amax(dim=-1) / scale
        worst = int(err.argmax())
        assert float(err[worst]) < 3e-2, f"launch {k}: token {worst // nq} head {worst % nq} off by {float(err[worst]):.3f}"


def test_accumulator_buffers_are_left_at_zero_by_their_readers(ops):
    """Decode-sized bfloat16 projections add their split shares into a persistent float32 buffer; the kernel
    that reads the buffer clears it, so that no clearing kernel runs.  Two rounds through the same buffers."""
    nq, nkv, d, page, H, I = 8, 2, 64, 16, 256, 320
    W = (nq + 2 * nkv) * d
    cpu = CpuOps()
    table = torch.empty(128, d // 2, 2); cpu.rope_table(table, 1e4, d)
    for rnd in range(2):
        T = 5
        h = g((T, H), torch.bfloat16, 80 + rnd)
        w_qkv = g((W, H), torch.bfloat16, 82 + rnd, 0.05)
        qkv = ops.projection_buffer(T, W, DEV, torch.bfloat16)
        assert float(qkv.abs().max()) == 0.0
        launches = ops.launches
        ops.gemm(h.to(DEV), w_qkv.to(DEV), qkv)
        assert ops.launches == launches + 1                       # no clearing kernel
        ref = (h.double() @ w_qkv.double().t())
        assert rel_err(qkv, ref) < 1e-5
        entries = [StepEntry(0, [0] * T, [])]
        tables = [[[3, 1]]]
        bg = build_step_batch(entries, [7], [0], tables, DEV)
        bc = build_step_batch(entries, [7], [0], tables, "cpu")
        cache_g = torch.zeros((4, 1, 2, nkv, page, d), dtype=torch.bfloat16, device=DEV)
        cache_c = torch.zeros((4, 1, 2, nkv, page, d), dtype=torch.bfloat16)
        q_g = torch.empty(T, nq * d, dtype=torch.bfloat16, device=DEV)
        q_c = torch.empty(T, nq * d, dtype=torch.bfloat16)
        qkv_host = qkv.cpu().clone()
        ops.qk_norm_rope_kv_write(qkv, q_g, None, None, 1e-6, table.to(DEV), d, bg, bg.block_tables[0], cache_g, 0, page,
                                  nq, nkv, d, True)
        cpu.qk_norm_rope_kv_write(qkv_host, q_c, None, None, 1e-6, table, d, bc, bc.block_tables[0], cache_c, 0, page,
                                  nq, nkv, d, True)
        assert rel_err(q_g, q_c) < 1e-2 and rel_err(cache_g, cache_c) < 1e-2
        assert float(qkv.abs().max()) == 0.0                      # cleared by its reader
        # gate/up accumulators, cleared by the SwiGLU kernel
        a = g((T, H), torch.bfloat16, 84 + rnd)
        wg, wu = g((I, H), torch.bfloat16, 86 + rnd, 0.05), g((I, H), torch.bfloat16, 88 + rnd, 0.05)
        out = torch.empty(T, I, dtype=torch.bfloat16, device=DEV)
        ops.gemm_swiglu(a.to(DEV), ops.merge_gate_up(wg.to(DEV), wu.to(DEV)), out)
        gate, up = a.double() @ wg.double().t(), a.double() @ wu.double().t()
        assert rel_err(out, (gate / (1 + torch.exp(-gate))) * up) < 1.2e-2
        assert float(ops.projection_buffer(T, 2 * I, DEV, torch.bfloat16).abs().max()) == 0.0
    ops.check_errors()


def test_attention_finds_one_far_key_among_hundreds(ops):
    """One key far back is made to dominate: a kernel that skips a page, or reads the wrong
    one, returns something else than that key's value."""
    nq, nkv, d, page = 4, 2, 64, 16
    old, new = [700], [1]
    for dt in (torch.float32, torch.bfloat16):
        entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, new, old, 0, dt, seed=40, layers=1, layer=0)
        far = 37
        pg, slot = tables[0][far // page], far % page
        q = qkv.view(1, nq + 2 * nkv, d)[:, :nq].contiguous()
        for kvh in range(nkv):
            cache[pg, 0, 0, kvh, slot] = 0
            cache[pg, 0, 0, kvh, slot, 3] = 60.0
        q[0, :, 3] = 40.0
        bg = build_step_batch(entries, old, [0], [tables], DEV)
        # the new token's own key/value sit at position 700
        p700 = tables[0][700 // page]
        cache[p700, 0] = 0
        out = torch.empty(1, nq * d, dtype=dt, device=DEV)
        ops.attention(q.view(1, nq * d).to(DEV), bg, bg.block_tables[0], cache.to(DEV), 0, page, out, nq, nkv, d, 1 / math.sqrt(d), 0)
        for h in range(nq):
            want = cache[pg, 0, 1, h // 2, slot].float()
            assert torch.allclose(out[0, h * d:(h + 1) * d].float().cpu(), want, atol=2e-2, rtol=2e-2)


def _dense_attention_on_gpu(q, cache, table, layer, page, first_pos, nq, nkv, d):
    """softmax(q k^T / sqrt(d)) v over keys 0..position, in float32 on the GPU, for one request whose
    rows sit at positions first_pos, first_pos + 1, ... (plain formulas; blocks of rows bound the memory)."""
    n = q.shape[0]
    total = first_pos + n
    pages = torch.tensor(table[:-(-total // page)], device=DEV)
    kv = cache[pages, layer].float()                               # [blocks, 2, nkv, page, d]
    k = kv[:, 0].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :total]
    v = kv[:, 1].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :total]
    qh = q.float().view(n, nq, d)
    out = torch.empty(n, nq, d, device=DEV)
    G = nq // nkv
    keys = torch.arange(total, device=DEV)
    for r0 in range(0, n, 256):
        rows = slice(r0, min(n, r0 + 256))
        pos = first_pos + torch.arange(rows.start, rows.stop, device=DEV)
        for h in range(nq):
            s = (qh[rows, h] @ k[h // G].t()) / math.sqrt(d)
            s = s.masked_fill(keys[None, :] > pos[:, None], float("-inf"))
            out[rows, h] = torch.softmax(s, dim=-1) @ v[h // G]
    return out.view(n, nq * d)


@pytest.mark.parametrize("new,old,splits", [(2085, 18000, None), (1, 33000, None), (1, 33000, 16), (9, 20000, 4)])
def test_attention_at_long_context(ops, new, old, splits):
    """Tens of thousands of keys behind the new tokens (a portion of a long prompt; a decoded token),
    with two keys made to stand out, one at the far end and one in the middle: offsets into the cache
    and the block table, the number of key blocks and the split of the key range at sizes that the
    other tests do not reach."""
    nq, nkv, d, page = 8, 2, 128, 16
    dt = torch.bfloat16
    entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, [new], [old], 0, dt, seed=120, layers=2)
    cache = cache.to(DEV)
    q = qkv[:, :nq * d].contiguous().view(-1, nq, d)
    q[:, :, 9] = 6.0                                               # score 6 * 24 / sqrt(128) = 12.7 against N(0, 1)
    for pos, boost in ((11, 24.0), (old // 2 + 3, 24.5)):
        cache[tables[0][pos // page], 1, 0, :, pos % page, 9] = boost
    q = q.view(-1, nq * d).to(DEV)
    bg = build_step_batch(entries, [old], [0], [tables], DEV)
    out = torch.full((new, nq * d), float("nan"), dtype=dt, device=DEV)
    if splits is None:
        ops.attention(q, bg, bg.block_tables[0], cache, 1, page, out, nq, nkv, d, 1 / math.sqrt(d), 0)
    else:
        ops.attention_bf16(q, bg, bg.block_tables[0], cache, 1, page, out, nq, nkv, d, 1 / math.sqrt(d), 0,
                           num_splits=splits)
    ops.check_errors()
    want = _dense_attention_on_gpu(q, cache, tables[0], 1, page, old, nq, nkv, d)
    assert torch.isfinite(out).all()
    assert rel_err(out, want) < 1e-2


def test_window_edge_is_exact(ops):
    """With window w the key at p-w+1 counts and the key at p-w does not."""
    nq, nkv, d, page, w = 2, 1, 32, 8, 9
    old, new = [30], [1]
    entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, new, old, w, torch.float32, seed=50, layers=1)
    p = 30
    cache[:, 0, 0] = 0
    q = torch.zeros(1, nq, d); q[0, :, 0] = 10.0
    def put(pos, score, val):
        pg, sl = tables[0][pos // page], pos % page
        cache[pg, 0, 0, 0, sl, 0] = score
        cache[pg, 0, 1, 0, sl] = val
    for pos in range(31):
        put(pos, 0.0, 0.0)
    put(p - w, 50.0, 7.0)          # just outside: must not be seen
    put(p - w + 1, 8.0, 3.0)       # first key inside
    bg = build_step_batch(entries, old, [0], [tables], DEV)
    out = torch.empty(1, nq * d, device=DEV)
    ops.attention(q.view(1, nq * d).to(DEV), bg, bg.block_tables[0], cache.to(DEV), 0, page, out, nq, nkv, d, 1 / math.sqrt(d), w)
    assert float(out.max()) <= 3.0 + 1e-4 and float(out.max()) > 2.9


WINDOW_EDGE_CASES = [
    # nq, nkv, d, page, new, old, window, splits
    (8, 2, 128, 16, 1, 100, 48, 1),      # decode: first key of the window (53) in the middle of a page
    (8, 2, 128, 16, 1, 100, 48, 4),      # the same with the key range shared out
    (8, 2, 128, 16, 1, 111, 48, 1),      # first key of the window (64) on a 64-key block boundary
    (8, 2, 128, 16, 1, 111, 48, 3),
    (4, 4, 64, 8, 1, 130, 40, 2),        # heads of 64, pages of 8
    (8, 2, 128, 16, 2, 100, 48, 1),      # a two-token portion: the rows of a tile have different first keys
    (8, 2, 128, 16, 140, 60, 48, 1),     # a portion of prompt size (the tcgen05 kernel): every row its own edge
    (4, 2, 64, 16, 150, 37, 40, 1),
    (16, 2, 128, 16, 3, 200, 100, None),  # eight heads a group, splits chosen by the library
]


@pytest.mark.parametrize("case", WINDOW_EDGE_CASES)
def test_window_edge_is_exact_in_the_bf16_kernels(ops, case):
    """Queries and keys are built so that, for EVERY query row at position p, the key at p - w (just outside
    the window) would take all the weight if it were seen (score 30 against 0), and the key at p - w + 1 (the
    first one inside) takes most of it (score 8): a kernel that is off by one at either side of the edge
    returns another key's value, far outside the tolerance.  Pages that the window of the first row has
    passed are given back (-1 in the block table)."""
    nq, nkv, d, page, new, old, w, splits = case
    dt = torch.bfloat16
    assert w < d
    entries, tables, cache, qkv = _paged_case(nq, nkv, d, page, [new], [old], w, dt, seed=130, layers=2)
    scale = 1 / math.sqrt(d)
    total = old + new
    cache[:, 1, 0] = 0
    for j in range(total):                                     # key j: one unit in dimension j mod d
        cache[tables[0][j // page], 1, 0, :, j % page, j % d] = 1.0
    q = torch.zeros(new, nq, d)
    for r in range(new):
        pos = old + r
        q[r, :, (pos - w) % d] = 30.0 / scale
        q[r, :, (pos - w + 1) % d] = 8.0 / scale
    q = q.to(dt).view(new, nq * d)
    first_needed = max(0, old - w + 1) // page
    tables[0] = [-1] * first_needed + tables[0][first_needed:]
    # what the released pages held is poison now
    cache = cache.clone()
    gone = torch.ones(cache.shape[0], dtype=torch.bool)
    gone[torch.tensor([pg for pg in tables[0] if pg >= 0])] = False
    cache[gone] = float("nan")
    bc = build_step_batch(entries, [old], [0], [tables], "cpu")
    bg = build_step_batch(entries, [old], [0], [tables], DEV)
    want = torch.empty(new, nq * d, dtype=dt)
    CpuOps().attention(q, bc, bc.block_tables[0], cache, 1, page, want, nq, nkv, d, scale, w)
    assert torch.isfinite(want).all()
    # the plain result is, to 2 %, the value of the first key inside the window: the construction bites
    for r in (0, new - 1):
        j = old + r - w + 1
        if j < 0:
            continue                                           # the window of this row starts before the sequence
        v = cache[tables[0][j // page], 1, 1, :, j % page].float()              # [nkv, d]
        got = want[r].float().view(nq, d)
        assert float((got - v.repeat_interleave(nq // nkv, 0)).abs().max()) < 0.05 * float(v.abs().max()) + 0.05
    out = torch.full((new, nq * d), float("nan"), dtype=dt, device=DEV)
    if splits is None:
        ops.attention(q.to(DEV), bg, bg.block_tables[0], cache.to(DEV), 1, page, out, nq, nkv, d, scale, w)
    else:
        ops.attention_bf16(q.to(DEV), bg, bg.block_tables[0], cache.to(DEV), 1, page, out, nq, nkv, d, scale, w,
                           num_splits=splits)
    ops.check_errors()
    assert torch.isfinite(out).all()
    assert rel_err(out, want) < 1e-2


@pytest.mark.parametrize("R,V", [(1, 100), (5, 311), (3, 151936), (64, 4097)])
def test_argmax_first_maximum(ops, R, V):
    logits = g((R, V), torch.float32, 60)
    logits[0, V // 2] = 99.0; logits[0, V - 1] = 99.0          # a tie: the lower id wins
    want = torch.empty(R, dtype=torch.int32); CpuOps().argmax(logits, want)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.argmax(logits.to(DEV), out)
    assert out.cpu().tolist() == want.tolist() and int(out[0]) == V // 2


@pytest.mark.parametrize("V", [311, 4097, 151936])
@pytest.mark.parametrize("peaked", [False, True, "crowded"])
def test_sampling_matches_plain_inverse_cdf(ops, V, peaked):
    R = 24
    logits = g((R, V), torch.float32, 61, 3.0)
    if peaked == "crowded" and V > 2000:
        # hundreds of equal top logits side by side: more candidates in one stretch of the row than its share of
        # the list holds, so the search goes back to passes over the whole row (and ties at the threshold are all kept)
        logits[:, 1000:1400] = 14.0
    elif peaked:
        # a few tokens stand far above a quiet rest, as a trained model's logits do: the tokens that can matter to
        # top-k / top-p are few, and the threshold is searched among them in shared memory; the wide random rows
        # above have tens of thousands of such tokens, and the large vocabulary takes the search over the whole row
        logits = logits * 0.4
        gen = torch.Generator().manual_seed(62)
        for r in range(R):
            ids = torch.randint(0, V, (12,), generator=gen)
            logits[r, ids] += 6.0 + 6.0 * torch.rand(12, generator=gen)
    rng = np.random.default_rng(0)
    temp = torch.tensor([0.0 if r % 6 == 0 else 0.5 + 0.1 * r for r in range(R)])
    u = torch.from_numpy(rng.random(R).astype(np.float32))
    for filt in (False, True):
        top_k = torch.tensor([0, 5, 50, 0] * 6, dtype=torch.int32) if filt else None
        top_p = torch.tensor([1.0, 1.0, 0.9, 0.5] * 6) if filt else None
        min_p = torch.tensor([0.0, 0.0, 0.0, 0.02] * 6) if filt else None
        want = torch.empty(R, dtype=torch.int32)
        CpuOps().sample(logits, temp, u, want, top_k, top_p, min_p)
        out = torch.empty(R, dtype=torch.int32, device=DEV)
        ops.sample(logits.to(DEV), temp.to(DEV), u.to(DEV), out,
                   None if top_k is None else top_k.to(DEV), None if top_p is None else top_p.to(DEV),
                   None if min_p is None else min_p.to(DEV))
        same = sum(int(a == b) for a, b in zip(out.cpu().tolist(), want.tolist()))
        assert same >= R - 1, (filt, out.cpu().tolist(), want.tolist())    # float32 vs float64 cumulative sums


def test_repetition_penalty(ops):
    logits = g((3, 50), torch.float32, 62)
    rows = torch.tensor([0, 0, 2], dtype=torch.int32); toks = torch.tensor([3, 7, 49], dtype=torch.int32)
    pen = torch.tensor([1.5, 1.5, 2.0])
    want = logits.clone(); CpuOps().repetition_penalty(want, rows, toks, pen)
    out = logits.clone().to(DEV)
    ops.repetition_penalty(out, rows.to(DEV), toks.to(DEV), pen.to(DEV))
    assert torch.allclose(out.cpu(), want, rtol=1e-6)
