"""Each part of a layer alone, built through the registry with sizes of its own, against
the plain function of the same part (tests/plain_qwen3.py), in 32-bit and in bfloat16."""

import pytest
import torch

import plain_qwen3 as P
from tffinfer_b200 import get_part
from tffinfer_b200.engine.batch import StepEntry
from host_twin import build_step_batch
from tffinfer_b200.parts import LayerContext, PartSpec, build_part

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 5e-6, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def ops():
    from tffinfer_b200.kernels.library import CudaKernels
    return CudaKernels()


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def rel(got, want):
    return float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())


def _load(part, weights, ops, dt):
    held = {}
    for name, spec in part.weight_specs().items():
        t = weights[name]
        assert tuple(t.shape) == tuple(spec.shape)
        held[name] = t.to(DEV, torch.float32 if spec.role == "vector" else dt).contiguous()
    part.load(held, ops, dt)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,eps", [(80, 1e-5), (4096, 1e-6)])
def test_rms_norm_part(ops, dt, dim, eps):
    part = build_part("norm", PartSpec("rms_norm", dict(dim=dim, eps=eps)))
    w = {"weight": 1 + 0.1 * rnd((dim,), 1)}
    _load(part, w, ops, dt)
    x = rnd((9, dim), 2, 2.0)
    got = part.forward(x.to(DEV), ops, dt)
    assert got.dtype == dt and rel(got, P.rms_norm(x.double(), w["weight"].double(), eps)) < TOL[dt]


@pytest.mark.parametrize("d,theta", [(16, 1e4), (48, 5e5), (128, 1e6)])
def test_rotary_part_table(ops, d, theta):
    part = build_part("position", PartSpec("rotary", dict(head_dim=d, theta=theta)))
    part.prepare(ops, DEV, 300)
    table, rot = part.rotary()
    ang = P.rope_angles(range(300), d, theta).double()
    assert rot == d
    assert float((table[..., 0].cpu().double() - torch.cos(ang)).abs().max()) < 2e-6
    assert float((table[..., 1].cpu().double() - torch.sin(ang)).abs().max()) < 2e-6


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,I", [(80, 112), (256, 1000)])
def test_swiglu_part(ops, dt, H, I):
    part = build_part("feed_forward", PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I), prefix="mlp"))
    w = {"gate_proj.weight": rnd((I, H), 3, 0.05), "up_proj.weight": rnd((I, H), 4, 0.05),
         "down_proj.weight": rnd((H, I), 5, 0.05)}
    if dt == torch.bfloat16:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    _load(part, w, ops, dt)
    h = rnd((11, H), 6).to(dt)
    res = rnd((11, H), 7)
    out = part.forward(h.to(DEV), LayerContext(batch=None, ops=ops), res.clone().to(DEV))
    want = res.double() + P.swiglu_mlp(h.double(), {f"mlp.{k}": v.double() for k, v in w.items()}, "mlp")
    assert rel(out, want) < TOL[dt]


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,nq,nkv,d,window,theta", [(64, 4, 2, 16, 0, 1e4), (96, 8, 2, 32, 0, 1e6),
                                                      (80, 6, 3, 48, 7, 5e5), (128, 2, 2, 128, 0, 1e6)])
def test_attention_part_with_cache_across_two_steps(ops, dt, H, nq, nkv, d, window, theta):
    eps = 1e-5
    part = build_part("mixer", PartSpec("gqa_attention", dict(hidden_size=H, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                                                              qk_norm=True, qk_norm_eps=eps, window=window), prefix="a"))
    rope = build_part("position", PartSpec("rotary", dict(head_dim=d, theta=theta)))
    rope.prepare(ops, DEV, 64)
    w = {"q_proj.weight": rnd((nq * d, H), 1, 0.08), "k_proj.weight": rnd((nkv * d, H), 2, 0.08),
         "v_proj.weight": rnd((nkv * d, H), 3, 0.08), "o_proj.weight": rnd((H, nq * d), 4, 0.08),
         "q_norm.weight": 1 + 0.1 * rnd((d,), 5), "k_norm.weight": 1 + 0.1 * rnd((d,), 6)}
    if dt == torch.bfloat16:
        w = {k: (v.bfloat16().float() if "proj" in k else v) for k, v in w.items()}
    _load(part, w, ops, dt)
    T, page = 29, 4
    h = rnd((T, H), 7).to(dt)
    cfg = dict(heads=nq, kv_heads=nkv, head_dim=d, eps=eps, theta=theta)
    want = P.attention_block(h.double(), {f"a.{k}": v.double() for k, v in w.items()}, "a", cfg, range(T), window)
    cache = torch.full((10, 1, 2, nkv, page, d), float("nan"), dtype=dt, device=DEV)
    table = [[7, 2, 9, 0, 5, 3, 8, 1]]
    got = []
    for start, n in ((0, 18), (18, 11)):                        # a portion, then the rest
        b = build_step_batch([StepEntry("r", [0] * n, [])], [start], [0], [table], DEV)
        ctx = LayerContext(batch=b, ops=ops, kv_cache=cache, kv_layer=0, block_table=b.block_tables[0],
                           page_size=page, write_cache=True, position=rope)
        res = torch.zeros(n, H, device=DEV)
        got.append(part.forward(h[start:start + n].to(DEV).contiguous(), ctx, res))
    assert rel(torch.cat(got), want) < TOL[dt]


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_pre_norm_block(ops, dt):
    H, I, nq, nkv, d, eps, theta = 96, 160, 8, 2, 32, 1e-5, 1e6
    mk = lambda fam, kind, params, prefix: build_part(fam, PartSpec(kind, params, prefix))
    block = get_part("block", "pre_norm")(
        mixer=mk("mixer", "gqa_attention", dict(hidden_size=H, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                                                qk_norm=True, qk_norm_eps=eps), "model.layers.0.self_attn"),
        feed_forward=mk("feed_forward", "swiglu", dict(hidden_size=H, intermediate_size=I), "model.layers.0.mlp"),
        mixer_norm=mk("norm", "rms_norm", dict(dim=H, eps=eps), "model.layers.0.input_layernorm"),
        ffn_norm=mk("norm", "rms_norm", dict(dim=H, eps=eps), "model.layers.0.post_attention_layernorm"))
    full = {}
    for i, p in enumerate(block.parts()):
        for name, spec in p.weight_specs().items():
            t = (1 + 0.1 * rnd(spec.shape, 10 + i)) if spec.role == "vector" else rnd(spec.shape, 20 + i + len(full), 0.08)
            full[p.full_name(name)] = t.bfloat16().float() if dt == torch.bfloat16 and spec.role != "vector" else t
        _load(p, {n: full[p.full_name(n)] for n in p.weight_specs()}, ops, dt)
    rope = build_part("position", PartSpec("rotary", dict(head_dim=d, theta=theta)))
    rope.prepare(ops, DEV, 64)
    T, page = 13, 8
    x = rnd((T, H), 3)
    cfg = dict(heads=nq, kv_heads=nkv, head_dim=d, eps=eps, theta=theta, windows=[0])
    want = P.decoder_layer(x.double(), {k: v.double() for k, v in full.items()}, 0, cfg, range(T))
    b = build_step_batch([StepEntry("r", [0] * T, [])], [0], [0], [[[1, 0]]], DEV)
    cache = torch.zeros((2, 1, 2, nkv, page, d), dtype=dt, device=DEV)
    ctx = LayerContext(batch=b, ops=ops, kv_cache=cache, kv_layer=0, block_table=b.block_tables[0], page_size=page,
                       write_cache=True, position=rope)
    got = block.forward(x.clone().to(DEV), ctx, dt)
    assert rel(got, want) < TOL[dt]
