"""The plain implementation checked against itself and against hand-computed cases: the oracle
of every other test has to be right by inspection."""
import math

import pytest
import torch

import plain_qwen3 as P
from helpers import tiny_config, make_model_dir

D = torch.float64


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=D)
    w = torch.tensor([2.0, 0.5], dtype=D)
    r = 1 / math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(P.rms_norm(x, w, 1e-6), torch.tensor([[3 * r * 2, 4 * r * 0.5]], dtype=D))


def test_silu_and_swiglu_by_hand():
    assert abs(float(P.silu(torch.tensor(0.0, dtype=D)))) == 0.0
    assert abs(float(P.silu(torch.tensor(1.0, dtype=D))) - 1 / (1 + math.exp(-1))) < 1e-15
    w = {"m.gate_proj.weight": torch.tensor([[1.0]], dtype=D), "m.up_proj.weight": torch.tensor([[2.0]], dtype=D),
         "m.down_proj.weight": torch.tensor([[3.0]], dtype=D)}
    h = torch.tensor([[0.5]], dtype=D)
    want = (0.5 / (1 + math.exp(-0.5))) * 1.0 * 3.0
    assert abs(float(P.swiglu_mlp(h, w, "m")) - want) < 1e-15


def test_rope_pairs_i_with_i_plus_half_and_keeps_relative_angles():
    d, theta = 8, 1e4
    x = torch.zeros(1, 1, d, dtype=D); x[0, 0, 1] = 1.0                 # element 1 pairs with element 1 + d/2 = 5
    ang = P.rope_angles([3], d, theta)
    y = P.rope_rotate_half(x, ang)[0, 0]
    f = math.exp(-(2 * 1 / d) * math.log(theta))
    a = float(torch.tensor(3.0, dtype=torch.float32) * torch.tensor(f, dtype=torch.float32))
    assert abs(float(y[1]) - math.cos(a)) < 1e-12 and abs(float(y[5]) - math.sin(a)) < 1e-12
    assert float(y.abs().sum()) == pytest.approx(abs(math.cos(a)) + abs(math.sin(a)))
    # q.k after rotation depends on the distance only
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, d, generator=g, dtype=D), torch.randn(1, 1, d, generator=g, dtype=D)
    def score(pq, pk):
        return float((P.rope_rotate_half(q, P.rope_angles([pq], d, theta)) * P.rope_rotate_half(k, P.rope_angles([pk], d, theta))).sum())
    assert abs(score(5, 2) - score(13, 10)) < 1e-5                      # float32 angles
    assert abs(score(5, 2) - score(5, 3)) > 1e-3


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    T, H, KV, d = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=D) for n in (H, KV, KV))
    full = P.causal_attention(q, k, v)
    # a prefix sees nothing of what follows
    assert torch.allclose(P.causal_attention(q[:5], k[:5], v[:5]), full[:5])
    # the first token attends to itself only
    assert torch.allclose(full[0], v[0].repeat_interleave(H // KV, 0))
    # query head h reads kv head h // 2: changing kv head 1 leaves heads 0 and 1 alone
    k2, v2 = k.clone(), v.clone(); k2[:, 1] += 1.0; v2[:, 1] -= 2.0
    other = P.causal_attention(q, k2, v2)
    assert torch.allclose(other[:, :2], full[:, :2]) and not torch.allclose(other[:, 2:], full[:, 2:])
    # window w: position p sees p-w+1 .. p
    win = P.causal_attention(q, k, v, window=3)
    assert torch.allclose(win[:3], full[:3])
    assert torch.allclose(win[6], P.causal_attention(q[4:7], k[4:7], v[4:7])[2])
    # by hand for one head: softmax of two scores
    s = torch.stack([q[1, 0] @ k[0, 0], q[1, 0] @ k[1, 0]]) / math.sqrt(d)
    p = torch.softmax(s, 0)
    assert torch.allclose(full[1, 0], p[0] * v[0, 0] + p[1] * v[1, 0])


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_model_is_causal_and_uses_its_options(tmp_path, name):
    d = make_model_dir(tmp_path, name)
    pm = P.PlainModel(d)
    cfg = tiny_config(name)
    assert pm.cfg["tied"] == cfg.tie_word_embeddings and pm.cfg["head_dim"] == cfg.head_dim
    assert pm.cfg["windows"] == [cfg.window_of_layer(i) for i in range(cfg.num_layers)]
    toks = [(7 * i + 3) % cfg.vocab_size for i in range(60)]
    full = pm.logits(toks)
    assert full.shape == (60, cfg.vocab_size)
    assert torch.allclose(pm.logits(toks[:17]), full[:17], atol=1e-12)
    changed = list(toks); changed[40] = (changed[40] + 1) % cfg.vocab_size
    other = pm.logits(changed)
    assert torch.allclose(other[:40], full[:40], atol=1e-12) and not torch.allclose(other[40:], full[40:])


def test_samplers_by_hand():
    logits = torch.tensor([0.0, math.log(3.0), math.log(3.0), -50.0], dtype=D)     # p = 1/7, 3/7, 3/7, ~0
    assert P.sample_greedy(logits) == 1                                   # first maximum
    assert P.sample_temperature(logits, 1.0, 0.10) == 0
    assert P.sample_temperature(logits, 1.0, 0.20) == 1
    assert P.sample_temperature(logits, 1.0, 0.90) == 2
    assert P.sample_temperature(logits, 0.0, 0.99) == 1                   # temperature 0 is greedy
    assert P.sample_temperature(logits, 1.0, 0.05, top_k=2) == 1          # token 0 is filtered out
    assert P.sample_temperature(logits, 1.0, 0.05, top_p=0.5) == 1
    assert P.sample_temperature(logits, 1.0, 0.05, min_p=0.5) == 1
    assert P.sample_temperature(logits, 1e-3, 0.999) in (1, 2)
