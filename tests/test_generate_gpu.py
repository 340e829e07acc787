"""Generation through the entry point on the GPU: greedy and sampled tokens against the
plain implementation, with and without CUDA graphs, long decoding, preemption."""
import random

import pytest

from helpers import tiny_config, make_model_dir, PAGE_SIZE
from plain_qwen3 import PlainModel, sample_temperature
from tffinfer_b200 import Engine, EngineConfig, SamplingParams
from tffinfer_b200.sampling import uniform_for

pytestmark = pytest.mark.gpu


def _engine(d, name, dtype, **kw):
    kw.setdefault("max_cache_tokens", 1024)
    kw.setdefault("max_live_requests", 4)
    return Engine(d, EngineConfig(dtype=dtype, page_size=PAGE_SIZE[name], **kw))


def _follows_plain(pm, prompt, generated, slack):
    """Every generated token is the plain implementation's choice, or within ``slack`` (relative
    to the largest logit) of it -- a near tie that rounding may flip."""
    toks = list(prompt)
    for t in generated:
        logits = pm.logits(toks)[-1]
        gap = float(logits.max() - logits[t]) / float(logits.abs().max())
        if gap > slack:
            return False
        toks.append(t)
    return True


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_float32_equals_plain(tmp_path, graphs):
    d = make_model_dir(tmp_path, "A")
    pm = PlainModel(d)
    rng = random.Random(5)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (1, 7, 33)]
    eng = _engine(d, "A", "float32", use_cuda_graphs=graphs, max_tokens_per_step=5)
    got = eng.generate(prompts, max_new_tokens=16)
    for p, g in zip(prompts, got):
        assert len(g) == 16 and _follows_plain(pm, p, g, 1e-5)
    eng.runner.ops.check_errors()


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_bfloat16_follows_plain_and_graphs_change_nothing(tmp_path, name):
    d = make_model_dir(tmp_path, name)
    pm = PlainModel(d)
    cfg = tiny_config(name)
    rng = random.Random(6)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (2, 13, 40)]
    outs = []
    for graphs in (False, True):
        eng = _engine(d, name, "bfloat16", use_cuda_graphs=graphs, max_tokens_per_step=16)
        outs.append(eng.generate(prompts, max_new_tokens=24))
        eng.runner.ops.check_errors()
    assert outs[0] == outs[1]
    for p, g in zip(prompts, outs[0]):
        assert _follows_plain(pm, p, g, 3e-2)


def test_decode_graphs_with_unequal_contexts(tmp_path):
    """Heads of 64 in bfloat16 (the split-key decode attention) with contexts from 5 to 610 tokens in one
    batch: decode-only steps are replayed as graphs captured per class of sum / longest context, requests
    finish at different times, and every token still follows the plain implementation."""
    d = make_model_dir(tmp_path, "D")
    pm = PlainModel(d)
    cfg = tiny_config("D")
    rng = random.Random(16)
    lens = (600, 37, 580, 5, 610, 90)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lens]
    news = [6, 14, 9, 14, 4, 12]
    for graphs in (True, False):
        eng = _engine(d, "D", "bfloat16", use_cuda_graphs=graphs, max_tokens_per_step=256, max_cache_tokens=4096,
                      max_live_requests=6)
        ids = [eng.add_request(p, SamplingParams(max_new_tokens=n)) for p, n in zip(prompts, news)]
        while eng.has_unfinished():
            eng.step()
        eng.runner.ops.check_errors()
        for i, p, n in zip(ids, prompts, news):
            g = eng.requests[i].generated
            assert len(g) == n and _follows_plain(pm, p, g, 3e-2)
        if graphs:
            classes = {(b, c) for b, st in eng.runner._graphs.items() for c in st["graphs"]}
            assert len({c for _, c in classes}) >= 2, classes      # more than one class was captured and replayed


def test_temperature_sampling_float32_equals_plain_whatever_the_batching(tmp_path):
    d = make_model_dir(tmp_path, "B")
    pm = PlainModel(d)
    rng = random.Random(7)
    prompts = [[rng.randrange(320) for _ in range(n)] for n in (2, 13, 40, 64)]
    sp = SamplingParams.make(temperature=0.7, seed=42, max_new_tokens=24)
    want = []
    for key, p in enumerate(prompts):
        toks, out = list(p), []
        for i in range(24):
            t = sample_temperature(pm.logits(toks)[-1], 0.7, uniform_for(42, key, i))
            out.append(t); toks.append(t)
        want.append(out)
    together = _engine(d, "B", "float32", max_tokens_per_step=7).generate(prompts, sp)
    alone = _engine(d, "B", "float32", max_live_requests=1, max_tokens_per_step=64).generate(prompts, sp)
    assert together == alone
    agree = sum(int(a == b) for g, w in zip(together, want) for a, b in zip(g, w))
    # a draw that lands within rounding of a boundary of the cumulative distribution may differ
    first_diff_ok = all(g == w or g[:next(i for i in range(24) if g[i] != w[i])] == w[:next(i for i in range(24) if g[i] != w[i])]
                        for g, w in zip(together, want))
    assert first_diff_ok and agree >= 0.9 * 24 * len(prompts)


def test_long_decoding_with_graphs_and_window(tmp_path):
    d = make_model_dir(tmp_path, "C")
    pm = PlainModel(d)
    rng = random.Random(8)
    prompts = [[rng.randrange(311) for _ in range(n)] for n in (5, 21)]
    eng = _engine(d, "C", "float32", use_cuda_graphs=True, max_tokens_per_step=8)
    got = eng.generate(prompts, max_new_tokens=300)
    for p, g in zip(prompts, got):
        assert len(g) == 300
        assert _follows_plain(pm, p, g[:64], 1e-5)
        # the last tokens, far into the decode: the whole sequence once through the plain model
        logits = pm.logits(p + g)
        for i in (250, 275, 299):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[g[i]]) / float(row.abs().max()) < 1e-5
    assert all(pool.num_free == pool.num_pages for pool in eng.runner.cache.pools)


def test_preemption_on_the_gpu_gives_the_same_tokens(tmp_path):
    d = make_model_dir(tmp_path, "A")
    rng = random.Random(9)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (9, 17, 30)]
    big = _engine(d, "A", "float32", max_cache_tokens=512, max_tokens_per_step=6).generate(prompts, max_new_tokens=20)
    small_eng = _engine(d, "A", "float32", max_cache_tokens=64, max_tokens_per_step=6)
    small = small_eng.generate(prompts, max_new_tokens=20)
    assert small == big and small_eng.scheduler.counters["preemptions"] > 0


def test_infer_runtime_and_cli(tmp_path, capsys):
    from tffinfer_b200 import InferRuntime
    from tffinfer_b200.cli import main
    d = make_model_dir(tmp_path, "A")
    rt = InferRuntime()
    rt.load_model([d], use_f16=True, n_ctx=64, page_size=4, max_cache_tokens=256)
    assert rt.init_runtime_context()
    rt.encode([[1, 2, 3], [4, 5]])
    out = []
    rt.infer(6, out)
    assert [len(o) for o in out] == [6, 6]
    assert main([d, "--prompt-ids", "1,2,3", "--prompt-ids", "4,5", "--n-predict", "6", "--page-size", "4",
                 "--max-cache-tokens", "256", "--json"]) == 0
    import json
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["outputs"] == out


@pytest.mark.parametrize("seed", [4, 8, 13, 15, 18, 30, 36])
def test_random_workloads_follow_plain(tmp_path, seed):
    """Prompts, numbers of new tokens, pool size, live requests, token budget, dtype and graphs drawn at
    random (the seeds kept are ones in which pages run out and requests are recomputed): every token
    is the plain implementation's choice and every page comes back."""
    rng = random.Random(1000 + seed)
    name = rng.choice("ABCD")
    dtype = rng.choice(["float32", "bfloat16"])
    cfg = tiny_config(name)
    d = make_model_dir(tmp_path, name)
    pm = PlainModel(d)
    page = PAGE_SIZE[name]
    n = rng.randint(2, 7)
    cap = min(cfg.max_position - 40, 300)
    lens = [rng.randint(1, cap) if rng.random() < 0.5 else rng.randint(1, 30) for _ in range(n)]
    news = [rng.randint(1, 30) for _ in range(n)]
    longest = max(-(-(l + m + 1) // page) * page for l, m in zip(lens, news))
    pool = longest + rng.choice([0, page, longest // 2, 2 * longest])
    live = rng.randint(1, 6)
    budget = rng.choice([2, 5, 16, 64, 256])
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(l)] for l in lens]
    eng = Engine(d, EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=pool, max_live_requests=live,
                                 max_tokens_per_step=budget, use_cuda_graphs=rng.random() < 0.7))
    ids = [eng.add_request(p, SamplingParams(max_new_tokens=m)) for p, m in zip(prompts, news)]
    steps = 0
    while eng.has_unfinished():
        eng.step()
        steps += 1
        assert steps < 5000
    eng.runner.ops.check_errors()
    assert eng.scheduler.counters["preemptions"] > 0
    for i, p, m in zip(ids, prompts, news):
        g = eng.requests[i].generated
        assert len(g) == m and _follows_plain(pm, p, g, 1e-5 if dtype == "float32" else 3e-2)
    assert all(pl.num_free == pl.num_pages for pl in eng.runner.cache.pools)


@pytest.mark.parametrize("seed", [43, 6, 45, 15, 56, 68])
def test_random_workloads_of_wide_models_follow_plain(tmp_path, seed):
    """The same at models with heads of 64 and 128 (the tensor-core products, the two tensor-core attention kernels
    side by side in mixed steps, decode steps replayed as CUDA graphs), in bfloat16: prompts of up to 600 tokens,
    pools in which requests give way, token budgets of 64 to 2048, steps launched ahead or not, drawn at random
    (seeds kept: ones with recomputation, windows, graphs and both ways of stepping among them)."""
    from test_random_configs_gpu import draw_wide_config
    from tffinfer_b200.weights import write_random_model
    cfg, page, _ = draw_wide_config(seed)
    rng = random.Random(5000 + seed)
    d = write_random_model(str(tmp_path / f"wide{seed}"), cfg, seed=seed)
    pm = PlainModel(d, device="cuda")
    n = rng.randint(2, 9)
    lens = [rng.randint(20, 600) if rng.random() < 0.6 else rng.randint(1, 40) for _ in range(n)]
    news = [rng.randint(3, 40) for _ in range(n)]
    longest = max(-(-(l + m + 1) // page) * page for l, m in zip(lens, news))
    pool = longest + rng.choice([0, page, longest // 2, 2 * longest, 4 * longest])
    live = rng.randint(1, 8)
    budget = rng.choice([64, 256, 300, 512, 2048])
    graphs = rng.random() < 0.7
    ahead = rng.random() < 0.7
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(l)] for l in lens]
    eng = Engine(d, EngineConfig(dtype="bfloat16", page_size=page, max_cache_tokens=pool, max_live_requests=live,
                                 max_tokens_per_step=budget, use_cuda_graphs=graphs, async_steps=ahead))
    ids = [eng.add_request(p, SamplingParams(max_new_tokens=m)) for p, m in zip(prompts, news)]
    steps = 0
    while eng.has_unfinished():
        eng.step()
        steps += 1
        assert steps < 20000
    eng.runner.ops.check_errors()
    assert eng.scheduler.counters["preemptions"] > 0
    for i, p, m in zip(ids, prompts, news):
        g = eng.requests[i].generated
        assert len(g) == m
        rows = pm.logits(list(p) + list(g))             # causal: row i is the next-token row of tokens 0..i
        for k, t in enumerate(g):
            row = rows[len(p) - 1 + k]
            gap = float(row.max() - row[t]) / float(row.abs().max())
            assert gap <= 3e-2, f"seed {seed}: request {i} token {k} is {gap:.3e} below the plain maximum"
    assert all(pl.num_free == pl.num_pages for pl in eng.runner.cache.pools)
