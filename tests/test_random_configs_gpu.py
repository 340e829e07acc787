"""Configurations drawn at random (head sizes in steps of 16, any number of heads and groups, widths,
feed-forward sizes and vocabularies that are no power of two and often no multiple of 8, windows on
some layers, tied and untied embeddings, page sizes 4 to 32), each replayed in portions mixed with
decoded tokens in few pages, in 32-bit and in bfloat16, against the plain implementation.  The sizes
decide which kernel runs (tensor-core or FMA products, the head-64/128 attention kernels or the
generic one), so a draw takes paths that the named tiny configurations do not."""
import random

import pytest

from helpers import FULL, SLIDE, trace_mixed, trace_portions, run_trace, first_bad
from plain_qwen3 import PlainModel
from tffinfer_b200.config import Qwen3Config, EngineConfig
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def draw_config(seed: int):
    rng = random.Random(seed)
    d = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128])
    nkv = rng.choice([1, 2, 3, 4])
    nq = nkv * rng.choice([1, 2, 3, 4, 5, 8])
    hidden = rng.choice([40, 72, 100, 136, 200, 264]) if rng.random() < 0.7 else rng.choice([37, 90, 150])
    inter = rng.choice([64, 96, 152, 192, 320]) if rng.random() < 0.7 else rng.choice([70, 131])
    layers = rng.choice([1, 2, 3])
    window = rng.choice([0, 0, 9, 24, 50])
    types = tuple(SLIDE if window and rng.random() < 0.5 else FULL for _ in range(layers))
    if window and SLIDE not in types:
        types = types[:-1] + (SLIDE,)
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=hidden, num_layers=layers, num_heads=nq,
                      num_kv_heads=nkv, head_dim=d, intermediate_size=inter,
                      vocab_size=rng.choice([97, 256, 311, 1000, 1031]),
                      rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]), rope_theta=rng.choice([1e4, 1e6, 5e5]),
                      max_position=1024, tie_word_embeddings=rng.random() < 0.4,
                      sliding_window=window if window else None, layer_types=types).validate()
    page = rng.choice([4, 8, 16, 32])
    prompts = [rng.randint(1, 40), rng.randint(20, 120), rng.randint(2, 300), rng.randint(60, 200)]
    return cfg, page, prompts


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_configuration_matches_plain(tmp_path, seed):
    cfg, page, prompts = draw_config(seed)
    d = write_random_model(str(tmp_path / f"draw{seed}"), cfg, seed=seed)
    rng = random.Random(100 + seed)
    decoded = 6
    reqs = {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + decoded)] for i, n in enumerate(prompts)}
    pm = PlainModel(d)
    want = {r: pm.logits(t) for r, t in reqs.items()}
    most = max(-(-len(t) // page) * page for t in reqs.values())
    pool = most + most // 2
    for dtype in ("float32", "bfloat16"):
        for mode in ("mixed", "portions"):
            if mode == "mixed":
                steps = trace_mixed(reqs, prompts, max_live=3, page_size=page, pool_tokens=pool, chunk=48)
                tokens = pool
            else:
                steps = trace_portions(reqs, sizes=(19, 2, 64, 3, 7))
                tokens = most
            runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=tokens,
                                                 max_live_requests=4, use_cuda_graphs=False))
            for c in runner.kv_caches:
                c.fill_(float("nan"))
            got = run_trace(runner, reqs, steps)
            runner.ops.check_errors()
            for r in reqs:
                bad = first_bad(got[r], want[r], TOL[dtype])
                assert bad is None, (f"seed {seed} {cfg} page {page} {mode}/{dtype}/{r}: first wrong position "
                                     f"{bad[0]} (rel err {bad[1]:.3e}) of {len(reqs[r])}")


def draw_wide_config(seed: int):
    """Heads of 64 or 128, 1 to 8 query heads a key/value head, widths up to 1536 and prompts of several hundred
    tokens: the tensor-core products in their prompt-sized forms, the projection with its epilogue, and the two
    tensor-core attention kernels over several tiles."""
    rng = random.Random(seed)
    d = rng.choice([64, 128, 128])
    nkv = rng.choice([1, 2, 4, 8])
    group = rng.choice([1, 2, 3, 4, 5, 6, 8])
    hidden = rng.choice([256, 512, 1024, 1536, 776])
    inter = rng.choice([512, 1024, 1536, 704, 1032])
    window = rng.choice([0, 0, 0, 70, 200])
    types = tuple(SLIDE if window and (i == 1 or rng.random() < 0.5) else FULL for i in range(2))
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=hidden, num_layers=2, num_heads=nkv * group,
                      num_kv_heads=nkv, head_dim=d, intermediate_size=inter, vocab_size=rng.choice([1000, 2311, 4096]),
                      rms_norm_eps=1e-6, rope_theta=rng.choice([1e4, 1e6]), max_position=2048,
                      tie_word_embeddings=rng.random() < 0.3, sliding_window=window if window else None,
                      layer_types=types).validate()
    page = rng.choice([8, 16, 16, 32, 64])
    prompts = [rng.randint(257, 900), rng.randint(130, 520), rng.randint(20, 300), rng.randint(300, 640)]
    return cfg, page, prompts


@pytest.mark.parametrize("seed", [165, 299, 37, 7, 23, 318, 401, 58])
def test_random_wide_configuration_in_bfloat16_matches_plain_run_after_run(tmp_path, seed):
    """Whole prompts with decoded tokens replayed as CUDA graphs, portions of 2 to 520 tokens, and portions mixed
    with decoded tokens in few pages; each cut twice in the same process, since kernels that follow each other
    without the pauses of first launches have shown an ordering fault that a first run hid.  The bar is 3e-2:
    500 draws of this kind gave 0.008 at the median position and never more than 0.019 at the worst one."""
    cfg, page, prompts = draw_wide_config(seed)
    d = write_random_model(str(tmp_path / f"wide{seed}"), cfg, seed=seed)
    rng = random.Random(1000 + seed)
    decoded = 5
    reqs = {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + decoded)] for i, n in enumerate(prompts)}
    pm = PlainModel(d, device="cuda")
    want = {r: pm.logits(t) for r, t in reqs.items()}
    del pm
    most = max(-(-len(t) // page) * page for t in reqs.values())
    total = sum(-(-len(t) // page) * page for t in reqs.values())
    for mode in ("whole", "portions", "mixed"):
        for again in range(2):
            if mode == "whole":
                steps = [([(r, 0, n)], []) for r, n in zip(reqs, prompts)]
                for k in range(decoded):
                    steps.append(([(r, n + k, 1) for r, n in zip(reqs, prompts)], list(reqs) if k == decoded - 1 else []))
                pool, graphs = total, True
            elif mode == "portions":
                steps = trace_portions(reqs, sizes=(300, 2, 131, 520, 3, 257, 64))
                pool, graphs = most, False
            else:
                pool, graphs = most + most // 2, False
                steps = trace_mixed(reqs, prompts, max_live=3, page_size=page, pool_tokens=pool, chunk=300, seed=seed + again)
            runner = ModelRunner(d, EngineConfig(dtype="bfloat16", page_size=page, max_cache_tokens=pool,
                                                 max_live_requests=4, use_cuda_graphs=graphs))
            for c in runner.kv_caches:
                c.fill_(float("nan"))
            got = run_trace(runner, reqs, steps, poison=True)
            runner.ops.check_errors()
            for r in reqs:
                bad = first_bad(got[r], want[r], 3e-2)
                assert bad is None, (f"seed {seed} {cfg} page {page} {mode} run {again} {r}: first wrong position "
                                     f"{bad[0]} (rel err {bad[1]:.3e}) of {len(reqs[r])}")
            del runner
