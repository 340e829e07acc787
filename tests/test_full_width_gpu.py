"""The engine at the layer sizes of an 8B model (width 4096, 32 query heads on 8 key/value
heads of 128, feed-forward 12288) and of a 14B model (width 5120, 40 query heads, feed-forward
17408), two layers and an odd vocabulary, against the plain
implementation (which runs in float64 on the GPU here, the formulas being the same): the
kernels take other paths at these sizes than at the tiny ones (tensor-core products with
every epilogue, the head-128 attention kernels, split keys)."""
import random

import pytest
import torch

from helpers import trace_tail_decode, trace_portions, trace_mixed, run_trace, first_bad
from plain_qwen3 import PlainModel
from tffinfer_b200.config import Qwen3Config, EngineConfig, read_config_json
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

# bfloat16: two layers at these widths give 0.009 at the median position and 0.012 at the worst (measured, run after run,
# the order of the float32 adds of split products moving single logits by up to 0.005 of the largest);
# a prompt attention that dropped one key block's probabilities for a few rows gave 0.06 there
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
PAGE = 16
PROMPTS = [300, 45, 131]
DECODED = 8


SHAPES = {"8b": (4096, 32, 12288, 32003), "14b": (5120, 40, 17408, 15013)}


@pytest.fixture(scope="module", params=list(SHAPES))
def wide(request, tmp_path_factory):
    hidden, heads, inter, vocab = SHAPES[request.param]
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=hidden, num_layers=2, num_heads=heads,
                      num_kv_heads=8, head_dim=128, intermediate_size=inter, vocab_size=vocab,
                      rms_norm_eps=1e-6, rope_theta=1e6, max_position=4096, tie_word_embeddings=False,
                      layer_types=("full_attention",) * 2).validate()
    d = write_random_model(str(tmp_path_factory.mktemp("wide")), cfg, seed=5)
    rng = random.Random(11)
    reqs = {f"w{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + DECODED)] for i, n in enumerate(PROMPTS)}
    pm = PlainModel(d, device="cuda")
    want = {r: pm.logits(t) for r, t in reqs.items()}
    del pm
    torch.cuda.empty_cache()
    return d, reqs, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["tail", "portions", "mixed"])
def test_full_width_layers_match_plain(wide, mode, dtype):
    d, reqs, want = wide
    most = max(-(-len(t) // PAGE) * PAGE for t in reqs.values())
    pool = most + most // 2 if mode == "mixed" else most
    if mode == "tail":
        steps = trace_tail_decode(reqs, tail=DECODED)
    elif mode == "portions":
        steps = trace_portions(reqs, sizes=(70, 2, 33, 128, 3, 17))
    else:
        steps = trace_mixed(reqs, PROMPTS, max_live=3, page_size=PAGE, pool_tokens=pool, chunk=64)
    runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=PAGE, max_cache_tokens=pool, max_live_requests=4,
                                         use_cuda_graphs=False))
    for c in runner.kv_caches:
        c.fill_(float("nan"))
    got = run_trace(runner, reqs, steps)
    for r in reqs:
        bad = first_bad(got[r], want[r], TOL[dtype])
        assert bad is None, (f"{mode}/{dtype}/{r}: first wrong position {bad[0]} (rel err {bad[1]:.3e}) "
                             f"of {len(reqs[r])}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_decode_steps_replayed_as_cuda_graphs_match_plain(wide, dtype):
    """The decode path the benchmark measures (device arrays of fixed size, CUDA-graph replay, split keys)
    at the full layer widths: every prompt in one step, then the three requests decode together."""
    d, reqs, want = wide
    pool = sum(-(-len(t) // PAGE) * PAGE for t in reqs.values())
    runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=PAGE, max_cache_tokens=pool, max_live_requests=4,
                                         use_cuda_graphs=True))
    for c in runner.kv_caches:
        c.fill_(float("nan"))
    steps = [([(r, 0, n)], []) for r, n in zip(reqs, PROMPTS)]
    for k in range(DECODED):
        steps.append(([(r, n + k, 1) for r, n in zip(reqs, PROMPTS)], list(reqs) if k == DECODED - 1 else []))
    got = run_trace(runner, reqs, steps, poison=True)
    assert any(st["graphs"] for st in runner._graphs.values())
    for r in reqs:
        bad = first_bad(got[r], want[r], TOL[dtype])
        assert bad is None, f"{dtype}/{r}: first wrong position {bad[0]} (rel err {bad[1]:.3e}) of {len(reqs[r])}"


def test_full_width_prompt_step_run_again_in_a_warm_process_matches_plain(wide):
    """The same prompts through fresh runners three times in one process.  From the second time on the kernels
    follow each other without the pauses of first launches, and a prompt attention whose warps could overtake
    one another (a product issued before a slower warp's probabilities were written) gave the last tokens
    of the 300-token prompt wrong logits from then on, never the first time."""
    d, reqs, want = wide
    most = max(-(-len(t) // PAGE) * PAGE for t in reqs.values())
    steps = trace_tail_decode(reqs, tail=DECODED)
    for again in range(3):
        runner = ModelRunner(d, EngineConfig(dtype="bfloat16", page_size=PAGE, max_cache_tokens=most,
                                             max_live_requests=4, use_cuda_graphs=False))
        got = run_trace(runner, reqs, steps)
        for r in reqs:
            bad = first_bad(got[r], want[r], TOL["bfloat16"])
            assert bad is None, (f"run {again}: {r}: first wrong position {bad[0]} (rel err {bad[1]:.3e}) "
                                 f"of {len(reqs[r])}")
        del runner


def test_small_portions_behind_a_long_context_match_plain(wide):
    """2,304 tokens of a prompt in two steps, then portions of 12 and of 40 tokens and two single tokens: the small
    portions behind more than 2,048 keys take the attention of 64-row tiles with the key range cut into shares
    (CudaKernels.portion_splits), the rest the kernels they always took."""
    d, _, _ = wide
    cfg = Qwen3Config.from_json_dict(read_config_json(d))
    rng = random.Random(23)
    toks = [rng.randrange(cfg.vocab_size) for _ in range(2304 + 12 + 40 + 2)]
    reqs = {"long": toks}
    pm = PlainModel(d, device="cuda")
    want = pm.logits(toks)
    del pm
    torch.cuda.empty_cache()
    steps = [([("long", 0, 1152)], []), ([("long", 1152, 1152)], []), ([("long", 2304, 12)], []),
             ([("long", 2316, 40)], []), ([("long", 2356, 1)], []), ([("long", 2357, 1)], ["long"])]
    pool = -(-len(toks) // PAGE) * PAGE
    for dtype in ("bfloat16", "float32"):
        runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=PAGE, max_cache_tokens=pool, max_live_requests=2,
                                             use_cuda_graphs=False))
        assert runner.ops.portion_splits(1, 12, 2316, cfg.num_heads, cfg.num_kv_heads) > 1
        for c in runner.kv_caches:
            c.fill_(float("nan"))
        got = run_trace(runner, reqs, steps)
        bad = first_bad(got["long"][2304:], want[2304:], TOL[dtype])
        assert bad is None, f"{dtype}: first wrong position {2304 + bad[0]} (rel err {bad[1]:.3e})"
        del runner
