"""The Qwen3-8B shape whole -- 36 layers of width 4096, 32 query heads on 8 key/value heads of 128,
feed-forward 12288, vocabulary 151936, untied output matrix -- in true 32-bit and in bfloat16 against the
plain implementation, on prompts of at most 64 tokens in three ways of cutting them.  The plain
implementation runs in float64 on the GPU (the formulas are those of tests/plain_qwen3.py; 8.2 G
parameters in float64 are 66 GB) and the engine is fed from the same dictionary of random tensors."""
import random

import pytest
import torch

from helpers import trace_tail_decode, trace_portions, trace_mixed, run_trace, first_bad
import plain_qwen3 as plain
from tffinfer_b200.config import Qwen3Config, EngineConfig
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights import random_tensors_on_device

pytestmark = pytest.mark.gpu

# Largest |difference| over the row's largest |logit|.  The tiny and the two-layer tests use 2e-5 in float32 and
# 4e-2 in bfloat16; here the sums are long and the layers many, and the bars follow from the arithmetic.  A float32 sum of K products added one after the other (the 32-bit product keeps one order of
# summation per output element, whatever the batch) carries a rounding error of about sqrt(K) * 2^-24 of its
# size; the two products of each layer that feed the residual stream (output projection, down projection) add
# errors that are independent from layer to layer, so after L layers the stream, and with it the logits, is off
# by about sqrt(2 L) * sqrt(K) * 2^-24 of its size: K = 12288, L = 36 give 5.6e-5.
#
# bfloat16: every layer rounds the rows it hands from kernel to kernel (normalised rows, queries, keys, values, the
# attention's output, the activation) to 8 bits of mantissa, 2^-9 of their size each; these errors are independent
# from layer to layer, so the logits are off by c * sqrt(L) * 2^-9 of their size.  Measured on this model with
# random weights: c = 2.7 for the mean over positions (0.0105 at 4 layers, 0.0275 at 36) and 2.9 to 4.3 for the
# largest of about 130 positions.  The bars are set at 1.3 times these: the mean over a request's positions may
# reach 3.5 * sqrt(L) * 2^-9 = 4.1e-2 and one position 5.4 * sqrt(L) * 2^-9 = 6.3e-2.  A fault of the cache or the
# batch (a wrong key, a missing page) moves a logit row by its own size, ten times these bars.
K_LONGEST, LAYERS = 12288, 36
TOL = {"float32": (2 * LAYERS) ** 0.5 * K_LONGEST ** 0.5 * 2.0 ** -24, "bfloat16": 5.4 * LAYERS ** 0.5 * 2.0 ** -9}
MEAN_TOL = {"float32": TOL["float32"], "bfloat16": 3.5 * LAYERS ** 0.5 * 2.0 ** -9}
PAGE = 16
LENGTHS = [64, 23, 41]
PROMPTS = [56, 15, 33]          # the rest of each sequence is fed as decoded tokens


@pytest.fixture(scope="module")
def whole_8b():
    total = torch.cuda.get_device_properties(0).total_memory
    if total < 140 * 2 ** 30:
        pytest.skip("needs a device with 140 GB (float64 copy of the weights beside the bfloat16 one)")
    cfg = Qwen3Config(architecture="Qwen3ForCausalLM", hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8,
                      head_dim=128, intermediate_size=12288, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6,
                      max_position=40960, tie_word_embeddings=False, layer_types=("full_attention",) * 36).validate()
    tensors = random_tensors_on_device(cfg, 3, "cuda", "bfloat16", norm_noise=0.1)
    rng = random.Random(17)
    reqs = {f"q{i}": [rng.randrange(cfg.vocab_size) for _ in range(n)] for i, n in enumerate(LENGTHS)}
    w64 = {k: v.to(torch.float64) for k, v in tensors.items()}
    pcfg = dict(hidden=4096, layers=36, heads=32, kv_heads=8, head_dim=128, inter=12288, vocab=151936, eps=1e-6,
                theta=1e6, max_pos=40960, tied=False, windows=[0] * 36)
    want = {r: plain.forward_logits(t, w64, pcfg).float().cpu() for r, t in reqs.items()}
    del w64
    torch.cuda.empty_cache()
    yield cfg, tensors, reqs, want
    del tensors
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_whole_8b_shape_matches_plain_in_three_cuts(whole_8b, dtype):
    cfg, tensors, reqs, want = whole_8b
    most = max(-(-len(t) // PAGE) * PAGE for t in reqs.values())
    pool = most + most // 2
    runner = ModelRunner(config=cfg, tensors=tensors,
                         engine_config=EngineConfig(dtype=dtype, page_size=PAGE, max_cache_tokens=pool,
                                                    max_live_requests=4, max_model_len=256, use_cuda_graphs=False))
    for c in runner.kv_caches:
        c.fill_(float("nan"))
    cuts = {"tail": trace_tail_decode(reqs, tail=8),
            "portions": trace_portions(reqs, sizes=(17, 2, 9, 31, 3)),
            "mixed": trace_mixed(reqs, PROMPTS, max_live=3, page_size=PAGE, pool_tokens=pool, chunk=12)}
    for mode, steps in cuts.items():
        stats = {}
        got = run_trace(runner, reqs, steps, poison=True, stats=stats)
        for r in reqs:
            bad = first_bad(got[r], want[r], TOL[dtype])
            assert bad is None, (f"{mode}/{dtype}/{r}: first wrong position {bad[0]} (rel err {bad[1]:.3e}) "
                                 f"of {len(reqs[r])}")
            scale = want[r].abs().amax(dim=-1, keepdim=True)
            mean = float(((got[r].double() - want[r].double()).abs() / scale).amax(dim=-1).mean())
            assert mean <= MEAN_TOL[dtype], f"{mode}/{dtype}/{r}: mean rel err over positions {mean:.3e}"
        if mode == "mixed":
            assert stats["pages_reused"] > 0
    runner.ops.check_errors()
    del runner
    torch.cuda.empty_cache()
