"""A toy architecture defined in tests/toy_parts.py -- a mixer with state of its own, a
routed feed-forward, an absolute position encoding, a layer that runs twice and a layer
that reads another layer's cache -- is registered, built from a random model folder and
stepped in portions, without a change to the framework's files."""
import os
import random

import pytest

from toy_parts import register_toy, ToyConfig, toy_plain_logits
from helpers import run_trace, trace_whole, trace_portions, trace_mixed, max_rel_err
from tffinfer_b200.config import EngineConfig
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights import write_random_model


def _case(tmp_path):
    register_toy()
    cfg = ToyConfig(architecture="ToyStateLM")
    d = write_random_model(str(tmp_path / "toy"), cfg, seed=5, store_dtype="float32")
    from safetensors.torch import load_file
    w = load_file(os.path.join(d, "model.safetensors"))
    rng = random.Random(1)
    reqs = {f"t{i}": [rng.randrange(cfg.vocab_size) for _ in range(n)] for i, n in enumerate([5, 23, 40, 17])}
    want = {r: toy_plain_logits(t, w, cfg) for r, t in reqs.items()}
    return d, cfg, reqs, want


def _check(runner, reqs, want, tol):
    # one KV group (the attention layer's first run); three state tensors (two runs of layer 0, one of layer 2)
    assert len(runner.groups) == 1 and runner.groups[0].num_layers == 1
    assert len(runner.states) == 3
    assert runner.bindings[4].write is False and runner.bindings[4].group == runner.bindings[1].group
    for steps in (trace_whole(reqs), trace_portions(reqs),
                  trace_mixed(reqs, [len(t) - 4 for t in reqs.values()], 4, 4, 96, 6)):
        got = run_trace(runner, reqs, steps)
        for r in reqs:
            err = max_rel_err(got[r], want[r])
            assert err < tol, (r, err)


def test_toy_architecture_steps_on_cpu_twins(tmp_path):
    from cpu_ops import CpuOps
    d, cfg, reqs, want = _case(tmp_path)
    runner = ModelRunner(d, EngineConfig(dtype="float32", page_size=4, max_cache_tokens=96, max_live_requests=4,
                                         device="cpu"), ops=CpuOps())
    _check(runner, reqs, want, 2e-5)


@pytest.mark.gpu
def test_toy_architecture_steps_on_the_gpu(tmp_path):
    d, cfg, reqs, want = _case(tmp_path)
    runner = ModelRunner(d, EngineConfig(dtype="float32", page_size=4, max_cache_tokens=96, max_live_requests=4,
                                         use_cuda_graphs=False))
    _check(runner, reqs, want, 5e-5)


# ------------------------------------------------------------------ generation with state of fixed size
def _follows_toy_plain(w, cfg, prompt, generated, slack):
    toks = list(prompt)
    for t in generated:
        row = toy_plain_logits(toks, w, cfg)[-1]
        gap = float(row.max() - row[t]) / float(row.abs().max())
        if gap > slack:
            return False
        toks.append(t)
    return True


def _generate_case(tmp_path):
    register_toy()
    cfg = ToyConfig(architecture="ToyStateLM")
    d = write_random_model(str(tmp_path / "toygen"), cfg, seed=9, store_dtype="float32")
    from safetensors.torch import load_file
    w = load_file(os.path.join(d, "model.safetensors"))
    rng = random.Random(2)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (5, 23, 17, 9, 14, 3)]
    return d, cfg, w, prompts


def _check_generation(eng, cfg, w, prompts, slack):
    """Six requests on four state slots and a pool of 48 tokens: slots are handed on from finished
    requests to new ones, and requests give way and are recomputed from position 0.  Each time the
    mixer's state must start from zero, although nobody calls ModelRunner.add_request here."""
    got = eng.generate(prompts, max_new_tokens=12)
    assert eng.scheduler.counters["preemptions"] > 0
    for p, g in zip(prompts, got):
        assert len(g) == 12 and _follows_toy_plain(w, cfg, p, g, slack), (p, g)
    eng.runner.cache.check()
    assert eng.runner.cache.slots.num_free == 4


@pytest.mark.parametrize("native", [True, False], ids=["native", "python"])
def test_a_mixer_with_state_generates_through_the_engine_on_cpu_twins(tmp_path, native):
    from cpu_ops import CpuOps
    from tffinfer_b200.engine import Engine
    d, cfg, w, prompts = _generate_case(tmp_path)
    ecfg = EngineConfig(dtype="float32", page_size=4, max_cache_tokens=48, max_live_requests=4,
                        max_tokens_per_step=6, device="cpu")
    from host_twin import TwinCacheManager
    runner = ModelRunner(d, ecfg, ops=CpuOps(), cache_factory=None if native else TwinCacheManager)
    _check_generation(Engine(runner=runner), cfg, w, prompts, 1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "eager"])
def test_a_mixer_with_state_generates_through_the_engine_on_the_gpu(tmp_path, graphs):
    """With the engine's defaults: decode-only steps are captured and replayed as CUDA graphs, and the step
    that is captured must advance the state once, not twice."""
    from tffinfer_b200.engine import Engine
    d, cfg, w, prompts = _generate_case(tmp_path)
    ecfg = EngineConfig(dtype="float32", page_size=4, max_cache_tokens=48, max_live_requests=4,
                        max_tokens_per_step=6, use_cuda_graphs=graphs)
    eng = Engine(d, ecfg)
    _check_generation(eng, cfg, w, prompts, 1e-5)
    if graphs:
        assert any(st["graphs"] for st in eng.runner._graphs.values()), "no decode step was replayed as a graph"
    eng.runner.ops.check_errors()
