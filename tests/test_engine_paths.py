"""Paths of the entry point that ordinary generation seldom takes, each with the kernels' plain twins on
the CPU and with the CUDA kernels: steps launched before the tokens of the step before have been read
(and the same without that), a stop token that is found one step late, a request aborted while a step
is in flight, and a repetition penalty (which makes the host read every step's tokens first)."""
import random

import pytest
import torch

from helpers import make_model_dir, tiny_config, PAGE_SIZE
from plain_qwen3 import PlainModel, sample_greedy, sample_temperature, repetition_penalty
from tffinfer_b200.config import EngineConfig
from tffinfer_b200.engine import Engine, ModelRunner
from tffinfer_b200.sampling import SamplingParams, uniform_for

BACKENDS = ["cpu_twins", pytest.param("cuda", marks=pytest.mark.gpu)]


def _engine(tmp_path, name, backend, **kw):
    d = make_model_dir(tmp_path, name)
    kw.setdefault("max_cache_tokens", 512)
    kw.setdefault("max_live_requests", 4)
    if backend == "cpu_twins":
        from cpu_ops import CpuOps
        ecfg = EngineConfig(dtype="float32", page_size=PAGE_SIZE[name], device="cpu", **kw)
        return d, Engine(runner=ModelRunner(d, ecfg, ops=CpuOps()))
    return d, Engine(d, EngineConfig(dtype="float32", page_size=PAGE_SIZE[name], **kw))


def _prompts(name, lens, seed):
    rng = random.Random(seed)
    v = tiny_config(name).vocab_size
    return [[rng.randrange(v) for _ in range(n)] for n in lens]


def _plain_generate(pm, prompt, n, params=None, key=0):
    toks, out = list(prompt), []
    for i in range(n):
        logits = pm.logits(toks)[-1].float()
        if params is not None and params.repetition_penalty != 1.0:
            logits = repetition_penalty(logits, toks, params.repetition_penalty)
        if params is None or params.is_greedy:
            t = sample_greedy(logits)
        else:
            t = sample_temperature(logits, params.temperature, uniform_for(params.seed, key, i),
                                   params.top_k, params.top_p, params.min_p)
        out.append(t)
        toks.append(t)
        if params is not None and t in params.eos_token_ids:
            break
    return out


def _drain(eng):
    """Steps until nothing is left; returns the outputs in the order they were handed out."""
    outs, steps = [], 0
    while eng.has_unfinished():
        outs += eng.step()
        steps += 1
        assert steps < 2000
    return outs


@pytest.mark.parametrize("backend", BACKENDS)
def test_outputs_do_not_depend_on_whether_steps_are_launched_ahead(tmp_path, backend):
    prompts = _prompts("B", (2, 13, 40, 21, 7), 3)
    sp = SamplingParams.make(temperature=0.8, seed=5, max_new_tokens=12)
    results, streams = [], []
    for ahead in (True, False):
        # five requests on four slots and a pool that does not hold them all: admissions wait, requests give way
        d, eng = _engine(tmp_path, "B", backend, async_steps=ahead, max_tokens_per_step=9, max_cache_tokens=136)
        ids = [eng.add_request(p, sp, key=i) for i, p in enumerate(prompts)]
        outs = _drain(eng)
        results.append([eng.requests[i].generated for i in ids])
        streams.append({i: [o.token for o in outs if o.request_id == i and o.token is not None] for i in ids})
        assert all(pool.num_free == pool.num_pages for pool in eng.runner.cache.pools)
    assert results[0] == results[1]
    pm = PlainModel(d)
    assert results[0] == [_plain_generate(pm, p, 12, sp, key=i) for i, p in enumerate(prompts)]
    for ids_stream, res in zip(streams, results):       # what step() hands out is what the requests hold
        assert [ids_stream[i] for i in sorted(ids_stream)] == res


@pytest.mark.parametrize("ahead", [True, False], ids=["ahead", "in_turn"])
@pytest.mark.parametrize("backend", BACKENDS)
def test_a_stop_token_found_one_step_late_voids_the_token_drawn_after_it(tmp_path, backend, ahead):
    d, eng = _engine(tmp_path, "A", backend, async_steps=ahead, max_tokens_per_step=16)
    pm = PlainModel(d)
    prompts = _prompts("A", (7, 19, 4), 11)
    # sampled at temperature 1 (greedy output of a random model soon repeats itself); the draws are a
    # function of (seed, request, index), so the plain implementation can follow them
    base = dict(temperature=1.0, seed=7, max_new_tokens=16)
    free_run = [_plain_generate(pm, p, 16, SamplingParams.make(**base), key=i) for i, p in enumerate(prompts)]
    # a stop token for the second request that the plain implementation's own output meets mid-run
    k = next(i for i in range(4, 15) if free_run[1][i] not in free_run[1][:i])
    stop = free_run[1][k]
    params = [SamplingParams.make(**base), SamplingParams.make(**base, eos_token_ids=(stop,)), SamplingParams.make(**base)]
    ids = [eng.add_request(p, sp, key=i) for i, (p, sp) in enumerate(zip(prompts, params))]
    outs = _drain(eng)
    got = [eng.requests[i] for i in ids]
    assert got[0].generated == free_run[0] and got[2].generated == free_run[2]
    assert got[1].generated == free_run[1][:k + 1] and got[1].finish_reason == "stop"
    assert got[0].finish_reason == got[2].finish_reason == "length"
    mine = [o for o in outs if o.request_id == ids[1]]
    assert [o.token for o in mine] == free_run[1][:k + 1], "the token drawn after the stop token must not be handed out"
    assert [o.finished for o in mine] == [False] * k + [True] and mine[-1].finish_reason == "stop"
    eng.runner.cache.check()
    assert all(pool.num_free == pool.num_pages for pool in eng.runner.cache.pools)
    assert eng.runner.cache.slots.num_free == 4


@pytest.mark.parametrize("backend", BACKENDS)
def test_abort_with_a_step_in_flight(tmp_path, backend):
    d, eng = _engine(tmp_path, "A", backend, async_steps=True, max_tokens_per_step=32)
    pm = PlainModel(d)
    prompts = _prompts("A", (9, 17, 5), 13)
    ids = [eng.add_request(p, SamplingParams(max_new_tokens=14), key=i) for i, p in enumerate(prompts)]
    outs = []
    for _ in range(5):
        outs += eng.step()
    assert eng._inflight is not None                       # a step has been launched and not read
    victim = eng.requests[ids[1]]
    before = len([o for o in outs if o.request_id == ids[1]])
    eng.abort(ids[1])
    assert victim.status == "finished" and victim.finish_reason == "abort" and ids[1] not in eng.requests
    assert eng._inflight is None
    eng.abort(ids[1])                                      # a second abort, and one of an unknown id, do nothing
    eng.abort("nobody")
    outs += _drain(eng)
    assert len([o for o in outs if o.request_id == ids[1]]) == before, "nothing is handed out for an aborted request"
    for i in (0, 2):
        assert eng.requests[ids[i]].generated == _plain_generate(pm, prompts[i], 14)
        assert [o.token for o in outs if o.request_id == ids[i]] == eng.requests[ids[i]].generated
    eng.runner.cache.check()
    assert all(pool.num_free == pool.num_pages for pool in eng.runner.cache.pools)
    assert eng.runner.cache.slots.num_free == 4
    # a waiting request can be aborted too, and the engine goes on
    a = eng.add_request(prompts[0], SamplingParams(max_new_tokens=3))
    b = eng.add_request(prompts[2], SamplingParams(max_new_tokens=3))
    eng.abort(a)
    _drain(eng)
    assert eng.requests[b].generated == _plain_generate(pm, prompts[2], 3)


@pytest.mark.parametrize("backend", BACKENDS)
def test_repetition_penalty_through_generate_equals_the_plain_sampler(tmp_path, backend):
    d, eng = _engine(tmp_path, "B", backend, max_tokens_per_step=11)
    pm = PlainModel(d)
    prompts = _prompts("B", (3, 30, 12), 17)
    plist = [SamplingParams(max_new_tokens=14, repetition_penalty=1.8),
             SamplingParams.make(temperature=0.9, seed=3, max_new_tokens=14, repetition_penalty=1.3, top_k=40),
             SamplingParams(max_new_tokens=14)]
    got = eng.generate(prompts, plist)
    want = [_plain_generate(pm, p, 14, sp, key=i) for i, (p, sp) in enumerate(zip(prompts, plist))]
    assert got == want
    # the penalty changed something: without it the first request repeats itself
    assert got[0] != _plain_generate(pm, prompts[0], 14)
    assert len(set(got[0])) == len(got[0]) or len(set(got[0])) > len(set(_plain_generate(pm, prompts[0], 14)))
