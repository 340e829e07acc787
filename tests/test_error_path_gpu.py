"""The way from a bounded wait that runs out inside a kernel to the caller, and the opt-in timers.

Every wait of the tcgen05 kernels on an mbarrier gives up after a fixed number of polls, raises the
library's error word and returns; in a correct run that never happens.  The library's self-test kernel
makes it happen without any fault: it waits, with a limit of a few thousand polls, on a barrier at which
nobody arrives.  The kernel returns by itself and the context stays usable."""
import json
import random

import pytest
import torch

from helpers import make_model_dir, PAGE_SIZE
from tffinfer_b200 import Engine, EngineConfig, SamplingParams
from tffinfer_b200.kernels.library import CudaKernels, KernelError
from tffinfer_b200.kernels.trace import KernelTrace

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_raises_the_error_word_and_the_word_clears():
    ops = CudaKernels()
    ops.check_errors()                                   # nothing pending
    ops.selftest_bounded_wait(arrive=True)               # the barrier's phase completes: the wait returns at once
    ops.check_errors()
    ops.selftest_bounded_wait(arrive=False, max_polls=3000)
    with pytest.raises(KernelError, match="bounded wait"):
        ops.check_errors()
    ops.check_errors()                                   # reading the word cleared it
    # the context is as usable as before
    x = torch.arange(8, device="cuda", dtype=torch.float32)
    assert float((x * 2).sum()) == 56.0


def test_the_error_word_reaches_engine_step_with_the_tokens_of_its_step(tmp_path):
    d = make_model_dir(tmp_path, "D")
    rng = random.Random(3)
    eng = Engine(d, EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE["D"], max_cache_tokens=1024, max_live_requests=4))
    for n in (20, 7):
        eng.add_request([rng.randrange(264) for _ in range(n)], SamplingParams(max_new_tokens=12))
    for _ in range(3):
        eng.step()
    eng.runner.ops.check_errors()
    # a kernel of the next step "stalls": the word is raised on the stream before that step's tokens are copied out
    eng.runner.ops.selftest_bounded_wait(arrive=False, max_polls=2000)
    with pytest.raises(KernelError, match="bounded wait"):
        for _ in range(3):                               # launched ahead: the step that reads those tokens raises
            eng.step()
    eng.runner.ops.check_errors()                        # cleared; the device still answers
    torch.cuda.synchronize()


def test_kernel_trace_times_every_call_of_a_step_and_writes_a_chrome_trace(tmp_path):
    d = make_model_dir(tmp_path, "D")
    eng = Engine(d, EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE["D"], max_cache_tokens=1024, max_live_requests=4,
                                 use_cuda_graphs=False))
    rng = random.Random(4)
    prompts = [[rng.randrange(264) for _ in range(n)] for n in (40, 9)]
    plain = eng.generate(prompts, max_new_tokens=4)
    launches = eng.runner.ops.launches
    with KernelTrace(eng.runner.ops) as trace:
        traced = eng.generate(prompts, max_new_tokens=4)
    assert traced == plain                               # tracing changes nothing
    summary = trace.summary()
    names = {n for n, _, _ in summary}
    assert {"embed", "rmsnorm", "argmax"} <= names and names & {"gemm_tc", "gemm_simt"} and \
        names & {"attention_bf16", "attention_generic"}
    assert all(ms >= 0 for _, _, ms in summary)
    innermost = sum(c for _, c, _ in summary)
    assert 0 < innermost <= eng.runner.ops.launches - launches
    path = tmp_path / "step.json"
    trace.write_chrome_trace(str(path))
    events = json.loads(path.read_text())["traceEvents"]
    assert len(events) == len(trace.records) and all(e["ph"] == "X" and e["dur"] >= 0 for e in events)
    # outside the ``with`` nothing is recorded any more
    n = len(trace.records)
    eng.generate(prompts[:1], max_new_tokens=2)
    assert len(trace.records) == n
