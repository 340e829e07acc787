"""Opt-in timing of every kernel call of a step, and a Chrome trace of it.

The reference dumps its Taskflow graph to ``task_flow_graph.json`` on every run and has the lines of a
``tf::ChromeObserver`` commented out (src/taskgraph/src/TaskFlowSchedule.cu:12-37); its only timing is whole
seconds around the decode loop (src/core/runtime/InferRuntime.cu:347,377-378).  Here nothing is recorded
unless asked for:

    with KernelTrace(runner.ops) as trace:
        runner.step(entries)                 # kernel by kernel (EngineConfig.use_cuda_graphs=False)
    for name, calls, ms in trace.summary():  # per kind of call, device time between its two events
        ...
    trace.write_chrome_trace("step.json")    # open in chrome://tracing or Perfetto

Inside the ``with`` every method of the kernel library that launches work records a CUDA event before and
after it on the current stream.  Calls made from inside another traced call (the product and the
norm/rotation kernel inside ``qkv_project``) are nested in the trace; the summary counts only the innermost
ones, so that nothing is counted twice.  The events serialise nothing, but a step replayed as a CUDA graph
makes no calls to trace: switch graphs off for the steps that are traced.  Times include the gaps between
the launches of a call, and under programmatic dependent launch a kernel's prologue may overlap its
predecessor: compare shares, and use a profiler for absolute figures.
"""
from __future__ import annotations

import json
from typing import List, Tuple

import torch

TRACED = ("embed", "rmsnorm", "gemm", "gemm_simt", "gemm_tc", "zero_f32", "gather_tokens", "swiglu", "gemm_swiglu",
          "qkv_project", "qk_norm_rope_kv_write", "attention", "attention_bf16", "attention_generic", "argmax",
          "sample", "repetition_penalty", "reset_state_slots", "logit_transform", "rope_table")


class KernelTrace:
    def __init__(self, ops):
        self.ops = ops
        self.records = []            # [name, depth, start event, end event, has children, detail]
        self._stack = []
        self._saved = {}

    def _wrap(self, name, fn):
        def traced(*args, **kwargs):
            rec = [name, len(self._stack), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
                   False, _detail(args)]
            if self._stack:
                self._stack[-1][4] = True
            self.records.append(rec)
            self._stack.append(rec)
            rec[2].record()
            try:
                return fn(*args, **kwargs)
            finally:
                rec[3].record()
                self._stack.pop()
        return traced

    def __enter__(self):
        for name in TRACED:
            fn = getattr(self.ops, name, None)
            if fn is not None:
                self._saved[name] = fn
                setattr(self.ops, name, self._wrap(name, fn))
        return self

    def __exit__(self, *exc):
        for name in self._saved:
            delattr(self.ops, name)          # the class's own method shows again
        self._saved = {}
        return False

    def timed(self) -> List[Tuple[str, int, float, float, bool, str]]:
        """(name, depth, start ms since the first call, duration ms, innermost, detail) of every call."""
        if not self.records:
            return []
        torch.cuda.synchronize()
        first = self.records[0][2]
        return [(name, depth, first.elapsed_time(a), a.elapsed_time(b), not has_children, detail)
                for name, depth, a, b, has_children, detail in self.records]

    def summary(self) -> List[Tuple[str, int, float]]:
        """(name, calls, total ms) of the innermost calls, largest total first."""
        agg = {}
        for name, _, _, ms, innermost, _ in self.timed():
            if innermost:
                c, t = agg.get(name, (0, 0.0))
                agg[name] = (c + 1, t + ms)
        return sorted(((n, c, t) for n, (c, t) in agg.items()), key=lambda x: -x[2])

    def write_chrome_trace(self, path: str) -> None:
        events = [{"name": name, "ph": "X", "pid": 0, "tid": 0, "ts": round(start * 1000.0, 3),
                   "dur": round(ms * 1000.0, 3), "args": {"shapes": detail}}
                  for name, depth, start, ms, _, detail in self.timed()]
        with open(path, "w") as f:
            json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)


def _detail(args) -> str:
    return " ".join("x".join(str(d) for d in a.shape) for a in args if isinstance(a, torch.Tensor))[:120]
