"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees, and decides what happens when pages run out.

The reference has none: ``infer`` walks the sequences one after another, a whole
prompt and then a decode loop (src/core/runtime/InferRuntime.cu:281-292, :348-375);
its request record is ``LLMSeq{_tokens, _is_finished, _eog_token_ids, _current_pos,
_is_prefilled}`` (src/core/runtime/BatchManager.h:19-72) and ``split_simple`` cuts a
flat batch every MAX_BATCH_SIZE tokens (BatchManager.cpp:135-152), the only hint of
a token budget.  Continuous batching is named as future work in its docs.

Policy
  * every step, each running request that is decoding takes one token first; what is
    left of ``max_tokens_per_step`` goes to running requests that still have prompt
    to compute, in order of admission, each ``min(rest of prompt, budget left)``;
    then waiting requests are admitted in arrival order while a slot, budget and
    pages for their first portion are there;
  * when a step's pages cannot all be had, the request admitted LAST is preempted:
    its pages and slot go back, it keeps its tokens (prompt + generated) and moves to
    the FRONT of the waiting queue, to be recomputed from the start; the draw for a
    token depends on (seed, request, index) only, so its output does not change;
  * a request that cannot fit even alone finishes with reason "out_of_memory";
    a prompt longer than the model allows is refused with reason "too_long"
    (the reference truncates with a warning, InferRuntime.cu:399-403).

The decisions of a pass are taken by the host runtime (``plan_step`` of the cache
manager: tffh_plan_step in csrc/host/host_runtime.cpp), which holds the pools and the
block tables, and come back as a list of events that are applied to the request
objects here.  Nothing of it touches the device, so it is tested without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from .. import log
from ..cache import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1      # stands in ``generated`` for a token that a launched step has drawn but the host has not read yet


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    key: int = 0                              # enters the sampling draw; stable across preemptions
    generated: List[int] = field(default_factory=list)
    status: str = WAITING
    finish_reason: Optional[str] = None
    num_preemptions: int = 0
    admitted_at: int = -1                     # admission counter, for choosing a victim

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    def __len__(self) -> int:
        return len(self.prompt) + len(self.generated)

    def token_slice(self, start: int, n: int) -> List[int]:
        """tokens[start:start + n] without joining the prompt and the generated tokens first."""
        lp = len(self.prompt)
        if start >= lp:
            return self.generated[start - lp:start - lp + n]
        if start + n <= lp:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.generated[:start + n - lp]


@dataclass
class PlanEntry:
    request: Request
    start: int                 # position of the first token of this portion
    tokens: List[int]
    samples: bool              # the portion ends at the request's last known token: a token is drawn
    gen_index: Optional[int] = None    # where in ``generated`` the drawn token goes (set when the step is launched)
    reason: Optional[str] = None       # why the request ends with this step, if it does and that is known at launch


@dataclass
class StepPlan:
    entries: List[PlanEntry]
    preempted: List[Request]
    finished: List[Request]    # finished without running (refused or out of memory)

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


@dataclass
class StepOutput:
    request_id: Hashable
    token: Optional[int]
    finished: bool
    finish_reason: Optional[str] = None


class Scheduler:
    def __init__(self, cache: CacheManager, max_tokens_per_step: int, max_model_len: int):
        self.cache = cache
        self.max_tokens_per_step = int(max_tokens_per_step)
        self.max_model_len = int(max_model_len)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._admissions = 0
        self.counters = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}

    # ---------------------------------------------------------------- intake
    def add(self, req: Request) -> None:
        req.status = WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -------------------------------------------------------------- planning
    def _finish(self, req: Request, reason: str, release: bool) -> None:
        if release:
            self.cache.release(req.id)
        if req in self.running:
            self.running.remove(req)
        req.status = FINISHED
        req.finish_reason = reason

    def schedule(self) -> StepPlan:
        """Decides the next step and takes its pages.  The plan's entries are ready to be run; after the
        step, call :meth:`update` with the drawn tokens (or :meth:`commit_launch` and, later,
        :meth:`resolve`)."""
        cache = self.cache
        order = sorted(self.running, key=lambda r: r.admitted_at)
        waiting = list(self.waiting)
        events = cache.plan_step(self.max_tokens_per_step, self.max_model_len,
                                 [r.id for r in order], [len(r) for r in order],
                                 [r.id for r in waiting], [len(r) for r in waiting], [len(r.prompt) for r in waiting])
        by_id = {r.id: r for r in order + waiting}
        preempted: List[Request] = []
        finished: List[Request] = []
        entries: List[PlanEntry] = []
        for kind, name, a, b in events:
            r = by_id[name]
            if kind == cache.EVENT_PREEMPT:
                self.running.remove(r)
                r.status = WAITING
                r.num_preemptions += 1
                self.counters["preemptions"] += 1
                self.waiting.appendleft(r)
                preempted.append(r)
                log.debug("request %r gives way (pages ran out); it will be recomputed from its %d tokens", r.id, len(r))
            elif kind == cache.EVENT_FINISH:
                (self.running if b else self.waiting).remove(r)
                r.status = FINISHED
                r.finish_reason = a
                finished.append(r)
                log.warning("request %r of %d tokens ends without running further: %s", r.id, len(r), a)
            elif kind == cache.EVENT_ADMIT:
                self.waiting.remove(r)
                r.status = RUNNING
                r.admitted_at = self._admissions
                self._admissions += 1
                self.running.append(r)
            else:                                   # EVENT_RUN: a tokens from position b
                entries.append(PlanEntry(r, b, r.token_slice(b, a), samples=(b + a == len(r))))
        return StepPlan(entries, preempted, finished)

    # ---------------------------------------------------------------- update
    def commit_launch(self, plan: StepPlan) -> None:
        """The step has been handed to the device.  Its tokens count as written; every request that
        draws a token gets a PENDING one (the value arrives with :meth:`resolve`); requests that end by
        count end now and give their pages back -- whoever takes those pages runs later on the device."""
        self.counters["steps"] += 1
        self.cache.commit_step([e.request.id for e in plan.entries], [len(e.tokens) for e in plan.entries])
        for e in plan.entries:
            r = e.request
            if len(e.tokens) == 1 and r.generated and e.start >= len(r.prompt):
                self.counters["decode_tokens"] += 1
            else:
                self.counters["prefill_tokens"] += len(e.tokens)
            if not e.samples:
                continue
            if len(r.generated) >= r.params.max_new_tokens:
                e.reason = "length"                    # nothing is drawn
            else:
                r.generated.append(PENDING)
                e.gen_index = len(r.generated) - 1
                if len(r.generated) >= r.params.max_new_tokens:
                    e.reason = "length"
                elif len(r) >= self.max_model_len:
                    e.reason = "max_position"
            if e.reason is not None:
                self._finish(r, e.reason, release=True)

    def resolve(self, plan: StepPlan, drawn: Dict[Hashable, int]) -> List[StepOutput]:
        """The drawn tokens of a launched step have reached the host: they replace the PENDING entries,
        stop tokens end their requests (tokens drawn after a stop token by a step that was already
        launched are dropped)."""
        outs: List[StepOutput] = []
        for r in plan.finished:
            outs.append(StepOutput(r.id, None, True, r.finish_reason))
        for e in plan.entries:
            if not e.samples:
                continue
            r = e.request
            if e.gen_index is None:
                outs.append(StepOutput(r.id, None, True, e.reason))
                continue
            if e.gen_index >= len(r.generated):
                continue                               # drawn after the request's stop token: void
            tok = int(drawn[r.id])
            r.generated[e.gen_index] = tok
            reason = e.reason
            if tok in r.params.eos_token_ids:
                del r.generated[e.gen_index + 1:]
                if r.status != FINISHED:
                    self._finish(r, "stop", release=True)
                r.finish_reason = reason = "stop"
            outs.append(StepOutput(r.id, tok, reason is not None, reason))
        return outs

    def update(self, plan: StepPlan, drawn: Dict[Hashable, int]) -> List[StepOutput]:
        """Launch and result in one: for callers that read the drawn tokens before the next step."""
        self.commit_launch(plan)
        return self.resolve(plan, drawn)

    # ------------------------------------------------------- for pipelined steps
    def has_pending_outside_running(self) -> bool:
        """A waiting request (preempted) still holds a PENDING token: its tokens cannot be sent yet."""
        return any(PENDING in r.generated for r in self.waiting)

    def may_run_out_of_pages(self) -> bool:
        """Every running request may ask for one more page in the next step."""
        return any(p.num_free < len(self.running) for p in self.cache.pools)
