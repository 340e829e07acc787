"""The Python entry point: model folder in, token ids out.

``Engine`` owns a ModelRunner (step function, cache, kernels), a Scheduler and a
Sampler.  ``InferRuntime`` offers the same through the names of the reference's
``LLMInferRuntime`` (src/core/runtime/InferRuntime.h:32-266; used by test/main.cu:18-67):
``load_model`` -> ``init_runtime_context`` -> ``encode`` -> ``infer(n_predict, out)``.
The reference tokenises text itself; this engine is tokens in, tokens out, so
``encode`` takes lists of token ids.
"""
from __future__ import annotations

import itertools
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from .. import log
from ..config import EngineConfig
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Scheduler, Request, StepOutput, PENDING


class Engine:
    def __init__(self, model_dir: Optional[str] = None, engine_config: Optional[EngineConfig] = None, *,
                 runner: Optional[ModelRunner] = None, **kwargs):
        """``kwargs`` are fields of EngineConfig (dtype, page_size, max_cache_tokens,
        max_live_requests, max_tokens_per_step, ...) when no ``engine_config`` is given."""
        if runner is None:
            ecfg = engine_config or EngineConfig(**kwargs)
            runner = ModelRunner(model_dir, ecfg)
        self.runner = runner
        self.ecfg = runner.ecfg
        self.scheduler = Scheduler(runner.cache, self.ecfg.max_tokens_per_step, runner.max_model_len)
        self.sampler = Sampler(runner.ops, runner.device)
        self.requests: Dict[Hashable, Request] = {}
        self._ids = itertools.count()
        self.step_events = None      # optional (start, end) CUDA events recorded around the step's device work
        self._inflight = None        # the step that has been launched and whose drawn tokens have not been read
        self._host_tokens = [None, None]   # pinned buffers the drawn tokens are copied to, used in turn
        self._host_flip = 0
        self._held_outputs: List[StepOutput] = []   # outputs read outside step() (abort), handed out by the next step()

    # --------------------------------------------------------------- requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None, key: Optional[int] = None) -> Hashable:
        n = next(self._ids)
        rid = request_id if request_id is not None else n
        if rid in self.requests and self.requests[rid].status != "finished":
            raise ValueError(f"request id {rid!r} is in use")
        vocab = self.runner.desc.vocab_size
        prompt = [int(t) for t in prompt]
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"prompt of request {rid!r} has a token id outside [0, {vocab})")
        req = Request(id=rid, prompt=prompt, params=params or SamplingParams(), key=n if key is None else key)
        self.requests[rid] = req
        self.scheduler.add(req)
        return rid

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None or bool(self._held_outputs)

    # ------------------------------------------------------------------- step
    def step(self) -> List[StepOutput]:
        """One scheduler step: plan, run the batch, draw tokens.

        With ``async_steps`` the drawn tokens stay on the device: the next step is planned and launched
        with them (count-based endings are known without their values) and only then are the tokens of
        the step before read, so the host works while the device does.  Outputs therefore come one call
        late; ``has_unfinished`` stays true until the last ones have been handed out.  Whenever the host
        needs token values first -- a preempted request to recompute, pages about to run out, a
        repetition penalty -- the step in flight is read before planning."""
        outs: List[StepOutput] = self._held_outputs
        self._held_outputs = []
        sched = self.scheduler
        if self._inflight is not None and (not self.ecfg.async_steps or sched.has_pending_outside_running()
                                           or sched.may_run_out_of_pages() or self._needs_token_values()):
            outs += self._resolve_inflight()
        plan = sched.schedule()
        if not plan.entries:
            sched.commit_launch(plan)
            outs += sched.resolve(plan, {})
            outs += self._resolve_inflight()
            return outs
        prev = self._inflight
        prev_rows = {r.id: i for i, r in enumerate(prev["samplers"])} if prev else {}
        entries = []
        for e in plan.entries:
            src = None
            if PENDING in e.tokens:
                src = [prev_rows[e.request.id] if t == PENDING else -1 for t in e.tokens]
            entries.append(StepEntry(e.request.id, e.tokens, [len(e.tokens) - 1] if e.samples else [], token_src=src))
        batch = self.runner.make_batch(entries, prev["tokens"] if prev else None)
        ev = self.step_events
        if ev is not None:
            ev[0].record()
        logits = self.runner.run_batch(batch)
        record = {"plan": plan, "samplers": [e.request for e in plan.entries if e.samples], "tokens": None,
                  "host": None, "event": None}
        samplers = record["samplers"]
        if samplers:
            need_seen = any(r.params.repetition_penalty != 1.0 for r in samplers)
            toks = self.sampler.sample(
                logits, [r.params for r in samplers], [r.key for r in samplers],
                [len(r.generated) for r in samplers],
                [r.tokens for r in samplers] if need_seen else None)
            record["tokens"] = toks
            if toks.is_cuda:
                i = self._host_flip                    # two pinned buffers in turn: the one of the step
                self._host_flip ^= 1                   # before may not have been read yet
                host = self._host_tokens[i]
                if host is None or host.numel() < toks.numel() + 1:
                    host = torch.zeros(max(256, toks.numel() + 1), dtype=torch.int32, pin_memory=True)
                    self._host_tokens[i] = host
                host[:toks.numel()].copy_(toks, non_blocking=True)
                # the kernels' error word travels with the tokens (last element of the buffer): a bounded wait
                # that ran out inside a kernel is reported when this step's tokens are read
                word = getattr(self.runner.ops, "error_word_async", None)
                if word is not None:
                    word(host, host.numel() - 1)
                    record["error_word"] = True
                record["host"] = host
                record["event"] = torch.cuda.Event()
                record["event"].record()
        if ev is not None:
            ev[1].record()
        sched.commit_launch(plan)
        self._inflight = record
        if prev is not None:
            outs += self._resolve(prev)
        if not self.ecfg.async_steps:
            outs += self._resolve_inflight()
        return outs

    def _needs_token_values(self) -> bool:
        return any(r.params.repetition_penalty != 1.0 for r in self.scheduler.running) or \
            any(r.params.repetition_penalty != 1.0 for r in self.scheduler.waiting)

    def _resolve(self, record) -> List[StepOutput]:
        drawn: Dict[Hashable, int] = {}
        if record["samplers"]:
            if record["event"] is not None:
                record["event"].synchronize()
                if record.get("error_word") and int(record["host"][-1]) != 0:
                    log.error("a bounded wait inside a kernel ran out during the step of %d requests whose tokens "
                              "were being read", len(record["samplers"]))
                    self.runner.ops.check_errors()             # raises
                host = record["host"][:len(record["samplers"])].tolist()
            else:
                host = record["tokens"].tolist()
            drawn = {r.id: t for r, t in zip(record["samplers"], host)}
        return self.scheduler.resolve(record["plan"], drawn)

    def _resolve_inflight(self) -> List[StepOutput]:
        if self._inflight is None:
            return []
        record, self._inflight = self._inflight, None
        return self._resolve(record)

    def abort(self, request_id: Hashable) -> None:
        """Ends a request now (reason "abort") and gives back what it holds.  A step in flight is read
        first (its pages must not go to another request while it still writes them); what it produced for
        the other requests is handed out by the next ``step()``, the aborted request's share is dropped."""
        self._held_outputs += [o for o in self._resolve_inflight() if o.request_id != request_id]
        r = self.requests.pop(request_id, None)
        if r is None or r.status == "finished":
            return
        if r in self.scheduler.waiting:
            self.scheduler.waiting.remove(r)
        self.scheduler._finish(r, "abort", release=r.status == "running")

    # --------------------------------------------------------------- generate
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None, *,
                 max_new_tokens: Optional[int] = None, temperature: float = 0.0, seed: int = 0,
                 return_requests: bool = False):
        """Runs the prompts to completion; returns the generated token ids of each."""
        if params is None:
            params = SamplingParams.make(temperature=temperature, seed=seed,
                                         max_new_tokens=16 if max_new_tokens is None else max_new_tokens)
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        ids = [self.add_request(p, sp, key=i) for i, (p, sp) in enumerate(zip(prompts, plist))]
        while self.has_unfinished():
            self.step()
        reqs = [self.requests[i] for i in ids]
        for i in ids:
            del self.requests[i]
        return reqs if return_requests else [r.generated for r in reqs]

    def stats(self) -> Dict[str, object]:
        s = dict(self.scheduler.counters)
        s.update(self.runner.cache.stats())
        s["kernel_launches"] = getattr(self.runner.ops, "launches", None)
        return s


class InferRuntime:
    """The reference's call sequence (test/main.cu:18-67) with its names.

        rt = InferRuntime()
        rt.load_model([model_dir], use_f16=True, n_ctx=4096, ...)
        rt.init_runtime_context()
        rt.encode([[1, 2, 3], [4, 5]])
        out = []
        rt.infer(64, out)          # out[i] = generated token ids of prompt i

    Flags of the reference's ModelConfig (src/core/model/BaseDefine.h:101-149) map as:
    ``_use_f16`` -> dtype bfloat16 (True) or float32 (False); ``_n_ctx`` -> max_model_len;
    ``_kv_data_type`` follows the dtype; ``_sampling_config`` -> ``sampling``.
    ``_rope_freq_base`` comes from config.json (rope_theta) and is not a flag here;
    ``_use_mmap`` is always on; ``_is_fuse_op`` is always on.
    """

    def __init__(self):
        self._model_dir = None
        self._ecfg = None
        self.engine: Optional[Engine] = None
        self._prompts: List[List[int]] = []
        self.sampling = SamplingParams()

    def load_model(self, model_files_path: Sequence[str], *, use_f16: bool = True, n_ctx: Optional[int] = None,
                   sampling: Optional[SamplingParams] = None, **engine_options) -> bool:
        if not model_files_path:
            raise ValueError("load_model needs the model folder")
        self._model_dir = model_files_path[0]
        self._ecfg = EngineConfig(dtype="bfloat16" if use_f16 else "float32", max_model_len=n_ctx, **engine_options)
        if sampling is not None:
            self.sampling = sampling
        return True

    def init_runtime_context(self) -> bool:
        self.engine = Engine(self._model_dir, self._ecfg)
        return True

    def encode(self, prompt_batches: Sequence[Sequence[int]]) -> int:
        """Stores the prompts (token ids); returns the longest length, as the reference does
        (src/core/runtime/InferRuntime.cu:383-425)."""
        self._prompts = [list(p) for p in prompt_batches]
        return max((len(p) for p in self._prompts), default=0)

    def infer(self, n_predict: int, responses: List[List[int]]) -> None:
        sp = SamplingParams(**{**self.sampling.__dict__, "max_new_tokens": n_predict})
        responses.extend(self.engine.generate(self._prompts, sp))
