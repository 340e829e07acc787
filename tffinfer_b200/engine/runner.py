"""The step function and what it owns: the model, its weights, the cache tensors and
the cache manager.

One call of :meth:`ModelRunner.step` runs exactly the tokens it is given -- portions
of prompts beside single decoded tokens, cut anywhere -- as one batch, reading what
earlier steps left in the cache, and returns float32 logits at the wanted places.
It stands where the reference has ``prefill`` / ``decode``
(src/core/runtime/InferRuntime.cu:294-381), which build and run a task graph for one
sequence at a time and return logits of every row to the host.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import torch

from .. import log
from ..cache import make_cache_manager, GroupSpec
from ..config import EngineConfig, read_config_json
from ..parts import Model, CacheBinding, KVNeed, StateNeed
from ..registry import get_architecture
from ..weights import load_model_weights
from .batch import StepEntry, StepBatch, packed_to_device, batch_from_device, BatchLayout

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class OutOfPages(RuntimeError):
    """A step needs more cache pages than are free.  Nothing was taken."""


class RequestError(ValueError):
    """A request the engine cannot run (unknown id, token out of range, too long)."""


def _make_ops(device: str):
    from ..kernels.library import CudaKernels
    if not str(device).startswith("cuda"):
        raise RuntimeError(f"tffinfer_b200 runs on CUDA devices only (sm_100a); got device '{device}'")
    return CudaKernels()


class ModelRunner:
    def __init__(self, model_dir: Optional[str] = None, engine_config: Optional[EngineConfig] = None, *,
                 config=None, tensors: Optional[Dict[str, torch.Tensor]] = None, ops=None, cache_factory=None):
        """Either ``model_dir`` (config.json + safetensors) or ``config`` with ``tensors``
        (name -> tensor, checked like a file).  ``ops`` overrides the kernel library and
        ``cache_factory(groups, page_size, pages_per_group, max_live_requests)`` the host runtime (tests
        hand in plain twins of either; the engine itself has one of each)."""
        self._cache_factory = cache_factory or make_cache_manager
        import tffinfer_b200.parts  # noqa: F401  registers the built-in parts
        import tffinfer_b200.models  # noqa: F401  registers the architectures
        self.ecfg = (engine_config or EngineConfig()).normalized()
        self.device = torch.device(self.ecfg.device)
        self.ops = ops if ops is not None else _make_ops(self.ecfg.device)
        self.act_dtype = _TORCH_DTYPES[self.ecfg.dtype]
        if model_dir is not None:
            cj = read_config_json(model_dir)
            archs = cj.get("architectures")
            if not isinstance(archs, list) or not archs:
                from ..config import ConfigError
                raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
            arch = get_architecture(archs[0])
            self.config = arch.read_config(cj)
        else:
            if config is None or tensors is None:
                raise ValueError("give model_dir, or config together with tensors")
            self.config = config
            arch = get_architecture(config.architecture)
        self.desc = arch.describe(self.config)
        self.model = Model(self.desc)
        expected = self.model.expected_tensors()
        if model_dir is not None:
            held = load_model_weights(model_dir, expected, self.act_dtype, self.device)
        else:
            from ..weights.loader import check_tensors
            held = check_tensors(tensors, expected, self.act_dtype, self.device)
        self.model.load(held, self.ops, self.act_dtype, self.device)
        del held
        log.info("model %s: %d layers in %d runs, width %d, vocabulary %d, %s", self.desc_name(), len(self.desc.layers),
                 len(self.desc.schedule), self.desc.hidden_size, self.desc.vocab_size, self.ecfg.dtype)
        self.max_model_len = min(self.ecfg.max_model_len or self.desc.max_position, self.desc.max_position)
        self._build_cache()

    def desc_name(self) -> str:
        return getattr(self.config, "architecture", type(self.config).__name__)

    # ------------------------------------------------------------------ cache
    def _build_cache(self) -> None:
        needs = self.model.cache_needs()
        groups: List[GroupSpec] = []
        members: List[List[int]] = []
        self.bindings: List[CacheBinding] = [CacheBinding() for _ in needs]
        state_specs = []
        for e, need in enumerate(needs):
            if isinstance(need, KVNeed):
                key = (need.num_kv_heads, need.head_dim, need.window)
                for g, spec in enumerate(groups):
                    if (spec.num_kv_heads, spec.head_dim, spec.window) == key:
                        break
                else:
                    groups.append(GroupSpec(0, need.num_kv_heads, need.head_dim, need.window))
                    members.append([])
                    g = len(groups) - 1
                self.bindings[e] = CacheBinding(group=g, layer_in_group=len(members[g]), write=True)
                members[g].append(e)
            elif isinstance(need, StateNeed):
                self.bindings[e] = CacheBinding(state_index=len(state_specs))
                state_specs.append(need)
        for e, entry in enumerate(self.desc.schedule):
            if entry.cache_of is not None:
                src = self.bindings[entry.cache_of]
                self.bindings[e] = CacheBinding(group=src.group, layer_in_group=src.layer_in_group,
                                                write=False, state_index=src.state_index)
        groups = [GroupSpec(len(m), s.num_kv_heads, s.head_dim, s.window) for s, m in zip(groups, members)]
        ps = self.ecfg.page_size
        elt = torch.empty((), dtype=self.act_dtype).element_size()
        page_bytes = [g.num_layers * 2 * g.num_kv_heads * ps * g.head_dim * elt for g in groups]
        if self.ecfg.max_cache_tokens is not None:
            n_pages = [max(1, -(-self.ecfg.max_cache_tokens // ps)) for _ in groups]
        elif groups:
            if self.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(self.device)
                budget = int(free * self.ecfg.memory_fraction)
            else:
                budget = 1 << 28
            per = max(1, budget // max(1, sum(page_bytes)))
            cap = -(-self.max_model_len // ps) * self.ecfg.max_live_requests
            n_pages = [max(1, min(per, cap)) for _ in groups]
        else:
            n_pages = []
        # one page and one state slot more than the pools hand out: padding rows of a
        # fixed-size batch write there and nobody reads them
        # [pages, layers, 2, kv heads, page, head] as the parts and kernels index it, stored with the layers
        # outermost: the pages that one layer's attention reads then lie within that layer's share of the
        # pool (with the pages outermost they were 64 KB out of every layers x 64 KB, each in another 2 MB
        # page of the address space, and the attention of a 40-layer model read a quarter slower for it)
        self.kv_caches = [
            torch.zeros((g.num_layers, n + 1, 2, g.num_kv_heads, ps, g.head_dim), dtype=self.act_dtype,
                        device=self.device).permute(1, 0, 2, 3, 4, 5)
            for n, g in zip(n_pages, groups)]
        self.dummy_pages = list(n_pages)
        self.dummy_slot = self.ecfg.max_live_requests
        self.states = [torch.zeros((self.ecfg.max_live_requests + 1,) + tuple(s.shape),
                                   dtype=_STATE_DTYPES[s.dtype], device=self.device) for s in state_specs]
        self._graphs = {}
        self.last_h2d_bytes = 0
        self._graph_pool = None
        self._capture_stream = None
        self.graph_buckets = [b for b in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
                              if b <= self.ecfg.max_live_requests] or [self.ecfg.max_live_requests]
        if self.graph_buckets[-1] < min(self.ecfg.max_live_requests, 256):
            self.graph_buckets.append(min(self.ecfg.max_live_requests, 256))
        self.table_width = max(1, -(-self.max_model_len // ps))
        self.cache = self._cache_factory(groups, ps, n_pages, self.ecfg.max_live_requests)
        self.groups = groups
        for g, (spec, n, pb) in enumerate(zip(groups, n_pages, page_bytes)):
            # the reference logs the size of its cache the same way (src/core/runtime/InferRuntime.cu:109-140)
            log.info("cache group %d: %d layers, %d kv heads of %d, %s: %d pages of %d tokens (%.1f MiB), %s",
                     g, spec.num_layers, spec.num_kv_heads, spec.head_dim,
                     f"window {spec.window}" if spec.window else "all keys", n, ps, n * pb / 2 ** 20, self.ecfg.dtype)
        if self.states:
            log.info("%d state tensors of %d slots", len(self.states), self.ecfg.max_live_requests)

    # --------------------------------------------------------------- requests
    def add_request(self, req: Hashable) -> bool:
        """Make ``req`` live (a state slot, empty block tables).  False if no slot is free.
        Fixed-size state is not touched here: the step that brings a request's token at position 0
        clears its slot on the device (``_forward``), whoever admitted the request."""
        return self.cache.admit(req) is not None

    def finish_request(self, req: Hashable) -> None:
        self.cache.release(req)

    def num_tokens(self, req: Hashable) -> int:
        return self.cache.num_tokens(req)

    # ------------------------------------------------------------------- step
    def make_batch(self, entries: Sequence[StepEntry], prev_tokens: Optional[torch.Tensor] = None) -> StepBatch:
        """Checks the entries, takes the pages they need (all or nothing) and builds
        the device-side batch.  Raises OutOfPages without side effects.  Entries with
        ``token_src`` take token ids from ``prev_tokens`` (int32, on the device)."""
        arrays = self._check_and_reserve(entries, prev_tokens)
        if self._graph_eligible(entries):
            batch = self._make_static_batch(entries, arrays)
            if batch.tok_src is not None:
                self.ops.gather_tokens(batch.token_ids, prev_tokens, batch.tok_src)
            return batch
        batch = packed_to_device(*self._pack(entries, arrays), self.device, pinned=self.device.type == "cuda")
        if batch.tok_src is not None:
            self.ops.gather_tokens(batch.token_ids, prev_tokens, batch.tok_src)
        self.last_h2d_bytes = batch.token_ids.numel() * 0 + 4 * (
            3 * batch.num_tokens + 4 * batch.num_requests + 1 + batch.num_logit_rows
            + sum(t.numel() for t in batch.block_tables))
        return batch

    def _check_and_reserve(self, entries, prev_tokens):
        """The checks of a step and its pages, all or nothing, by the host runtime: the entries are gathered
        into flat arrays once (they are packed from the same arrays afterwards), token ids are checked on the
        array, and one call checks the requests and takes the pages of the whole step or none."""
        arrays = self.cache.gather_step(entries)
        tok = arrays.tokens if arrays.tok_src is None else arrays.tokens[arrays.tok_src < 0]
        if tok.size and (int(tok.min()) < 0 or int(tok.max()) >= self.desc.vocab_size):
            for e in entries:
                toks = e.tokens if e.token_src is None else [t for t, s in zip(e.tokens, e.token_src) if s < 0]
                if toks and (min(toks) < 0 or max(toks) >= self.desc.vocab_size):
                    raise RequestError(f"request {e.req!r}: token id outside [0, {self.desc.vocab_size})")
        if arrays.has_src and prev_tokens is None:
            e = next(e for e in entries if e.token_src is not None)
            raise RequestError(f"request {e.req!r} takes tokens from a previous step, but none was given")
        status, detail = self.cache.reserve_step(arrays, self.max_model_len)
        if status == 1:
            return arrays
        if status == 0:
            g, need, free = detail
            raise OutOfPages(f"step needs {need} pages in cache group {g}, {free} are free")
        req = entries[detail].req
        raise RequestError({-2: f"request {req!r} is not live (add_request first)",
                            -6: f"request {req!r} appears twice in one step",
                            -1: f"request {req!r} brings no tokens",
                            -7: f"request {req!r} would exceed the maximum length {self.max_model_len}",
                            }.get(status, f"request {req!r}: the host runtime refused the step ({status})"))

    # ------------------------------------------------------------ CUDA graphs
    def _graph_eligible(self, entries) -> bool:
        return (self.ecfg.use_cuda_graphs and self.device.type == "cuda"
                and len(entries) <= self.graph_buckets[-1]
                and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries))

    def _pack(self, entries, arrays=None, **kw):
        """The step's integer arrays in one host buffer, packed by the host runtime, which holds the
        positions, slots and block tables itself."""
        return self.cache.pack_step(entries, arrays=arrays, **kw)

    def _make_static_batch(self, entries, arrays=None) -> StepBatch:
        """Decode-only steps use device arrays of fixed address and size, one set per
        batch-size bucket, so that the step can be replayed as a CUDA graph.  A graph fixes the
        geometry of its launches, and how the attention shares out the key range depends on how
        unequal the contexts are: a bucket has one graph per class of that (batch.key_split_class)."""
        bucket = next(b for b in self.graph_buckets if b >= len(entries))
        st = self._graphs.get(bucket)
        if st is None:
            layout = BatchLayout(bucket, bucket, bucket, tuple(self.table_width for _ in self.groups))
            st = {"layout": layout,
                  "host": torch.empty(layout.total, dtype=torch.int32, pin_memory=True),
                  "dev": torch.empty(layout.total, dtype=torch.int32, device=self.device),
                  "graphs": {}}
            self._graphs[bucket] = st
        if st.get("copied") is not None:
            st["copied"].synchronize()              # the last copy out of the staging buffer has finished
        arr, layout, info = self._pack(entries, arrays, pad_requests=bucket, widths=st["layout"].widths,
                                       dummy_pages=self.dummy_pages, dummy_slot=self.dummy_slot,
                                       out=st["host"].numpy())
        st["dev"].copy_(st["host"], non_blocking=True)
        if st.get("copied") is None:
            st["copied"] = torch.cuda.Event()
        st["copied"].record()
        self.last_h2d_bytes = layout.total * 4
        batch = batch_from_device(st["dev"], layout, info)
        batch.graph_bucket = bucket
        classify = getattr(self.ops, "key_split_class", None)
        batch.key_split_class = classify(batch.h_sorted_kv_lens) if classify is not None else 1
        return batch

    def _run_graph(self, batch: StepBatch) -> torch.Tensor:
        graphs = self._graphs[batch.graph_bucket]["graphs"]
        st = graphs.get(batch.key_split_class)
        if st is None:
            # The first step of a class runs kernel by kernel and its logits are the step's result; the
            # capture that follows records the same launches without running them, and replays start
            # with the next step.  (Running the step once more as a replay would write the same keys and
            # values again, which is harmless, but would advance a mixer's fixed-size state twice.)
            eager = self._forward(batch)
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            launches = getattr(self.ops, "launches", 0)
            # Captured on a stream of its own, as torch.cuda.graph does it, but without that context's
            # gc.collect() and empty_cache(): giving the allocator's cached blocks back to the driver in the
            # middle of serving cost the steps around a capture tens of milliseconds (and now and then
            # hundreds) in frees and fresh allocations.
            if self._capture_stream is None:
                self._capture_stream = torch.cuda.Stream()
            main = torch.cuda.current_stream()
            self._capture_stream.wait_stream(main)
            with torch.cuda.stream(self._capture_stream):
                g.capture_begin(pool=self._graph_pool)
                try:
                    logits = self._forward(batch)
                finally:
                    g.capture_end()
            main.wait_stream(self._capture_stream)
            graphs[batch.key_split_class] = {"graph": g, "logits": logits,
                                             "launches": getattr(self.ops, "launches", 0) - launches}
            if hasattr(self.ops, "launches"):
                self.ops.launches = launches        # recorded, not run
            return eager[:batch.real_logit_rows]
        st["graph"].replay()
        if hasattr(self.ops, "launches"):
            self.ops.launches += st["launches"]
        return st["logits"][:batch.real_logit_rows]

    def _forward(self, batch: StepBatch) -> torch.Tensor:
        try:
            for state in self.states:       # requests that start (again) at position 0 start from zero state
                self.ops.reset_state_slots(state, batch.slots, batch.pos_start)
            return self.model.forward(batch, self.ops, self.act_dtype, self.bindings, self.kv_caches,
                                      batch.block_tables, self.ecfg.page_size, self.states)
        except Exception:
            reset = getattr(self.ops, "reset_accumulators", None)
            if reset is not None:
                reset()            # a step cut short may leave accumulator buffers half used
            raise

    def run_batch(self, batch: StepBatch) -> torch.Tensor:
        if getattr(batch, "graph_bucket", None) is not None:
            return self._run_graph(batch)
        return self._forward(batch)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the entries as one batch; returns float32 logits [wanted rows, vocab] in
        the order of the entries and of their ``want`` lists."""
        entries = list(entries)
        batch = self.make_batch(entries)
        logits = self.run_batch(batch)
        for e in entries:
            self.cache.commit(e.req, len(e.tokens))
        return logits
