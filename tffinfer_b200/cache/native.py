"""The cache manager, the planner of a scheduler pass and the step packer: the C++ host runtime
(csrc/host/host_runtime.cpp) behind a Python class.  Keys and values live in pages with a block table per
request, one page pool per group of layers with the same need, and slots for fixed-size state.

This is the one host runtime of the engine.  A plain Python twin with the same interface lives with the
tests (tests/host_twin.py); they drive both with the same random orders of requests and compare every
answer.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from ..csrc import build as _build
from .spec import GroupSpec, CacheAccountingError

_i32p = ctypes.POINTER(ctypes.c_int)
_i64p = ctypes.POINTER(ctypes.c_int64)
_NO_SLOT = -100
_ERR_ARGUMENT, _ERR_UNKNOWN, _ERR_LIVE, _ERR_ACCOUNTING, _ERR_TOO_SMALL = -1, -2, -3, -4, -5

_lib = None


def host_library():
    """Loads (building first if needed) the host-runtime library; fails loudly if it cannot."""
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(_build.host_library_path(build=True))
        lib.tffh_cache_create.restype = ctypes.c_void_p
        lib.tffh_cache_create.argtypes = [ctypes.c_int, _i32p, ctypes.c_int, _i32p, ctypes.c_int]
        lib.tffh_cache_destroy.argtypes = [ctypes.c_void_p]
        lib.tffh_cache_destroy.restype = None
        lib.tffh_last_error.argtypes = [ctypes.c_void_p]
        lib.tffh_last_error.restype = ctypes.c_char_p
        for name in ("tffh_admit", "tffh_is_live", "tffh_num_tokens", "tffh_slot_of", "tffh_release"):
            getattr(lib, name).argtypes = [ctypes.c_void_p, ctypes.c_int64]
        for name in ("tffh_reserve", "tffh_commit"):
            getattr(lib, name).argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        lib.tffh_pages_needed.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, _i32p]
        lib.tffh_block_table.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, _i32p, ctypes.c_int]
        lib.tffh_check.argtypes = [ctypes.c_void_p]
        lib.tffh_count.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        lib.tffh_plan_step.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, _i64p, _i32p,
                                       ctypes.c_int, _i64p, _i32p, _i32p, _i32p, ctypes.c_int]
        lib.tffh_reserve_step.argtypes = [ctypes.c_void_p, ctypes.c_int, _i64p, _i32p, ctypes.c_int, _i32p]
        lib.tffh_commit_step.argtypes = [ctypes.c_void_p, ctypes.c_int, _i64p, _i32p]
        lib.tffh_pack_step.restype = ctypes.c_int64
        lib.tffh_pack_step.argtypes = [ctypes.c_void_p, ctypes.c_int, _i64p, _i32p, _i32p, _i32p, _i32p, _i32p,
                                       ctypes.c_int, _i32p, _i32p, ctypes.c_int, _i32p, ctypes.c_int64, _i32p]
        _lib = lib
    return _lib


def _p32(a: Optional[np.ndarray]):
    return a.ctypes.data_as(_i32p) if a is not None else None


class StepArrays:
    """The entries of a step as flat arrays (NativeCacheManager.gather_step)."""
    __slots__ = ("n", "reqs", "q_lens", "tokens", "want_start", "want", "tok_src", "has_src")

    def __init__(self, n, reqs, q_lens, tokens, want_start, want, tok_src, has_src):
        self.n, self.reqs, self.q_lens, self.tokens = n, reqs, q_lens, tokens
        self.want_start, self.want, self.tok_src, self.has_src = want_start, want, tok_src, has_src


class _PoolView:
    """What the scheduler and the statistics read of one page pool."""
    def __init__(self, owner: "NativeCacheManager", group: int):
        self._o, self._g = owner, group

    @property
    def num_pages(self) -> int:
        return self._o._count(0, self._g)

    @property
    def num_free(self) -> int:
        return self._o._count(1, self._g)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.num_free

    @property
    def high_water(self) -> int:
        return self._o._count(2, self._g)


class _SlotView:
    def __init__(self, owner: "NativeCacheManager"):
        self._o = owner

    @property
    def num_free(self) -> int:
        return self._o._count(3, 0)


class NativeCacheManager:
    """Page pools, slots and block tables of the live requests; the state lives in the C++ object."""

    def __init__(self, groups: Sequence[GroupSpec], page_size: int, pages_per_group: Sequence[int],
                 max_live_requests: int):
        if len(groups) != len(pages_per_group):
            raise ValueError("one page count per group is needed")
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if any(n <= 0 for n in pages_per_group):
            raise ValueError("a page pool needs at least one page")
        if max_live_requests <= 0:
            raise ValueError("a slot pool needs at least one slot")
        self.lib = host_library()
        self.groups = list(groups)
        self.page_size = int(page_size)
        windows = np.asarray([g.window for g in groups], dtype=np.int32)
        pages = np.asarray(list(pages_per_group), dtype=np.int32)
        self._h = self.lib.tffh_cache_create(len(groups), _p32(windows), self.page_size, _p32(pages),
                                             int(max_live_requests))
        if not self._h:
            raise ValueError("the host runtime refused these cache sizes")
        self.pools = [_PoolView(self, g) for g in range(len(groups))]
        self.slots = _SlotView(self)
        self._handle: Dict[Hashable, int] = {}       # request name -> 64-bit handle
        self._next = 1
        self._need = np.zeros(max(1, len(groups)), dtype=np.int32)
        self._info = np.zeros(8, dtype=np.int32)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                self.lib.tffh_cache_destroy(h)
            except Exception:        # the interpreter is shutting down and the library is gone
                pass

    # ------------------------------------------------------------- plumbing
    def _raise(self, code: int):
        words = self.lib.tffh_last_error(self._h).decode()
        if code == _ERR_ACCOUNTING or code == _ERR_LIVE:
            raise CacheAccountingError(words)
        if code == _ERR_UNKNOWN:
            raise KeyError(words)
        raise ValueError(words)

    def _count(self, what: int, group: int) -> int:
        n = self.lib.tffh_count(self._h, what, group)
        if n < 0:
            self._raise(n)
        return n

    def _h_of(self, req: Hashable) -> int:
        try:
            return self._handle[req]
        except KeyError:
            raise KeyError(req) from None

    # ------------------------------------------------------------- requests
    def admit(self, req: Hashable) -> Optional[int]:
        if req in self._handle:
            raise CacheAccountingError(f"request {req!r} is already live")
        h = self._next
        slot = self.lib.tffh_admit(self._h, h)
        if slot == _NO_SLOT:
            return None
        if slot < 0:
            self._raise(slot)
        self._next += 1
        self._handle[req] = h
        return slot

    def is_live(self, req: Hashable) -> bool:
        return req in self._handle

    def num_tokens(self, req: Hashable) -> int:
        n = self.lib.tffh_num_tokens(self._h, self._h_of(req))
        if n < 0:
            self._raise(n)
        return n

    def slot_of(self, req: Hashable) -> int:
        s = self.lib.tffh_slot_of(self._h, self._h_of(req))
        if s < 0:
            self._raise(s)
        return s

    # ---------------------------------------------------------------- pages
    def pages_needed(self, req: Hashable, n_new: int) -> List[int]:
        st = self.lib.tffh_pages_needed(self._h, self._h_of(req), int(n_new), _p32(self._need))
        if st < 0:
            self._raise(st)
        return self._need[:len(self.groups)].tolist()

    def reserve(self, req: Hashable, n_new: int) -> bool:
        if n_new < 0:
            raise ValueError("n_new must be >= 0")
        st = self.lib.tffh_reserve(self._h, self._h_of(req), int(n_new))
        if st < 0:
            self._raise(st)
        return bool(st)

    def commit(self, req: Hashable, n_new: int) -> None:
        st = self.lib.tffh_commit(self._h, self._h_of(req), int(n_new))
        if st < 0:
            self._raise(st)

    def release(self, req: Hashable) -> None:
        h = self._handle.pop(req)
        st = self.lib.tffh_release(self._h, h)
        if st < 0:
            self._raise(st)

    def block_table(self, req: Hashable, group: int) -> List[int]:
        h = self._h_of(req)
        n = self.lib.tffh_block_table(self._h, h, group, None, 0)
        if n < 0:
            self._raise(n)
        out = np.empty(max(1, n), dtype=np.int32)
        n = self.lib.tffh_block_table(self._h, h, group, _p32(out), out.shape[0])
        if n < 0:
            self._raise(n)
        return out[:n].tolist()

    def max_blocks(self, reqs: Sequence[Hashable]) -> int:
        return max((len(self.block_table(r, g)) for r in reqs for g in range(len(self.groups))), default=0)

    # --------------------------------------------------------------- checks
    def check(self) -> None:
        st = self.lib.tffh_check(self._h)
        if st < 0:
            self._raise(st)

    def stats(self) -> Dict[str, object]:
        return {"pages_total": [p.num_pages for p in self.pools],
                "pages_free": [p.num_free for p in self.pools],
                "pages_high_water": [p.high_water for p in self.pools],
                "slots_free": self.slots.num_free, "live_requests": self._count(4, 0)}

    # ------------------------------------------------------------- planning
    EVENT_PREEMPT, EVENT_FINISH, EVENT_ADMIT, EVENT_RUN = 1, 2, 3, 4
    REASONS = {1: "out_of_memory", 2: "too_long", 3: "empty_prompt"}

    def plan_step(self, budget_tokens: int, max_model_len: int, running: Sequence, running_len: Sequence[int],
                  waiting: Sequence, waiting_len: Sequence[int], waiting_prompt_len: Sequence[int]):
        """The decisions of one scheduler pass, taken by the C++ host runtime (tffh_plan_step): which running
        requests bring how many tokens, who is preempted, who ends without running, who is admitted; the pages
        of the chosen are taken.  ``running`` are live request names in the order of their admission,
        ``waiting`` the queue in arrival order.  Returns events (kind, name, a, b) in the order they happened:
        (EVENT_PREEMPT, name, 0, 0), (EVENT_FINISH, name, reason, was_running), (EVENT_ADMIT, name, slot, 0),
        (EVENT_RUN, name, tokens, start)."""
        nr, nw = len(running), len(waiting)
        rh = np.fromiter((self._h_of(r) for r in running), dtype=np.int64, count=nr) if nr else np.zeros(1, np.int64)
        rl = np.asarray(list(running_len) or [0], dtype=np.int32)
        wh = np.arange(self._next, self._next + max(1, nw), dtype=np.int64)     # handles the admitted would get
        wl = np.asarray(list(waiting_len) or [0], dtype=np.int32)
        wp = np.asarray(list(waiting_prompt_len) or [0], dtype=np.int32)
        cap = 2 * (nr + nw) + 4
        ev = np.zeros(4 * cap, dtype=np.int32)
        n = self.lib.tffh_plan_step(self._h, int(budget_tokens), int(max_model_len), nr, rh.ctypes.data_as(_i64p),
                                    _p32(rl), nw, wh.ctypes.data_as(_i64p), _p32(wl), _p32(wp), _p32(ev), cap)
        self._next += nw
        if n < 0:
            self._raise(n)
        out = []
        for kind, uid, a, b in ev[:4 * n].reshape(n, 4).tolist():
            name = running[uid] if uid < nr else waiting[uid - nr]
            handle = int(rh[uid]) if uid < nr else int(wh[uid - nr])
            if kind == self.EVENT_PREEMPT or (kind == self.EVENT_FINISH and b):
                del self._handle[name]
            elif kind == self.EVENT_ADMIT:
                self._handle[name] = handle
            out.append((kind, name, self.REASONS[a] if kind == self.EVENT_FINISH else a, b))
        return out

    # ------------------------------------------------------ a whole step at once
    def gather_step(self, entries) -> "StepArrays":
        """The entries of a step as flat arrays (handles, token counts, token ids, wanted places, source rows):
        gathered once, used by the checks, by reserve_step and by pack_step.  A request that is not live
        gets the handle 0, which never is: the library then says which entry it was."""
        n = len(entries)
        if n == 0:
            raise ValueError("a step needs at least one request and every request at least one token")
        handle = self._handle
        reqs = np.fromiter((handle.get(e.req, 0) for e in entries), dtype=np.int64, count=n)
        q_lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=n)
        if int(q_lens.sum()) == n and int(q_lens.min()) == 1:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=n).astype(np.int32)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries] +
                                    [np.zeros(1, dtype=np.int64)]).astype(np.int32)[:int(q_lens.sum())]
        want_start = np.zeros(n + 1, dtype=np.int32)
        np.cumsum(np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=n), out=want_start[1:])
        want = np.fromiter((int(w) for e in entries for w in e.want), dtype=np.int32, count=int(want_start[-1]))
        if want.shape[0] == 0:
            want = np.zeros(1, dtype=np.int32)
        has_src = any(e.token_src is not None for e in entries)
        tok_src = None
        if has_src:
            tok_src = np.concatenate([np.asarray(e.token_src, dtype=np.int32) if e.token_src is not None
                                      else np.full(len(e.tokens), -1, dtype=np.int32) for e in entries])
        return StepArrays(n, reqs, q_lens, tokens, want_start, want, tok_src, has_src)

    def reserve_step(self, arrays: "StepArrays", max_model_len: int = 0):
        """Checks the step's requests and takes the pages all of them need, or none (tffh_reserve_step).
        Returns (1, None) when taken, (0, (group, needed, free)) when the pages do not suffice, and
        (code, index of the entry) for a request that is not live (-2), appears twice (-6), brings no
        tokens (-1) or would grow beyond ``max_model_len`` (-7)."""
        detail = np.zeros(3, dtype=np.int32)
        st = self.lib.tffh_reserve_step(self._h, arrays.n, arrays.reqs.ctypes.data_as(_i64p), _p32(arrays.q_lens),
                                        int(max_model_len), _p32(detail))
        if st == 1:
            return 1, None
        if st == 0:
            return 0, tuple(int(x) for x in detail)
        if st == _ERR_ACCOUNTING:
            self._raise(st)
        return st, int(detail[0])

    def commit_step(self, reqs: Sequence[Hashable], counts: Sequence[int]) -> None:
        n = len(reqs)
        if n == 0:
            return
        h = np.fromiter((self._h_of(r) for r in reqs), dtype=np.int64, count=n)
        c = np.asarray(list(counts), dtype=np.int32)
        st = self.lib.tffh_commit_step(self._h, n, h.ctypes.data_as(_i64p), _p32(c))
        if st < 0:
            self._raise(st)

    # -------------------------------------------------------------- packing
    def pack_step(self, entries, *, pad_requests: int = 0, widths: Optional[Sequence[int]] = None,
                  dummy_pages: Optional[Sequence[int]] = None, dummy_slot: int = 0,
                  out: Optional[np.ndarray] = None, arrays: Optional["StepArrays"] = None):
        """The step's integer arrays in one int32 buffer (layout: engine.batch.BatchLayout), with positions,
        slots and block tables taken from this manager.  Returns (array, layout, info); ``info`` holds the
        host-side figures launch decisions need.  ``pad_requests`` fills the batch up with padding requests
        (one token at position 0 writing to ``dummy_pages`` / ``dummy_slot``), ``widths`` fixes the block-table
        widths, ``out`` is a buffer to pack into, ``arrays`` what gather_step made of the entries."""
        from ..engine.batch import BatchLayout
        if arrays is None:
            arrays = self.gather_step(entries)
        n, reqs, q_lens, tokens = arrays.n, arrays.reqs, arrays.q_lens, arrays.tokens
        want_start, want, tok_src, has_src = arrays.want_start, arrays.want, arrays.tok_src, arrays.has_src
        if (q_lens <= 0).any():
            raise ValueError("a step needs at least one request and every request at least one token")
        if (reqs == 0).any():
            raise KeyError(entries[int(np.argmax(reqs == 0))].req)
        G = len(self.groups)
        w = np.asarray(list(widths) if widths is not None else [0] * G, dtype=np.int32)
        if w.shape[0] == 0:
            w = np.zeros(1, dtype=np.int32)
        dp = np.asarray(list(dummy_pages), dtype=np.int32) if dummy_pages is not None and G else None
        info = self._info
        if out is None:
            # ask for the size first (the widths are chosen by the library when none are given)
            wq = w.copy()
            st = self.lib.tffh_pack_step(self._h, n, reqs.ctypes.data_as(_i64p), _p32(q_lens), _p32(tokens),
                                         _p32(want_start), _p32(want), _p32(tok_src), int(pad_requests), _p32(wq),
                                         _p32(dp), int(dummy_slot), None, 0, _p32(info))
            if st != _ERR_TOO_SMALL:
                self._raise(st)
            out = np.empty(int(info[0]), dtype=np.int32)
        st = self.lib.tffh_pack_step(self._h, n, reqs.ctypes.data_as(_i64p), _p32(q_lens), _p32(tokens),
                                     _p32(want_start), _p32(want), _p32(tok_src), int(pad_requests), _p32(w),
                                     _p32(dp), int(dummy_slot), _p32(out), out.shape[0], _p32(info))
        if st < 0:
            self._raise(st)
        T, B, R = int(info[0]), int(info[1]), int(info[2])
        layout = BatchLayout(T, B, R, tuple(int(x) for x in w[:G]))
        if layout.total != out.shape[0]:
            raise ValueError("the given buffer does not fit the batch layout")
        offs = layout.offsets()
        q_start = out[offs[3]:offs[3] + B + 1]
        q_all = np.diff(q_start).astype(np.int32)
        pos_start = out[offs[4]:offs[4] + B].copy()
        kv_len = out[offs[5]:offs[5] + B]
        order = out[offs[8]:offs[8] + B]
        meta = dict(max_q_len=int(info[3]), max_kv_len=int(info[4]), q_lens=q_all, pos_start=pos_start,
                    sorted_q_lens=q_all[order], sorted_kv_lens=np.where(order < n, kv_len[order], 0),
                    has_token_src=has_src, all_decode=bool(info[6]), real_requests=n, real_logit_rows=int(info[7]))
        return out, layout, meta
