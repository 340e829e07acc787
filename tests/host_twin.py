"""The plain twin of the C++ host runtime (tffinfer_b200/csrc/host/host_runtime.cpp): page pools, slots,
block tables, the decisions of a scheduler pass, the checks of a step and the packing of its integer
arrays, all in Python.  It is test equipment: the engine never uses it by itself.  It has the interface of
``tffinfer_b200.cache.NativeCacheManager`` (the product), so that a test can hand it to ``ModelRunner`` and
``Scheduler`` in its place; tests/test_native_host.py drives the two with the same random orders of
requests and compares every answer, page id by page id, every plan and every packed array.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from tffinfer_b200.cache import GroupSpec, CacheAccountingError, NO_PAGE
from tffinfer_b200.engine.batch import StepEntry, BatchLayout, NUM_FLAT, packed_to_device


class PagePool:
    FREE = None

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))   # pop() gives page 0 first
        self._owner: List[Optional[Hashable]] = [self.FREE] * self.num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int, owner: Hashable) -> Optional[List[int]]:
        """``n`` pages for ``owner``, or None (and nothing taken) if fewer are free."""
        if owner is self.FREE:
            raise ValueError("owner must not be None")
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._owner[p] is not self.FREE:
                raise CacheAccountingError(f"page {p} on the free list is owned by {self._owner[p]!r}")
            self._owner[p] = owner
        self.high_water = max(self.high_water, self.num_used)
        return out

    def free(self, pages, owner: Hashable) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise CacheAccountingError(f"page {p} does not exist")
            if self._owner[p] is self.FREE:
                raise CacheAccountingError(f"page {p} freed twice")
            if self._owner[p] != owner:
                raise CacheAccountingError(f"page {p} is owned by {self._owner[p]!r}, freed by {owner!r}")
            self._owner[p] = self.FREE
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is either on the free list once or owned; none is lost."""
        if len(set(self._free)) != len(self._free):
            raise CacheAccountingError("a page is on the free list twice")
        for p in self._free:
            if self._owner[p] is not self.FREE:
                raise CacheAccountingError(f"free page {p} has owner {self._owner[p]!r}")
        owned = sum(1 for o in self._owner if o is not self.FREE)
        if owned + len(self._free) != self.num_pages:
            raise CacheAccountingError("pages lost: owned + free != total")


class SlotPool:
    """Slots for per-request state of fixed size: one slot per live request.  The slot
    id travels with the request through every step even when no layer keeps state."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("a slot pool needs at least one slot")
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))
        self._owner: List[Optional[Hashable]] = [None] * self.num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, owner: Hashable) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        if self._owner[s] is not None:
            raise CacheAccountingError(f"slot {s} on the free list is owned by {self._owner[s]!r}")
        self._owner[s] = owner
        return s

    def free(self, slot: int, owner: Hashable) -> None:
        if not (0 <= slot < self.num_slots) or self._owner[slot] is None:
            raise CacheAccountingError(f"slot {slot} freed twice or does not exist")
        if self._owner[slot] != owner:
            raise CacheAccountingError(f"slot {slot} is owned by {self._owner[slot]!r}, freed by {owner!r}")
        self._owner[slot] = None
        self._free.append(slot)

    def check(self) -> None:
        owned = sum(1 for o in self._owner if o is not None)
        if len(set(self._free)) != len(self._free) or owned + len(self._free) != self.num_slots:
            raise CacheAccountingError("slot accounting broken")


@dataclass
class RequestCache:
    slot: int
    num_tokens: int = 0                       # tokens whose keys/values are in the cache
    reserved_tokens: int = 0                  # tokens a step is allowed to write up to
    tables: List[List[int]] = field(default_factory=list)   # per group: physical page per logical block


class TwinCacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, pages_per_group: Sequence[int],
                 max_live_requests: int):
        if len(groups) != len(pages_per_group):
            raise ValueError("one page count per group is needed")
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.pools = [PagePool(n) for n in pages_per_group]
        self.slots = SlotPool(max_live_requests)
        self.requests: Dict[Hashable, RequestCache] = {}

    # ------------------------------------------------------------- requests
    def admit(self, req: Hashable) -> Optional[int]:
        """A state slot and empty block tables for a new request; None if no slot is free."""
        if req in self.requests:
            raise CacheAccountingError(f"request {req!r} is already live")
        slot = self.slots.alloc(req)
        if slot is None:
            return None
        self.requests[req] = RequestCache(slot=slot, tables=[[] for _ in self.groups])
        return slot

    def is_live(self, req: Hashable) -> bool:
        return req in self.requests

    def num_tokens(self, req: Hashable) -> int:
        return self.requests[req].num_tokens

    def slot_of(self, req: Hashable) -> int:
        return self.requests[req].slot

    # ---------------------------------------------------------------- pages
    def _first_needed_block(self, g: int, num_tokens: int) -> int:
        """First logical block a query at position >= num_tokens can still read."""
        w = self.groups[g].window
        if w <= 0:
            return 0
        first_key = max(0, num_tokens - w + 1)     # query at p sees keys p-w+1 .. p
        return first_key // self.page_size

    def pages_needed(self, req: Hashable, n_new: int) -> List[int]:
        """Pages each group must still take so that ``n_new`` more tokens can be written."""
        rc = self.requests[req]
        total = rc.num_tokens + n_new
        blocks = -(-total // self.page_size)
        return [max(0, blocks - len(t)) for t in rc.tables]

    def reserve(self, req: Hashable, n_new: int) -> bool:
        """Take the pages for ``n_new`` more tokens in every group, or none at all."""
        if n_new < 0:
            raise ValueError("n_new must be >= 0")
        rc = self.requests[req]
        need = self.pages_needed(req, n_new)
        if any(n > p.num_free for n, p in zip(need, self.pools)):
            return False
        for g, n in enumerate(need):
            got = self.pools[g].alloc(n, req)
            assert got is not None
            rc.tables[g].extend(got)
        rc.reserved_tokens = max(rc.reserved_tokens, rc.num_tokens + n_new)
        return True

    def commit(self, req: Hashable, n_new: int) -> None:
        """``n_new`` tokens were written by a step.  Pages that every later query's
        window has passed go back to their pool."""
        rc = self.requests[req]
        if rc.num_tokens + n_new > rc.reserved_tokens:
            raise CacheAccountingError(
                f"request {req!r}: {n_new} tokens committed beyond the {rc.reserved_tokens} reserved")
        rc.num_tokens += n_new
        for g in range(len(self.groups)):
            first = self._first_needed_block(g, rc.num_tokens)
            t = rc.tables[g]
            gone = [t[b] for b in range(min(first, len(t))) if t[b] != NO_PAGE]
            if gone:
                self.pools[g].free(gone, req)
                for b in range(min(first, len(t))):
                    t[b] = NO_PAGE

    def commit_step(self, reqs: Sequence[Hashable], counts: Sequence[int]) -> None:
        """``counts[i]`` tokens of ``reqs[i]`` were written by one step."""
        for r, n in zip(reqs, counts):
            self.commit(r, n)

    def release(self, req: Hashable) -> None:
        """The request ended (finished, aborted or preempted): everything goes back."""
        rc = self.requests.pop(req)
        for g, t in enumerate(rc.tables):
            self.pools[g].free([p for p in t if p != NO_PAGE], req)
        self.slots.free(rc.slot, req)

    def block_table(self, req: Hashable, group: int) -> List[int]:
        return self.requests[req].tables[group]

    def max_blocks(self, reqs: Sequence[Hashable]) -> int:
        return max((len(t) for r in reqs for t in self.requests[r].tables), default=0)

    # --------------------------------------------------------------- checks
    def check(self) -> None:
        """No page lost, none held twice, owners consistent with the block tables."""
        for g, pool in enumerate(self.pools):
            pool.check()
            seen = {}
            for r, rc in self.requests.items():
                for p in rc.tables[g]:
                    if p == NO_PAGE:
                        continue
                    if p in seen:
                        raise CacheAccountingError(f"group {g}: page {p} held by {seen[p]!r} and {r!r}")
                    if pool.owner_of(p) != r:
                        raise CacheAccountingError(f"group {g}: page {p} in table of {r!r} is owned by "
                                                   f"{pool.owner_of(p)!r}")
                    seen[p] = r
            if len(seen) != pool.num_used:
                raise CacheAccountingError(f"group {g}: {pool.num_used} pages taken, {len(seen)} in block tables")
        self.slots.check()

    def stats(self) -> Dict[str, object]:
        return {"pages_total": [p.num_pages for p in self.pools],
                "pages_free": [p.num_free for p in self.pools],
                "pages_high_water": [p.high_water for p in self.pools],
                "slots_free": self.slots.num_free, "live_requests": len(self.requests)}


    # ------------------------------------------------------------- planning
    EVENT_PREEMPT, EVENT_FINISH, EVENT_ADMIT, EVENT_RUN = 1, 2, 3, 4

    def _fits_alone(self, length: int, budget_tokens: int) -> bool:
        """Whether a request of ``length`` tokens can ever run, alone (the rule of tffh_plan_step)."""
        for spec, pool in zip(self.groups, self.pools):
            most = length
            if spec.window > 0:
                most = min(most, spec.window + budget_tokens + 2 * self.page_size)
            if most > pool.num_pages * self.page_size:
                return False
        return True

    def plan_step(self, budget_tokens: int, max_model_len: int, running: Sequence, running_len: Sequence[int],
                  waiting: Sequence, waiting_len: Sequence[int], waiting_prompt_len: Sequence[int]):
        """The decisions of one scheduler pass, as tffh_plan_step takes them: decoded tokens first (one each),
        then portions of prompts in order of admission under the token budget, then admissions in arrival
        order while a slot, budget and pages are there; when pages run out the request admitted last gives
        way (alone, it ends with out_of_memory).  Returns the same events in the same order."""
        events = []
        run = list(zip(running, running_len))                  # in order of admission
        wait = list(zip(waiting, waiting_len, waiting_prompt_len))
        while True:
            budget = int(budget_tokens)
            free = [p.num_free for p in self.pools]
            chosen = []
            ok = True
            for decoding in (True, False):
                if not ok:
                    break
                for name, length in run:
                    left = length - self.num_tokens(name)
                    if (left != 1) if decoding else (left <= 1):
                        continue
                    if budget <= 0:
                        break
                    n = min(left, budget)
                    need = self.pages_needed(name, n)
                    if any(x > f for x, f in zip(need, free)):
                        ok = False
                        break
                    free = [f - x for f, x in zip(free, need)]
                    budget -= n
                    chosen.append((name, n))
                else:
                    continue
                break
            if not ok:
                name, length = run.pop()
                self.release(name)
                if not run:
                    events.append((self.EVENT_FINISH, name, "out_of_memory", 1))
                else:
                    events.append((self.EVENT_PREEMPT, name, 0, 0))
                    wait.insert(0, (name, length, 1))
                continue
            w = 0
            while w < len(wait) and budget > 0:
                name, length, prompt_len = wait[w]
                if prompt_len == 0 or length > max_model_len:
                    events.append((self.EVENT_FINISH, name, "too_long" if prompt_len else "empty_prompt", 0))
                    w += 1
                    continue
                if not self._fits_alone(length, budget_tokens):
                    events.append((self.EVENT_FINISH, name, "out_of_memory", 0))
                    w += 1
                    continue
                if self.slots.num_free == 0:
                    break
                n = min(length, budget)
                blocks = -(-n // self.page_size)
                if any(blocks > f for f in free):
                    break
                slot = self.admit(name)
                events.append((self.EVENT_ADMIT, name, slot, 0))
                free = [f - blocks for f in free]
                budget -= n
                run.append((name, length))
                chosen.append((name, n))
                w += 1
            break
        for name, n in chosen:
            start = self.num_tokens(name)
            assert self.reserve(name, n), "pages were counted but could not be taken"
            events.append((self.EVENT_RUN, name, n, start))
        return events

    # ------------------------------------------------------ a whole step at once
    def gather_step(self, entries):
        if len(entries) == 0:
            raise ValueError("a step needs at least one request and every request at least one token")
        from types import SimpleNamespace
        tokens = np.asarray([t for e in entries for t in e.tokens], dtype=np.int64).astype(np.int32)
        has_src = any(e.token_src is not None for e in entries)
        tok_src = None
        if has_src:
            tok_src = np.concatenate([np.asarray(e.token_src, dtype=np.int32) if e.token_src is not None
                                      else np.full(len(e.tokens), -1, dtype=np.int32) for e in entries])
        return SimpleNamespace(entries=list(entries), tokens=tokens, tok_src=tok_src, has_src=has_src)

    def reserve_step(self, arrays, max_model_len: int = 0):
        """The checks of a step and its pages, all or nothing, with the answers of tffh_reserve_step."""
        seen = set()
        for i, e in enumerate(arrays.entries):
            if e.req not in self.requests:
                return -2, i
            if e.req in seen:
                return -6, i
            seen.add(e.req)
            if len(e.tokens) == 0:
                return -1, i
            if max_model_len > 0 and self.num_tokens(e.req) + len(e.tokens) > max_model_len:
                return -7, i
        need = [0] * len(self.groups)
        for e in arrays.entries:
            for g, n in enumerate(self.pages_needed(e.req, len(e.tokens))):
                need[g] += n
        for g, n in enumerate(need):
            if n > self.pools[g].num_free:
                return 0, (g, n, self.pools[g].num_free)
        for e in arrays.entries:
            assert self.reserve(e.req, len(e.tokens))
        return 1, None

    def pack_step(self, entries, *, arrays=None, **kw):
        for e in entries:
            if e.req not in self.requests:
                raise KeyError(e.req)
        starts = [self.num_tokens(e.req) for e in entries]
        slots = [self.slot_of(e.req) for e in entries]
        tables = [[self.block_table(e.req, g) for e in entries] for g in range(len(self.groups))]
        return pack_step(entries, starts, slots, tables, **kw)


def pack_step(entries: Sequence[StepEntry], starts: Sequence[int], slots: Sequence[int],
              tables: Sequence[Sequence[Sequence[int]]], *, pad_requests: int = 0,
              widths: Optional[Sequence[int]] = None, dummy_pages: Optional[Sequence[int]] = None, dummy_slot: int = 0,
              out: Optional[np.ndarray] = None):
    """Packs the step into one int32 array.  Returns (array, layout, info).

    entries[i] starts at position starts[i]; tables[g][i] is request i's block table in
    group g (page ids, -1 for pages that were given back).  With ``pad_requests`` > len(entries)
    the batch is filled up with padding requests (one token 0 at position 0, logits asked)."""
    nreal = len(entries)
    q_lens = np.array([len(e.tokens) for e in entries], dtype=np.int32)
    if nreal == 0 or (q_lens <= 0).any():
        raise ValueError("a step needs at least one request and every request at least one token")
    npad = max(0, pad_requests - nreal)
    B = nreal + npad
    if npad:
        q_lens = np.concatenate([q_lens, np.ones(npad, dtype=np.int32)])
    T = int(q_lens.sum())
    q_start = np.zeros(B + 1, dtype=np.int32)
    np.cumsum(q_lens, out=q_start[1:])
    pos_start = np.zeros(B, dtype=np.int32)
    pos_start[:nreal] = np.asarray(starts, dtype=np.int32)
    kv_len = pos_start + q_lens
    token_ids = np.zeros(T, dtype=np.int32)
    if T - npad == nreal:           # every real request brings one token
        token_ids[:nreal] = [e.tokens[0] for e in entries]
    else:
        token_ids[:T - npad] = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
    tok_req = np.repeat(np.arange(B, dtype=np.int32), q_lens)
    positions = (np.arange(T, dtype=np.int32) - np.repeat(q_start[:-1], q_lens) + np.repeat(pos_start, q_lens)).astype(np.int32)
    rows = []
    for i, e in enumerate(entries):
        for w in e.want:
            if not (0 <= int(w) < int(q_lens[i])):
                raise ValueError(f"request {e.req!r}: wanted place {w} is outside its {int(q_lens[i])} tokens")
            rows.append(int(q_start[i]) + int(w))
    real_rows = len(rows)
    rows.extend(int(q_start[nreal + j]) for j in range(npad))
    G = len(tables)
    if widths is None:
        widths = [max(1, max((len(t) for t in tables[g]), default=0)) for g in range(G)]
    layout = BatchLayout(T, B, len(rows), tuple(int(w) for w in widths))
    if out is None:
        out = np.empty(layout.total, dtype=np.int32)
    elif out.shape[0] != layout.total:
        raise ValueError("the given buffer does not fit the batch layout")
    offs = layout.offsets()
    slot_arr = np.full(B, dummy_slot, dtype=np.int32)
    slot_arr[:nreal] = np.asarray(slots, dtype=np.int32)
    # requests ordered by the number of tokens they bring (shortest first): kernels that treat
    # single decoded tokens and long portions differently take a prefix or a suffix of this order
    # by the number of new tokens, and among equals the longest context first: the attention launches take
    # their requests in this order, and work items that start first should be the long ones
    req_order = np.lexsort((-kv_len, q_lens)).astype(np.int32)
    tok_src = np.full(T, -1, dtype=np.int32)
    has_src = False
    for i, e in enumerate(entries):
        if e.token_src is not None:
            tok_src[q_start[i]:q_start[i] + len(e.tokens)] = np.asarray(e.token_src, dtype=np.int32)
            has_src = True
    if has_src:
        token_ids[tok_src >= 0] = 0
    for o, arr in zip(offs[:NUM_FLAT], (token_ids, positions, tok_req, q_start, pos_start, kv_len, slot_arr,
                                        np.asarray(rows, dtype=np.int32), req_order, tok_src)):
        out[o:o + arr.shape[0]] = arr
    for g in range(G):
        w = layout.widths[g]
        bt = out[offs[NUM_FLAT + g]:offs[NUM_FLAT + g] + B * w].reshape(B, w)
        bt[:nreal] = -1
        bt[nreal:] = dummy_pages[g] if dummy_pages is not None else -1
        for i, t in enumerate(tables[g]):
            n = len(t)
            if n > w:
                raise ValueError("a block table is wider than the batch layout allows")
            if n:
                bt[i, :n] = t
    info = dict(max_q_len=int(q_lens.max()), max_kv_len=int(kv_len.max()), q_lens=q_lens, pos_start=pos_start,
                sorted_q_lens=q_lens[req_order], sorted_kv_lens=np.where(req_order < nreal, kv_len[req_order], 0),
                has_token_src=has_src,
                all_decode=bool((q_lens == 1).all()), real_requests=nreal, real_logit_rows=real_rows)
    return out, layout, info



def build_step_batch(entries: Sequence[StepEntry], starts: Sequence[int], slots: Sequence[int],
                     tables: Sequence[Sequence[Sequence[int]]], device, pinned: bool = False) -> StepBatch:
    """Packs the step and copies it to ``device`` in one transfer."""
    arr, layout, info = pack_step(entries, starts, slots, tables)
    return packed_to_device(arr, layout, info, device, pinned)
