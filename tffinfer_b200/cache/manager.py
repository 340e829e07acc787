"""Cache manager: keys and values in pages with a block table per request, one page
pool per group of layers with the same need, and slots for fixed-size state.

Reference counterpart: LLMKVCache / PageManager / LayerKVContext
(src/core/runtime/KVCache.h:36-473): one page table per (sequence, layer), pages of
32 tokens of one layer, growth by ``append_token`` one page at a time, exhaustion
reported by a ``false`` that the caller ignores (KVCache.cpp:23-26;
ModelCreatorBase.cpp:307-312).  Differences here:

* a page holds ``page_size`` tokens of ALL layers of its group (one physical page id
  is valid for every layer of the group), so there is one block table per request
  and group;
* layers whose mixers declare different needs (all keys / a window of keys) are in
  different groups with pools of their own;
* ``reserve`` takes what a step needs in every group or nothing at all, and says so;
* pages go back to the pool when a request ends and when a window has passed them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from .pages import PagePool, SlotPool, CacheAccountingError

NO_PAGE = -1


@dataclass(frozen=True)
class GroupSpec:
    """A group of schedule entries with one need.  ``window`` 0 = all keys are kept."""
    num_layers: int
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass
class RequestCache:
    slot: int
    num_tokens: int = 0                       # tokens whose keys/values are in the cache
    reserved_tokens: int = 0                  # tokens a step is allowed to write up to
    tables: List[List[int]] = field(default_factory=list)   # per group: physical page per logical block


class CacheManager:
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
