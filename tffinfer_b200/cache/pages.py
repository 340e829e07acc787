"""Page pool: fixed number of pages, a last-in-first-out free list, and an owner
record per page so that a page held twice or freed twice is an error, not a wrong
result.  The reference's PageManager is a vector of pages with a LIFO free list
(src/core/runtime/KVCache.h:81-100) whose pages are never given back during a run
(LLMKVCache::clear is never called, KVCache.h:445-455); here they are."""
from __future__ import annotations

from typing import Hashable, List, Optional


class CacheAccountingError(RuntimeError):
    """The page accounting was violated (double free, foreign page, lost page)."""


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
