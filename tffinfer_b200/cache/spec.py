"""What the cache manager is told about the model, and the error it raises.

Reference counterpart of the whole package: LLMKVCache / PageManager / LayerKVContext
(src/core/runtime/KVCache.h:36-473): one page table per (sequence, layer), pages of 32 tokens of one
layer, growth by ``append_token`` one page at a time, exhaustion reported by a ``false`` that the caller
ignores (KVCache.cpp:23-26; ModelCreatorBase.cpp:307-312), pages never given back during a run
(KVCache.h:445-455).  Differences here:

* a page holds ``page_size`` tokens of ALL layers of its group (one physical page id is valid for every
  layer of the group), so there is one block table per request and group;
* layers whose mixers declare different needs (all keys / a window of keys) are in different groups with
  pools of their own;
* a step's pages are taken in every group for every request of the step, or none at all;
* pages go back to the pool when a request ends and when a window has passed them, and are used again;
* every page has an owner: a page held twice, freed twice or lost is an error, not a wrong result.
"""
from __future__ import annotations

from dataclasses import dataclass

NO_PAGE = -1          # entry of a block table whose page was given back (a window has passed it)


@dataclass(frozen=True)
class GroupSpec:
    """A group of schedule entries with one need.  ``window`` 0 = all keys are kept."""
    num_layers: int
    num_kv_heads: int
    head_dim: int
    window: int = 0


class CacheAccountingError(RuntimeError):
    """The page accounting was violated (double free, foreign page, lost page)."""
