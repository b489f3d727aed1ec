"""The cache manager: which pages and which slot each live request holds.

Layers declare what they need to keep between steps (:class:`PagedNeed`: keys and values
that grow with the tokens, all of them or a window; :class:`SlotNeed`: state of fixed size).
Layers with the same need form a *group*; each paged group has pages and block tables of
its own, each slot group one tensor indexed by the request's slot.  Pages are taken as
tokens are scheduled (never ahead for a whole request), are given back when the request ends
or, in a windowed group, when the window has passed them, and are handed out again without
being cleared: readers mask by length, never by content.

The reference allocates every page of ``prompt + max_tokens`` at admission
(``pkg/inference/batch_scheduler.go:214-218``, ``paged_kvcache.go:177-194``), has one
group only, and keeps per-request conv state on the host
(``batch_scheduler.go:240-243,437-458``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from .pages import OutOfPages, OutOfSlots, PagePool, SlotPool


@dataclass(frozen=True)
class PagedNeed:
    """Keys and values per token: ``n_kv_heads * head_dim`` each; ``window`` None = keep all."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class SlotNeed:
    """A state of fixed ``shape`` per request, set to ``init`` when a request starts.
    ``dtype`` names the element type the layer keeps it in ("float32", "bfloat16", "float16",
    "int32"); layers that differ in any of the three get groups of their own."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
    init: float = 0.0


@dataclass
class _Request:
    slot: int
    length: int = 0                                       # tokens whose state is in the cache
    tables: List[List[int]] = field(default_factory=list)  # per paged group: page index -> page id, -1 freed
    first_live: List[int] = field(default_factory=list)    # per paged group: first page index still held


class CacheManager:
    """Host-side accounting for ``max_requests`` slots and one page pool per paged group."""

    def __init__(self, paged_needs: Sequence[PagedNeed], pages_per_group: Sequence[int],
                 page_size: int, max_requests: int, max_seq_len: int):
        if page_size <= 0 or page_size & (page_size - 1):
            raise ValueError(f"page_size must be a power of two, got {page_size}")
        if len(paged_needs) != len(pages_per_group):
            raise ValueError("one page count per paged group is needed")
        self.page_size = page_size
        self.paged_needs = tuple(paged_needs)
        self.pools = [PagePool(n) for n in pages_per_group]
        self.slots = SlotPool(max_requests)
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self.max_pages_per_request = -(-max_seq_len // page_size)
        self._req: Dict[Hashable, _Request] = {}
        self.windowed = any(n.window is not None for n in self.paged_needs)
        # the block tables once more as arrays, one row per slot, kept in step with the lists:
        # the step function gathers the rows of a batch in one indexing operation
        self.table_rows = [np.full((max_requests, self.max_pages_per_request), -1, dtype=np.int32)
                           for _ in self.pools]

    # ---------------------------------------------------------------- requests
    def admit(self, req_id: Hashable) -> int:
        """Give the request a slot (its state there must be zeroed by the caller)."""
        if req_id in self._req:
            raise KeyError(f"request {req_id!r} is already live")
        slot = self.slots.take_one()
        g = len(self.pools)
        self._req[req_id] = _Request(slot, 0, [[] for _ in range(g)], [0] * g)
        return slot

    def is_live(self, req_id) -> bool:
        return req_id in self._req

    def live_requests(self):
        return list(self._req)

    def length(self, req_id) -> int:
        return self._req[req_id].length

    def slot(self, req_id) -> int:
        return self._req[req_id].slot

    def table(self, req_id, group: int) -> List[int]:
        return self._req[req_id].tables[group]

    # ---------------------------------------------------------------- pages
    def _passed(self, group: int, length: int) -> int:
        """Number of leading pages that no query at position >= length can see."""
        w = self.paged_needs[group].window
        if w is None:
            return 0
        first_visible = length - w + 1           # lowest key position the next query reads
        return max(0, first_visible // self.page_size)

    def pages_to_take(self, req_id, n_new: int) -> List[int]:
        """Per group, pages that extending the request by ``n_new`` tokens takes from the pool
        (after the pages its window has passed are given back)."""
        r = self._req[req_id]
        end_pages = -(-(r.length + n_new) // self.page_size)
        return [max(0, end_pages - len(t)) for t in r.tables]

    def pages_freed_first(self, req_id) -> List[int]:
        r = self._req[req_id]
        return [max(0, min(self._passed(g, r.length), len(r.tables[g])) - r.first_live[g])
                for g in range(len(self.pools))]

    def can_extend(self, req_id, n_new: int) -> bool:
        r = self._req[req_id]
        if r.length + n_new > self.max_seq_len:
            return False
        take, freed = self.pages_to_take(req_id, n_new), self.pages_freed_first(req_id)
        return all(t <= p.free + f for t, p, f in zip(take, self.pools, freed))

    def extend(self, req_id, n_new: int) -> None:
        """Make room for ``n_new`` more tokens: all groups or none (:class:`OutOfPages`)."""
        r = self._req[req_id]
        if n_new < 0:
            raise ValueError("n_new must be >= 0")
        if r.length + n_new > self.max_seq_len:
            raise OutOfPages(f"request {req_id!r} would hold {r.length + n_new} tokens, capacity {self.max_seq_len}")
        if not self.windowed and n_new <= self.slack(req_id):
            return                                            # fits in the pages it holds
        if not self.can_extend(req_id, n_new):
            raise OutOfPages(f"request {req_id!r} needs {self.pages_to_take(req_id, n_new)} pages, "
                             f"free {[p.free for p in self.pools]}")
        for g, pool in enumerate(self.pools):
            t = r.tables[g]
            passed = min(self._passed(g, r.length), len(t))
            for j in range(r.first_live[g], passed):
                pool.give_back(t[j])
                t[j] = -1
                self.table_rows[g][r.slot, j] = -1
            r.first_live[g] = max(r.first_live[g], passed)
        for g, (pool, n) in enumerate(zip(self.pools, self.pages_to_take(req_id, n_new))):
            if n:
                new = pool.take(n)
                t = r.tables[g]
                self.table_rows[g][r.slot, len(t):len(t) + n] = new
                t.extend(new)

    def slack(self, req_id) -> int:
        """Tokens the request can still add without taking a page."""
        r = self._req[req_id]
        if not r.tables:
            return self.max_seq_len - r.length
        return min(len(t) for t in r.tables) * self.page_size - r.length

    def advance(self, req_id, n_new: int) -> None:
        """The step that wrote ``n_new`` tokens has been issued."""
        r = self._req[req_id]
        cap = min(len(t) for t in r.tables) * self.page_size if r.tables else self.max_seq_len
        if r.length + n_new > cap:
            raise RuntimeError(f"request {req_id!r}: advancing to {r.length + n_new} beyond its pages ({cap})")
        r.length += n_new

    def release(self, req_id) -> int:
        """Give back everything the request holds; returns its slot."""
        r = self._req.pop(req_id)
        for g, (pool, t) in enumerate(zip(self.pools, r.tables)):
            for p in t:
                if p >= 0:
                    pool.give_back(p)
            self.table_rows[g][r.slot, :len(t)] = -1
        self.slots.give_back(r.slot)
        return r.slot

    # ---------------------------------------------------------------- accounting
    def pages_free(self) -> List[int]:
        return [p.free for p in self.pools]

    def slots_free(self) -> int:
        return self.slots.free

    def pages_held(self, req_id) -> List[int]:
        return [sum(1 for p in t if p >= 0) for t in self._req[req_id].tables]

    def check(self) -> None:
        """Invariants: every page is free or held by exactly one request; same for slots."""
        for g, pool in enumerate(self.pools):
            held: List[int] = []
            for r in self._req.values():
                held.extend(p for p in r.tables[g] if p >= 0)
            if len(held) != len(set(held)):
                raise AssertionError(f"group {g}: a page is held twice")
            if sorted(held) != pool.held_pages():
                raise AssertionError(f"group {g}: pages held by requests and by the pool differ")
            if len(held) + pool.free != pool.num_pages:
                raise AssertionError(f"group {g}: a page is lost")
        for g in range(len(self.pools)):
            for r in self._req.values():
                row = self.table_rows[g][r.slot]
                if row[:len(r.tables[g])].tolist() != r.tables[g] or (row[len(r.tables[g]):] != -1).any():
                    raise AssertionError(f"group {g}: the table array of slot {r.slot} differs from its list")
        slots = [r.slot for r in self._req.values()]
        if len(slots) != len(set(slots)) or sorted(slots) != self.slots.held_pages():
            raise AssertionError("slot bookkeeping is inconsistent")
