"""The cache manager: pages of keys and values with a block table per request, and slots of
fixed-size per-request state.  Pure host bookkeeping; the tensors live in
:mod:`.storage`.

Layer runs whose mixers keep keys and values are put into *groups* by what they need to
keep: all keys (``window`` None) or the last ``window`` of them.  Each group has a pool and
block tables of its own, because a windowed group gives pages back while a request is
still running.  One page id of a group indexes the pages of every run of that group
(nanovllm/engine/block_manager.py:47-131 has one such pool for all layers).

A request's logical page i holds tokens [i * page_size, (i + 1) * page_size).  Its table
lists the physical page of every logical page, -1 where a window has passed and the page
was given back.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .page_pool import OutOfPages, PagePool, StateSlotAllocator


@dataclass(frozen=True)
class GroupSpec:
    window: int | None      # None: keep every key


@dataclass
class _Request:
    tables: list[list[int]]                 # per group: physical page per logical page (-1: given back)
    released: list[int]                     # per group: logical pages [0, released) were given back
    state_slot: int | None = None
    num_tokens: int = 0                     # tokens that have pages


class CacheManager:
    def __init__(self, groups: list[GroupSpec], page_size: int, num_pages: int | list[int], num_state_slots: int = 0):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        counts = num_pages if isinstance(num_pages, (list, tuple)) else [num_pages] * len(self.groups)
        if len(counts) != len(self.groups):
            raise ValueError("one page count per group is needed")
        self.pools = [PagePool(n) for n in counts]
        self.slots = StateSlotAllocator(num_state_slots) if num_state_slots > 0 else None
        self._requests: dict[object, _Request] = {}

    # ------------------------------------------------------------------ queries
    def __contains__(self, req_id) -> bool:
        return req_id in self._requests

    def num_live(self) -> int:
        return len(self._requests)

    def _first_needed_page(self, g: int, num_computed: int) -> int:
        """The first logical page a query at position >= num_computed can still read."""
        w = self.groups[g].window
        if w is None:
            return 0
        return max(0, num_computed - w + 1) // self.page_size

    def pages_needed(self, req_id, num_tokens: int) -> list[int]:
        """New pages per group so that tokens [0, num_tokens) of the request are covered."""
        req = self._requests.get(req_id)
        total = -(-num_tokens // self.page_size)
        return [max(0, total - (len(req.tables[g]) if req else 0)) for g in range(len(self.groups))]

    def can_allocate(self, req_id, num_tokens: int) -> bool:
        need = self.pages_needed(req_id, num_tokens)
        if any(n > pool.num_free for n, pool in zip(need, self.pools)):
            return False
        if req_id not in self._requests and self.slots is not None and not self.slots.can_allocate():
            return False
        return True

    def block_table(self, req_id, group: int = 0) -> list[int]:
        return self._requests[req_id].tables[group]

    def state_slot(self, req_id) -> int | None:
        return self._requests[req_id].state_slot

    def num_tokens(self, req_id) -> int:
        return self._requests[req_id].num_tokens

    # ------------------------------------------------------------------ changes
    def allocate(self, req_id, num_tokens: int) -> None:
        """Make sure tokens [0, num_tokens) of the request have pages in every group; a new request also
        gets its state slot.  Raises :class:`OutOfPages` and changes nothing if any group falls short."""
        if not self.can_allocate(req_id, num_tokens):
            raise OutOfPages(f"request {req_id!r}: no room for {num_tokens} tokens "
                             f"(free pages per group: {[p.num_free for p in self.pools]})")
        req = self._requests.get(req_id)
        if req is None:
            slot = self.slots.allocate() if self.slots is not None else None
            req = self._requests[req_id] = _Request([[] for _ in self.groups], [0] * len(self.groups), slot)
        for g, n in enumerate(self.pages_needed(req_id, num_tokens)):
            req.tables[g].extend(self.pools[g].allocate(n))
        req.num_tokens = max(req.num_tokens, num_tokens)

    def release_behind_window(self, req_id, num_computed: int) -> int:
        """Give back the pages of windowed groups that no position >= num_computed can read.
        Returns how many pages were freed."""
        req = self._requests[req_id]
        freed = 0
        for g in range(len(self.groups)):
            first = min(self._first_needed_page(g, num_computed), len(req.tables[g]))
            if first > req.released[g]:
                pages = [p for p in req.tables[g][req.released[g]:first] if p >= 0]
                self.pools[g].free(pages)
                for i in range(req.released[g], first):
                    req.tables[g][i] = -1
                req.released[g] = first
                freed += len(pages)
        return freed

    def free(self, req_id) -> None:
        """The request has ended (or is preempted): everything it holds goes back."""
        req = self._requests.pop(req_id)
        for g, table in enumerate(req.tables):
            self.pools[g].free([p for p in reversed(table) if p >= 0])
        if req.state_slot is not None:
            self.slots.release(req.state_slot)

    def check(self) -> None:
        """No page lost, held twice or freed twice."""
        for g, pool in enumerate(self.pools):
            pool.check()
            held = [p for r in self._requests.values() for p in r.tables[g] if p >= 0]
            assert len(held) == len(set(held)), f"group {g}: a page is held twice"
            assert set(held) == pool._used, f"group {g}: held pages and the pool's used set differ"
        if self.slots is not None:
            self.slots.check()
            held = [r.state_slot for r in self._requests.values()]
            assert len(held) == len(set(held)) and set(held) == self.slots._used
