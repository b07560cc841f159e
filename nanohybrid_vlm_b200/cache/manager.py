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

Prefix reuse (the reference's default for this architecture, nanovllm/engine/block_manager.py:102-108,
696-749, 811-825): every full page gets a hash chained over the page's token ids and the hash of the page
before it; a new request whose leading pages hash (and compare) equal to pages still in the pool shares
them instead of computing them.  The last page of a request is never shared, so at least one token is
always computed.  Reuse is only offered when every group keeps all keys and the model has no fixed-size
state: a window or a state cannot be rebuilt from shared pages.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass

import numpy as np

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
    serial: int = 0                         # a number no other request record of this manager ever had
    hashed: int = 0                         # leading full pages whose content hash has been taken (prefix reuse)
    chain: int = 0                          # the hash of the last of them (0: none yet)


class CacheManager:
    def __init__(self, groups: list[GroupSpec], page_size: int, num_pages: int | list[int], num_state_slots: int = 0,
                 enable_prefix_cache: bool = False):
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
        if enable_prefix_cache and not self.prefix_cache_possible(self.groups, num_state_slots):
            raise ValueError("prefix reuse needs groups that keep every key and a model without per-request state")
        self.prefix_cache = enable_prefix_cache
        self.has_windows = any(g.window is not None for g in self.groups)
        self._serial = 0
        # per group: hash -> page, and for every page that carries a hash: (hash, its token ids)
        self._by_hash: list[dict[int, int]] = [{} for _ in self.groups]
        self._page_info: list[dict[int, tuple[int, tuple]]] = [{} for _ in self.groups]
        self.prefix_hits = 0            # pages shared instead of computed, over the manager's life

    @staticmethod
    def prefix_cache_possible(groups, num_state_slots: int) -> bool:
        return num_state_slots == 0 and all(g.window is None for g in groups)

    # ------------------------------------------------------------------ prefix reuse
    @staticmethod
    def _page_hash(prev: int, tokens) -> int:
        h = hashlib.blake2b(digest_size=8)
        h.update(int(prev).to_bytes(8, "little", signed=False))
        h.update(np.asarray(tokens, dtype=np.int64).tobytes())
        return int.from_bytes(h.digest(), "little")

    def _probe(self, token_ids) -> list[list[int]]:
        """Per group: the pages that hold the request's leading full pages already (never its last page)."""
        ps = self.page_size
        n_lookup = (-(-len(token_ids) // ps)) - 1
        hits: list[list[int]] = [[] for _ in self.groups]
        prev = 0
        for i in range(max(0, n_lookup)):
            chunk = tuple(token_ids[i * ps:(i + 1) * ps])
            prev = self._page_hash(prev, chunk)
            found = []
            for g in range(len(self.groups)):
                page = self._by_hash[g].get(prev)
                if page is None or self._page_info[g].get(page, (None, None))[1] != chunk:
                    found = None
                    break
                found.append(page)
            if found is None:
                break
            for g, page in enumerate(found):
                hits[g].append(page)
        return hits

    def can_admit(self, req_id, token_ids) -> bool:
        """Room for a new request's tokens, counting the pages it can share."""
        if not self.prefix_cache or req_id in self._requests:
            return self.can_allocate(req_id, len(token_ids))
        total = -(-len(token_ids) // self.page_size)
        for g, pages in enumerate(self._probe(token_ids)):
            from_free = sum(1 for p in pages if self.pools[g].is_free(p))
            if total - len(pages) + from_free > self.pools[g].num_free:
                return False
        return True

    def admit(self, req_id, token_ids) -> int:
        """Pages for a new request's tokens; returns how many leading tokens are already in the cache
        (a multiple of the page size; 0 without prefix reuse)."""
        if not self.prefix_cache or req_id in self._requests:
            self.allocate(req_id, len(token_ids))
            return 0
        if not self.can_admit(req_id, token_ids):
            raise OutOfPages(f"request {req_id!r}: no room for {len(token_ids)} tokens "
                             f"(free pages per group: {[p.num_free for p in self.pools]})")
        hits = self._probe(token_ids)
        req = self._requests[req_id] = _Request([[] for _ in self.groups], [0] * len(self.groups), None)
        self._serial += 1
        req.serial = self._serial
        for g, pages in enumerate(hits):
            for page in pages:
                self.pools[g].share(page)
            req.tables[g].extend(pages)
        n_hit = len(hits[0]) if hits else 0
        self.prefix_hits += n_hit
        if n_hit:
            req.hashed = n_hit
            req.chain = self._page_info[0][hits[0][-1]][0]
        self.allocate(req_id, len(token_ids))
        return n_hit * self.page_size

    def commit(self, req_id, token_ids, num_computed: int) -> None:
        """After a step: the request's pages that are now full and computed get their hashes, so that later
        requests can find them."""
        if not self.prefix_cache:
            return
        req = self._requests.get(req_id)
        if req is None:
            return
        ps = self.page_size
        full = min(num_computed, len(token_ids)) // ps
        if full <= req.hashed:
            return                                  # the usual step: no page has filled up
        # every group holds the same tokens, so one chain of hashes serves all of them
        prev = req.chain
        for j in range(req.hashed, full):
            chunk = tuple(token_ids[j * ps:(j + 1) * ps])
            prev = self._page_hash(prev, chunk)
            for g in range(len(self.groups)):
                page = req.tables[g][j]
                if prev not in self._by_hash[g]:
                    self._by_hash[g][prev] = page
                    self._page_info[g][page] = (prev, chunk)
                # else the same contents already sit on another page: this one stays anonymous
        req.hashed, req.chain = full, prev

    def _forget(self, g: int, pages) -> None:
        """Pages that are handed out for new contents lose their hashes."""
        for p in pages:
            info = self._page_info[g].pop(p, None)
            if info is not None and self._by_hash[g].get(info[0]) == p:
                del self._by_hash[g][info[0]]

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

    def covers(self, req_id, num_tokens: int) -> bool:
        """True if the request's pages already cover tokens [0, num_tokens) in every group (the usual decode step)."""
        req = self._requests.get(req_id)
        if req is None:
            return False
        total = -(-num_tokens // self.page_size)
        for t in req.tables:
            if len(t) < total:
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
        req = self._requests.get(req_id)
        if req is not None:
            # the usual decode step: the pages the request holds already cover the new token
            total = -(-num_tokens // self.page_size)
            if all(len(t) >= total for t in req.tables):
                if num_tokens > req.num_tokens:
                    req.num_tokens = num_tokens
                return
        if not self.can_allocate(req_id, num_tokens):
            raise OutOfPages(f"request {req_id!r}: no room for {num_tokens} tokens "
                             f"(free pages per group: {[p.num_free for p in self.pools]})")
        req = self._requests.get(req_id)
        if req is None:
            slot = self.slots.allocate() if self.slots is not None else None
            req = self._requests[req_id] = _Request([[] for _ in self.groups], [0] * len(self.groups), slot)
            self._serial += 1
            req.serial = self._serial
        for g, n in enumerate(self.pages_needed(req_id, num_tokens)):
            fresh = self.pools[g].allocate(n)
            if self.prefix_cache:
                self._forget(g, fresh)
            req.tables[g].extend(fresh)
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
            if not self.prefix_cache:
                assert len(held) == len(set(held)), f"group {g}: a page is held twice"
            assert set(held) == pool._used, f"group {g}: held pages and the pool's used set differ"
            for p in set(held):
                assert pool.ref_count(p) == held.count(p), f"group {g}: page {p} has the wrong number of holders"
            for h, p in self._by_hash[g].items():
                assert self._page_info[g][p][0] == h, f"group {g}: the hash tables disagree about page {p}"
        if self.slots is not None:
            self.slots.check()
            held = [r.state_slot for r in self._requests.values()]
            assert len(held) == len(set(held)) and set(held) == self.slots._used
