"""Fixed-size cache pages and slots of per-request state: the bookkeeping, on the host.

:class:`PagePool` hands out page ids first-in first-out: a page that was given back goes
to the tail of the free queue and comes out again after the pages freed before it
(nanovllm/engine/block_manager.py:96-131 keeps a deque and a used set the same way), so a
trace with few pages reuses them in an order that tests can predict.
:class:`StateSlotAllocator` does the same for slots of fixed-size state
(nanovllm/engine/hybrid_state.py:19-83).
"""
from __future__ import annotations

from collections import deque


class OutOfPages(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must not be negative")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(num_pages))
        self._used: set[int] = set()
        self._refs: dict[int, int] = {}         # holders of each used page (more than one only with prefix reuse)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return len(self._used)

    def allocate(self, n: int) -> list[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.popleft() for _ in range(n)]
        self._used.update(pages)
        for p in pages:
            self._refs[p] = 1
        return pages

    def share(self, page: int) -> None:
        """One more holder for `page`: a used page gets another reference; a free page (whose contents a
        prefix lookup found still intact) leaves the free queue and is used again."""
        if page in self._used:
            self._refs[page] += 1
        else:
            self._free.remove(page)
            self._used.add(page)
            self._refs[page] = 1

    def is_free(self, page: int) -> bool:
        return page not in self._used

    def ref_count(self, page: int) -> int:
        return self._refs.get(page, 0)

    def free(self, pages) -> None:
        pages = list(pages)
        bad = [p for p in pages if p not in self._used]
        if bad or len(set(pages)) != len(pages):
            raise RuntimeError(f"pages freed twice or never allocated: {bad or pages}")
        for p in pages:
            self._refs[p] -= 1
            if self._refs[p] == 0:
                del self._refs[p]
                self._used.remove(p)
                self._free.append(p)

    def check(self) -> None:
        """Every page is either free or used, exactly once."""
        free = list(self._free)
        assert len(set(free)) == len(free), "a page is in the free queue twice"
        assert not (set(free) & self._used), "a page is both free and used"
        assert len(free) + len(self._used) == self.num_pages, "a page was lost"
        assert set(self._refs) == self._used and all(r > 0 for r in self._refs.values()), "reference counts are off"


class StateSlotAllocator:
    def __init__(self, num_slots: int):
        if num_slots < 0:
            raise ValueError("num_slots must not be negative")
        self.num_slots = num_slots
        self._free: deque[int] = deque(range(num_slots))
        self._used: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def can_allocate(self) -> bool:
        return bool(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages(f"no state slot free of {self.num_slots}")
        slot = self._free.popleft()
        self._used.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._used:
            raise RuntimeError(f"state slot {slot} released twice or never allocated")
        self._used.remove(slot)
        self._free.append(slot)

    def check(self) -> None:
        free = list(self._free)
        assert len(set(free)) == len(free) and not (set(free) & self._used)
        assert len(free) + len(self._used) == self.num_slots
