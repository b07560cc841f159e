"""The cache manager's books: no page lost, held twice or freed twice, under random orders of
requests; first-in first-out reuse; windowed groups give pages back early; state slots."""
import numpy as np
import pytest

from nanohybrid_vlm_b200.cache import CacheManager, GroupSpec, OutOfPages, PagePool, StateSlotAllocator


def test_pool_is_first_in_first_out():
    pool = PagePool(4)
    assert pool.allocate(3) == [0, 1, 2]
    pool.free([1])
    pool.free([0])
    assert pool.allocate(3) == [3, 1, 0]          # freed pages come back in the order they were freed
    with pytest.raises(OutOfPages):
        pool.allocate(1)
    with pytest.raises(RuntimeError, match="twice"):
        pool.free([2, 2])
    pool.free([2])
    with pytest.raises(RuntimeError, match="twice"):
        pool.free([2])
    pool.check()


def test_state_slots():
    slots = StateSlotAllocator(2)
    a, b = slots.allocate(), slots.allocate()
    assert (a, b) == (0, 1) and not slots.can_allocate()
    with pytest.raises(OutOfPages):
        slots.allocate()
    slots.release(a)
    with pytest.raises(RuntimeError):
        slots.release(a)
    assert slots.allocate() == 0
    slots.check()


def test_tables_grow_page_by_page():
    cm = CacheManager([GroupSpec(None)], page_size=8, num_pages=5)
    cm.allocate("a", 9)
    assert cm.block_table("a") == [0, 1] and cm.state_slot("a") is None
    cm.allocate("a", 16)
    assert cm.block_table("a") == [0, 1]            # still fits
    cm.allocate("a", 17)
    assert cm.block_table("a") == [0, 1, 2]
    assert cm.pages_needed("b", 24) == [3] and not cm.can_allocate("b", 24)
    with pytest.raises(OutOfPages):
        cm.allocate("b", 24)
    assert "b" not in cm and cm.pools[0].num_free == 2   # a failed allocation changes nothing
    cm.free("a")
    cm.allocate("b", 24)
    assert cm.block_table("b") == [3, 4, 2]          # reused pages: last freed first (reverse order), after the never-used ones
    cm.check()


def test_window_group_gives_pages_back_early():
    cm = CacheManager([GroupSpec(None), GroupSpec(10)], page_size=4, num_pages=[16, 16])
    cm.allocate("a", 30)
    assert len(cm.block_table("a", 0)) == 8 and len(cm.block_table("a", 1)) == 8
    # after 30 computed tokens the next query (position 30) reads keys 21..30: pages 0..4 are done with
    assert cm.release_behind_window("a", 30) == 5
    assert cm.block_table("a", 1)[:5] == [-1] * 5 and all(p >= 0 for p in cm.block_table("a", 1)[5:])
    assert all(p >= 0 for p in cm.block_table("a", 0))
    assert cm.release_behind_window("a", 30) == 0
    cm.allocate("a", 33)
    assert len(cm.block_table("a", 1)) == 9 and cm.pools[1].num_used == 4
    cm.check()
    cm.free("a")
    assert cm.pools[0].num_free == 16 and cm.pools[1].num_free == 16
    cm.check()


def test_requests_need_a_state_slot_when_the_model_has_state():
    cm = CacheManager([GroupSpec(None)], page_size=4, num_pages=100, num_state_slots=2)
    cm.allocate("a", 3)
    cm.allocate("b", 3)
    assert {cm.state_slot("a"), cm.state_slot("b")} == {0, 1}
    assert not cm.can_allocate("c", 3)
    with pytest.raises(OutOfPages):
        cm.allocate("c", 3)
    cm.free("a")
    cm.allocate("c", 3)
    assert cm.state_slot("c") == 0
    cm.check()


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_the_books_straight(seed):
    rng = np.random.default_rng(seed)
    cm = CacheManager([GroupSpec(None), GroupSpec(int(rng.integers(5, 40)))], page_size=int(rng.integers(1, 9)),
                      num_pages=[60, 60], num_state_slots=5)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.3 and len(live) < 5:
            n = int(rng.integers(1, 50))
            if cm.can_allocate(next_id, n):
                cm.allocate(next_id, n)
                live[next_id] = n
            else:
                with pytest.raises(OutOfPages):
                    cm.allocate(next_id, n)
            next_id += 1
        elif action < 0.75 and live:
            rid = int(rng.choice(list(live)))
            n = live[rid] + int(rng.integers(1, 12))
            if cm.can_allocate(rid, n):
                cm.allocate(rid, n)
                live[rid] = n
                cm.release_behind_window(rid, n - int(rng.integers(0, 3)))
        elif live:
            rid = int(rng.choice(list(live)))
            cm.free(rid)
            del live[rid]
            with pytest.raises(KeyError):
                cm.free(rid)
        cm.check()
        for rid, n in live.items():
            table = cm.block_table(rid, 0)
            assert len(table) == -(-n // cm.page_size) and all(p >= 0 for p in table)
    for rid in list(live):
        cm.free(rid)
    cm.check()
    assert all(pool.num_free == pool.num_pages for pool in cm.pools) and cm.slots.num_free == 5


def test_prefix_reuse_shares_full_pages_but_never_the_last():
    cm = CacheManager([GroupSpec(None)], page_size=4, num_pages=12, enable_prefix_cache=True)
    a = list(range(100, 114))                                  # 14 tokens: pages 0,1,2 full, page 3 partial
    assert cm.admit("a", a) == 0 and cm.block_table("a") == [0, 1, 2, 3]
    cm.commit("a", a, 14)
    b = a[:10] + [7, 7, 7]                                     # shares two full pages, differs in the third
    assert cm.can_admit("b", b)
    assert cm.admit("b", b) == 8 and cm.block_table("b")[:2] == [0, 1] and cm.prefix_hits == 2
    assert cm.pools[0].ref_count(0) == 2 and cm.pools[0].ref_count(2) == 1
    cm.check()
    c = a[:8]                                                  # exactly two pages: the last is never shared
    assert cm.admit("c", c) == 4 and cm.block_table("c")[0] == 0 and cm.block_table("c")[1] not in (1,)
    cm.check()
    cm.free("a")
    assert cm.pools[0].ref_count(0) == 2 and cm.pools[0].ref_count(1) == 1    # still held by b (and c)
    cm.free("b"); cm.free("c")
    assert cm.pools[0].num_free == 12
    # freed pages keep their contents until they are handed out again: the same prompt finds them
    assert cm.admit("d", a) == 12 and cm.block_table("d")[:3] == [0, 1, 2]
    cm.check()
    cm.free("d")
    # a page that is handed out for other contents forgets its hash
    filler = list(range(500, 548))
    cm.admit("e", filler)                                       # takes all 12 pages
    cm.free("e")
    assert cm.admit("f", a) == 0
    cm.check()


def test_prefix_reuse_counts_shared_free_pages_against_the_free_pool():
    cm = CacheManager([GroupSpec(None)], page_size=4, num_pages=4, enable_prefix_cache=True)
    a = list(range(16))
    cm.admit("a", a); cm.commit("a", a, 16); cm.free("a")       # all four pages free, three of them findable
    b = a[:12] + [99] * 8                                       # needs 5 pages, shares 3: 2 fresh + 3 taken from the free queue
    assert not cm.can_admit("b", b)
    with pytest.raises(OutOfPages):
        cm.admit("b", b)
    assert "b" not in cm and cm.pools[0].num_free == 4
    c = a[:12] + [99]                                           # 4 pages, shares 3
    assert cm.can_admit("c", c) and cm.admit("c", c) == 12
    cm.check()


def test_prefix_reuse_is_refused_for_windows_and_state():
    with pytest.raises(ValueError):
        CacheManager([GroupSpec(None), GroupSpec(8)], page_size=4, num_pages=8, enable_prefix_cache=True)
    with pytest.raises(ValueError):
        CacheManager([GroupSpec(None)], page_size=4, num_pages=8, num_state_slots=2, enable_prefix_cache=True)


@pytest.mark.parametrize("seed", range(3))
def test_prefix_reuse_random_orders(seed):
    rng = np.random.default_rng(seed)
    cm = CacheManager([GroupSpec(None)], page_size=4, num_pages=40, enable_prefix_cache=True)
    stems = [rng.integers(0, 50, 24).tolist() for _ in range(3)]
    live = {}
    for step in range(400):
        if rng.random() < 0.5 and len(live) < 5:
            toks = stems[int(rng.integers(3))][:int(rng.integers(1, 25))] + rng.integers(50, 60, int(rng.integers(0, 6))).tolist()
            if cm.can_admit(step, toks):
                cached = cm.admit(step, toks)
                assert cached % 4 == 0 and cached < len(toks)
                live[step] = toks
                cm.commit(step, toks, len(toks))
        elif live:
            rid = int(rng.choice(list(live)))
            if rng.random() < 0.5:
                live[rid] = live[rid] + [int(rng.integers(0, 60))]
                if cm.can_allocate(rid, len(live[rid])):
                    cm.allocate(rid, len(live[rid]))
                    cm.commit(rid, live[rid], len(live[rid]))
                else:
                    live[rid].pop()
            else:
                cm.free(rid)
                del live[rid]
        cm.check()
    for rid in list(live):
        cm.free(rid)
    cm.check()
    assert cm.pools[0].num_free == 40 and cm.prefix_hits > 0


def test_a_page_is_hashed_once_even_when_its_contents_sit_elsewhere(monkeypatch):
    """Committing after every step costs a hash only when a page fills up: also for a request whose full page
    repeats contents that another page already holds (that page stays anonymous), and for a request that began
    behind shared pages (its chain continues from the last of them)."""
    cm = CacheManager([GroupSpec(None)], page_size=4, num_pages=16, enable_prefix_cache=True)
    calls = []
    real = CacheManager._page_hash
    monkeypatch.setattr(CacheManager, "_page_hash", staticmethod(lambda prev, toks: calls.append(tuple(toks)) or real(prev, toks)))
    a = list(range(10))
    cm.admit("a", a)
    calls.clear()                                               # (admission hashes too: it looks pages up)
    cm.commit("a", a, 10)                                       # two full pages
    assert calls == [tuple(a[:4]), tuple(a[4:8])]
    cm.commit("a", a, 10)
    assert len(calls) == 2                                      # nothing new: nothing hashed
    cm.free("a")                                                # the pages are free but still findable
    b = a[:8] + [50, 51]                                        # b: first page shared, second (the same contents
    assert cm.admit("b", b[:8]) == 4                            # as a's, whose page still holds that hash) its own:
    calls.clear()                                               # the last page of what is admitted is never shared
    cm.commit("b", b[:8], 8)
    assert calls == [tuple(a[4:8])]                             # one new page: hashed once (and left anonymous)
    for n in range(9, 11):                                      # decode steps inside the third page: no hashing
        cm.allocate("b", n)
        cm.commit("b", b[:n], n)
    assert len(calls) == 1
    b += [52, 53]
    cm.allocate("b", 12)
    cm.commit("b", b, 12)                                       # the third page is full now
    assert calls[1:] == [tuple(b[8:12])]
    # and the chain through the anonymous page is the right one: a request with b's tokens finds pages 1 and 3
    probe = cm._probe(b + [0])
    assert len(probe[0]) == 3
    cm.check()


def test_covers_tells_whether_pages_are_needed():
    cm = CacheManager([GroupSpec(None), GroupSpec(6)], page_size=4, num_pages=[8, 8])
    assert not cm.covers("x", 1)
    cm.allocate("x", 5)
    assert cm.covers("x", 8) and not cm.covers("x", 9)
    cm.allocate("x", 7)                                         # no page needed: only the count moves
    assert cm.num_tokens("x") == 7 and cm.block_table("x", 0) == [0, 1]
    cm.allocate("x", 9)
    assert cm.block_table("x", 0) == [0, 1, 2] and cm.covers("x", 12)
    cm.check()
