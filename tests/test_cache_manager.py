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
