"""The batch builder's arrays on the host, without a GPU: whatever steps came before (decode steps over the
same requests, whose block-table rows are kept in the buffer, requests swapped at a row, other batch sizes,
mixed steps, failed builds), the tables and slots that a step copies are the cache manager's own."""
import random

import numpy as np
import pytest

from nanohybrid_vlm_b200.cache import CacheManager, GroupSpec
from nanohybrid_vlm_b200.engine.batch import BatchBuilder, StepItem

VOCAB = 50


def make(num_pages=64, page_size=4, groups=None, max_seqs=8, max_pages=16):
    cm = CacheManager(groups or [GroupSpec(None)], page_size, num_pages)
    return cm, BatchBuilder(cm, VOCAB, "cpu", max_tokens=64, max_seqs=max_seqs, max_pages_per_seq=max_pages)


def check_against_manager(cm, builder, items, batch, pad_to=None):
    """Every array of the step, from the cache manager's books."""
    ps = cm.page_size
    S = pad_to or len(items)
    t = 0
    for s, it in enumerate(items):
        n = len(it.tokens)
        assert batch.host_cu_q[s] == t
        assert batch.token_ids[t:t + n].tolist() == it.tokens
        assert batch.positions[t:t + n].tolist() == list(range(it.start, it.start + n))
        assert int(batch.kv_len[s]) == it.start + n and int(batch.q_start[s]) == it.start
        for g, gt in enumerate(batch.groups):
            table = cm.block_table(it.req_id, g)
            row = gt.block_tables[s].tolist()
            k = min(len(table), len(row))
            assert row[:k] == list(table[:k]), f"row {s} of group {g} is not request {it.req_id!r}'s table"
            assert all(x == -1 for x in row[k:])
            for j in range(n):
                p = it.start + j
                page = table[p // ps]
                assert int(gt.slot_mapping[t + j]) == (page * ps + p % ps if page >= 0 else -1)
        t += n
    for s in range(len(items), S):          # idle entries read no page and store nowhere
        for gt in batch.groups:
            assert set(gt.block_tables[s].tolist()) == {-1} and int(gt.slot_mapping[t]) == -1
        assert int(batch.kv_len[s]) == 1
        t += 1


def decode_items(cm, held, rids):
    items = []
    for r in rids:
        cm.allocate(r, held[r] + 1)
        items.append(StepItem(r, [held[r] % VOCAB], held[r], [0]))
        held[r] += 1
    return items


def test_a_request_swapped_at_a_row_with_an_equal_table_length():
    cm, b = make()
    held = {}
    for r, n in (("a", 5), ("b", 6), ("c", 9)):
        cm.allocate(r, n)
        held[r] = n
    for _ in range(2):
        items = decode_items(cm, held, ["a", "b", "c"])
        check_against_manager(cm, b, items, b.build(items, table_width=8, pad_to=4), pad_to=4)
    b_pages = list(cm.block_table("b"))
    held.pop("b")
    cm.free("b")
    cm.allocate("d", 6)                       # another request at b's row, with as many pages as b had in the last step
    held["d"] = 6
    assert len(cm.block_table("d")) == len(b_pages) == 2 and cm.block_table("d") != b_pages
    items = decode_items(cm, held, ["a", "d", "c"])
    check_against_manager(cm, b, items, b.build(items, table_width=8, pad_to=4), pad_to=4)
    # the same request given up and admitted again under its old name (a preempted request coming back)
    n = held["a"]
    cm.free("a")
    cm.allocate("x", 3)                       # takes the pages a had, so that a's new ones differ
    cm.allocate("a", n)
    items = decode_items(cm, held, ["a", "d", "c"])
    check_against_manager(cm, b, items, b.build(items, table_width=8, pad_to=4), pad_to=4)


def test_a_failed_build_leaves_no_kept_rows_behind():
    cm, b = make()
    held = {}
    for r, n in (("a", 5), ("b", 6)):
        cm.allocate(r, n)
        held[r] = n
    items = decode_items(cm, held, ["a", "b"])
    b.build(items, table_width=8, pad_to=2)
    # a step of the same shape that fails after it rewrote row 0: c at a's row, then a token id out of range
    cm.allocate("c", 7)
    bad = [StepItem("c", [1], 6, [0]), StepItem("b", [VOCAB + 3], held["b"] - 1, [0])]
    with pytest.raises(ValueError, match="token ids"):
        b.build(bad, table_width=8, pad_to=2)
    again = [StepItem("a", [1], held["a"] - 1, [0]), StepItem("b", [2], held["b"] - 1, [0])]
    check_against_manager(cm, b, again, b.build(again, table_width=8, pad_to=2), pad_to=2)
    # and one that fails before any row is written: a request whose pages do not cover the step
    with pytest.raises(RuntimeError, match="pages cover"):
        b.build([StepItem("a", [1], held["a"] + 9, [0]), StepItem("b", [2], held["b"] - 1, [0])], table_width=8, pad_to=2)
    check_against_manager(cm, b, again, b.build(again, table_width=8, pad_to=2), pad_to=2)


@pytest.mark.parametrize("windowed", [False, True])
@pytest.mark.parametrize("seed", range(6))
def test_random_runs_of_steps(seed, windowed):
    """Random lives of requests: decode steps in changing company and batch size (padded to a bucket or not),
    prompt portions beside decoded tokens, requests that end, are given up and come back, few pages."""
    rng = random.Random(seed)
    groups = [GroupSpec(None), GroupSpec(6)] if windowed else [GroupSpec(None)]
    cm, b = make(num_pages=40, page_size=4, groups=groups)
    held: dict[str, int] = {}
    names = iter(f"r{i}" for i in range(10 ** 6))
    for step in range(300):
        live = list(held)
        kind = rng.random()
        if kind < 0.15 and len(live) < 6 or not live:
            r = next(names)
            n = rng.randint(1, 9)
            if not cm.can_allocate(r, n):
                continue
            cm.allocate(r, n)
            held[r] = n
            others = [x for x in live if rng.random() < 0.5 and cm.can_allocate(x, held[x] + 1)][:3]
            items = [StepItem(r, [rng.randrange(VOCAB) for _ in range(n)], 0, [n - 1])]
            for x in others:                                     # a mixed step: decoded tokens beside the prompt
                if not cm.can_allocate(x, held[x] + 1):
                    continue
                items += decode_items(cm, held, [x])
            rng.shuffle(items)
            check_against_manager(cm, b, items, b.build(items))
        elif kind < 0.25:
            r = rng.choice(live)
            n = held.pop(r)
            cm.free(r)
            if rng.random() < 0.5 and cm.can_allocate(r, n):     # given up and recomputed later under the same name
                cm.allocate(r, n)
                held[r] = n
        else:
            rids = [x for x in live if held[x] < 40]
            if rng.random() < 0.3:
                rids = rng.sample(rids, rng.randint(1, len(rids))) if rids else []
            ok = []
            for x in rids:
                if cm.can_allocate(x, held[x] + 1):
                    ok += [x]
                    cm.allocate(x, held[x] + 1)
            if not ok:
                continue
            items = decode_items(cm, held, ok)
            bucket = next(k for k in (1, 2, 4, 8) if k >= len(items)) if rng.random() < 0.8 else None
            batch = b.build(items, table_width=12 if bucket else None, pad_to=bucket)
            check_against_manager(cm, b, items, batch, pad_to=bucket)
            for x in ok:
                cm.release_behind_window(x, held[x])
        cm.check()
