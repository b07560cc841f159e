"""The scheduler's decisions, without a GPU: a fake model "computes" each step."""
import pytest

from nanohybrid_vlm_b200.cache import CacheManager, GroupSpec
from nanohybrid_vlm_b200.engine.scheduler import Scheduler
from nanohybrid_vlm_b200.engine.sequence import Sequence, SequenceStatus
from nanohybrid_vlm_b200.sampling import SamplingParams


def make(num_pages=16, page_size=4, max_num_seqs=8, budget=32, max_model_len=64, eos=-1, **kw):
    cache = CacheManager([GroupSpec(None)], page_size, num_pages)
    return Scheduler(cache, max_num_seqs=max_num_seqs, max_num_batched_tokens=budget, max_model_len=max_model_len,
                     eos=eos, **kw), cache


def seq(n, max_tokens=4, **kw):
    return Sequence(list(range(1, n + 1)), SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw))


def run_step(s, token=9):
    """One step with a fake model: every request that reached its end gets `token`."""
    plan = s.schedule()
    shape = [(q.seq_id, q.num_cached_tokens, q.num_scheduled_tokens) for q in plan.seqs]
    tokens = [token if q.num_cached_tokens + q.num_scheduled_tokens == len(q) else None for q in plan.seqs]
    s.postprocess(plan.seqs, tokens)
    s.cache.check()
    return plan, shape


def test_prompts_are_cut_under_the_token_budget():
    s, cache = make(num_pages=32, budget=10)
    a, b = seq(7), seq(12)
    s.add(a); s.add(b)
    plan, shape = run_step(s)
    assert shape == [(a.seq_id, 0, 7), (b.seq_id, 0, 3)]          # b is cut where the budget ends
    assert (plan.num_prefill_tokens, plan.num_decode_tokens) == (10, 0)
    assert a.status == SequenceStatus.RUNNING and b.status == SequenceStatus.WAITING and len(a) == 8
    plan, shape = run_step(s)
    assert shape == [(a.seq_id, 7, 1), (b.seq_id, 3, 9)]          # a decodes beside b's second portion
    assert (plan.num_prefill_tokens, plan.num_decode_tokens) == (9, 1)
    plan, shape = run_step(s)
    assert shape == [(a.seq_id, 8, 1), (b.seq_id, 12, 1)]


def test_forced_portion_size_and_prefill_first():
    s, _ = make(num_pages=64, budget=64, policy="prefill_first", max_portion=5)
    a = seq(3)
    s.add(a)
    run_step(s)
    b = seq(12)
    s.add(b)
    _, shape = run_step(s)
    assert shape == [(b.seq_id, 0, 5)]                            # nothing decodes while a prompt waits
    _, shape = run_step(s)
    assert shape == [(b.seq_id, 5, 5)]
    _, shape = run_step(s)
    assert shape == [(b.seq_id, 10, 2)]
    _, shape = run_step(s)
    assert shape == [(a.seq_id, 3, 1), (b.seq_id, 12, 1)]


def test_admission_waits_for_pages_and_for_a_free_place():
    s, cache = make(num_pages=4, page_size=4, max_num_seqs=2)
    a, b, c = seq(9, max_tokens=2), seq(5, max_tokens=2), seq(2, max_tokens=2)
    for q in (a, b, c):
        s.add(q)
    _, shape = run_step(s)
    assert [x[0] for x in shape] == [a.seq_id]                    # b needs 2 pages, 1 is free; c waits behind b
    while not a.is_finished:
        run_step(s)
    _, shape = run_step(s)
    assert [x[0] for x in shape] == [b.seq_id, c.seq_id]
    s2, _ = make(num_pages=64, max_num_seqs=2)
    qs = [seq(3), seq(3), seq(3)]
    for q in qs:
        s2.add(q)
    _, shape = run_step(s2)
    assert [x[0] for x in shape] == [qs[0].seq_id, qs[1].seq_id]  # max_num_seqs live requests


def test_finishing_frees_pages():
    s, cache = make(eos=9)
    a = seq(5, max_tokens=10)
    b = seq(5, max_tokens=10, ignore_eos=True)
    s.add(a); s.add(b)
    run_step(s, token=9)                                          # a meets eos at once, b ignores it
    assert a.is_finished and not b.is_finished and a.seq_id not in cache
    for _ in range(9):
        run_step(s, token=9)
    assert b.is_finished and b.num_completion_tokens == 10 and s.is_finished()
    assert cache.pools[0].num_free == cache.pools[0].num_pages
    c = seq(60, max_tokens=100)
    s.add(c)
    while not c.is_finished:
        run_step(s, token=3)
    assert len(c) == 64                                           # stopped by max_model_len


def test_when_pages_run_out_the_request_with_least_work_is_preempted_and_recomputed():
    s, cache = make(num_pages=5, page_size=4, budget=64)
    a, b = seq(8, max_tokens=8), seq(4, max_tokens=8)
    s.add(a); s.add(b)
    run_step(s)                                                   # a holds 2 pages, b holds 1; both now 9 / 5 long
    _, shape = run_step(s)                                        # a needs a third page, b a second: 5 in use
    assert cache.pools[0].num_free == 0
    for _ in range(3):
        run_step(s)                                               # 12 / 8 long, pages full
    plan, shape = run_step(s)                                     # a needs a 4th page: b (least computed) is preempted
    assert plan.preempted_seq_ids == [b.seq_id] and [x[0] for x in shape] == [a.seq_id]
    assert b.status == SequenceStatus.WAITING and b.num_cached_tokens == 0 and b.seq_id not in cache
    assert s.num_preemptions == 1 and s.num_recomputed_tokens == 8 and len(b) == 9    # its tokens are kept
    while not a.is_finished:
        plan, shape = run_step(s)
        assert all(x[0] == a.seq_id for x in shape)               # b cannot come back while a holds the pages
    _, shape = run_step(s)
    assert shape == [(b.seq_id, 0, 9)]                            # recomputed from its first token, generated ones too
    while not s.is_finished():
        run_step(s)
    assert b.num_completion_tokens == 8 and cache.pools[0].num_free == 5


def test_a_lone_request_preempts_itself_and_then_nothing_can_progress():
    s, cache = make(num_pages=2, page_size=4, max_model_len=64)
    a = seq(7, max_tokens=1)
    s.add(a)                                                      # fits: 7 + 1 tokens = 2 pages
    run_step(s)
    assert a.is_finished
    with pytest.raises(ValueError, match="never fit"):
        s.add(seq(7, max_tokens=5))                               # could need 3 pages
    with pytest.raises(ValueError, match="max_model_len"):
        s.add(seq(64))
    with pytest.raises(RuntimeError, match="cannot make progress"):
        s.schedule()


@pytest.mark.parametrize("policy", ["decode_first", "prefill_first"])
def test_a_pool_smaller_than_the_work_is_worked_off_under_both_policies(policy):
    """4 pages of 4 tokens, two requests of 9 tokens (3 pages each): the second can be admitted only when
    the first has finished.  Under "prefill_first" the first decodes on while the second waits for room."""
    s, cache = make(num_pages=4, page_size=4, policy=policy)
    a, b = seq(9, max_tokens=3), seq(9, max_tokens=3)
    s.add(a); s.add(b)
    _, shape = run_step(s)
    assert shape == [(a.seq_id, 0, 9)]
    _, shape = run_step(s)
    assert shape == [(a.seq_id, 9, 1)]                            # b finds no room, a goes on
    steps = 2
    while not s.is_finished():
        run_step(s)
        steps += 1
        assert steps < 20
    assert a.num_completion_tokens == 3 and b.num_completion_tokens == 3
    assert cache.pools[0].num_free == 4 and s.num_preemptions == 0


@pytest.mark.parametrize("policy", ["decode_first", "prefill_first"])
def test_more_requests_than_places_and_pages_all_finish(policy):
    """More requests than max_num_seqs, in a pool that holds two of them at a time, arriving while others
    run: every one finishes with all its tokens, whatever the policy, and every page comes back."""
    import random
    rng = random.Random(3)
    s, cache = make(num_pages=6, page_size=4, max_num_seqs=2, budget=16, policy=policy, max_model_len=32)
    todo = [seq(rng.randint(1, 10), max_tokens=rng.randint(1, 6)) for _ in range(9)]
    all_seqs = list(todo)
    for q in todo[:3]:
        s.add(q)
    todo = todo[3:]
    steps = 0
    while todo or not s.is_finished():
        if todo and (steps % 2 == 0 or s.is_finished()):
            s.add(todo.pop(0))
        plan, _ = run_step(s)
        if policy == "prefill_first" and plan.num_prefill_tokens:
            assert plan.num_decode_tokens == 0                    # nothing decodes beside a prompt portion
        steps += 1
        assert steps < 400
    assert all(q.is_finished and q.num_completion_tokens == q.max_tokens for q in all_seqs)
    assert cache.pools[0].num_free == 6
