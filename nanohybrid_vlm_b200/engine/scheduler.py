"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  It decides; the cache manager keeps the books and the runner computes.

Policy, after nanovllm/engine/scheduler.py (queues :133-134, budget :544-547, portions
:836-839, preemption :350-378,492-514,906-949, no progress :898-903, finishing :972-983):

* ``waiting`` holds new, partly prefilled and preempted requests, first come first served;
  ``running`` holds requests whose prompt is done.
* One step = one mixed batch.  Running requests get one token each first ("decode_first");
  what is left of ``max_num_batched_tokens`` goes to the head of ``waiting``, whose prompt is
  cut where the budget ends and goes on from there in the next step.  With
  "prefill_first" nothing decodes while a request waits and can be served; when the head of the
  queue finds no room, the running requests decode instead, finish and make room.  (The
  reference preempts running requests for the head there, :674-719; with two requests that
  each fill the pool that never ends, so this engine lets them finish.)
* A request is admitted only if pages for all its current tokens (and a state slot, if the
  model needs one) are free and fewer than ``max_num_seqs`` requests are live; else the
  queue waits behind it.
* When a decoding request needs a page and none is free, the running request with the
  least computed tokens (ties: the oldest) that is not yet part of this step is
  preempted: its pages go back, it returns to the tail of ``waiting`` and is later
  recomputed from its first token, generated tokens included.  If there is no other, the
  request preempts itself.
* A step that can schedule nothing raises: the engine would spin.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache import CacheManager
from .sequence import PENDING, Sequence, SequenceStatus


@dataclass
class SchedulePlan:
    seqs: list[Sequence] = field(default_factory=list)     # in batch order; seq.num_scheduled_tokens is set
    num_decode_tokens: int = 0
    num_prefill_tokens: int = 0
    preempted_seq_ids: list[int] = field(default_factory=list)


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_num_seqs: int, max_num_batched_tokens: int, max_model_len: int,
                 eos: int = -1, policy: str = "decode_first", max_portion: int | None = None):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.eos = eos
        self.policy = policy
        self.max_portion = max_portion          # test hook: no portion of a prompt is longer than this
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()
        self.num_preemptions = 0
        self.num_recomputed_tokens = 0

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, seq: Sequence) -> None:
        if len(seq) >= self.max_model_len:
            raise ValueError(f"prompt of {len(seq)} tokens leaves no room to generate within max_model_len "
                             f"{self.max_model_len}")
        most = min(len(seq) + seq.max_tokens - 1, self.max_model_len)   # the last token chosen is never fed back
        for g, pool in enumerate(self.cache.pools):
            if -(-most // self.cache.page_size) > pool.num_pages:
                raise ValueError(f"request of up to {most} tokens can never fit the cache "
                                 f"({pool.num_pages} pages of {self.cache.page_size} tokens)")
        self.waiting.append(seq)

    # ------------------------------------------------------------------ one step's plan
    def schedule(self) -> SchedulePlan:
        plan = SchedulePlan()
        budget = self.max_num_batched_tokens
        scheduled: set[int] = set()

        strict_prefill = self.policy == "prefill_first" and bool(self.waiting)
        if not strict_prefill:
            budget = self._schedule_decodes(plan, budget, scheduled)

        while self.waiting and budget > 0 and len(plan.seqs) < self.max_num_seqs:
            seq = self.waiting[0]
            if seq.seq_id not in self.cache:
                live = self.cache.num_live()
                if live >= self.max_num_seqs or not self.cache.can_admit(seq.seq_id, seq.token_ids):
                    break
                # leading pages that an earlier request left in the cache are shared, not computed again
                seq.num_cached_tokens = self.cache.admit(seq.seq_id, seq.token_ids)
            remaining = len(seq) - seq.num_cached_tokens
            n = min(remaining, budget, self.max_portion or remaining)
            seq.num_scheduled_tokens = n
            plan.seqs.append(seq)
            scheduled.add(seq.seq_id)
            plan.num_prefill_tokens += n
            budget -= n
            if n == remaining:
                self.waiting.popleft()
                seq.status = SequenceStatus.RUNNING
                self.running.append(seq)
            else:
                break   # a prompt was cut: the budget (or the portion limit) is used up for this step

        if strict_prefill and not plan.seqs:
            # the head of the queue found no room (pages, state slot or max_num_seqs): the running requests
            # go on instead, so that they finish and give back what it waits for
            budget = self._schedule_decodes(plan, budget, scheduled)
        if not plan.seqs:
            raise RuntimeError("Scheduler cannot make progress: no request fits the free cache pages and budget "
                               f"(waiting {len(self.waiting)}, running {len(self.running)}, free pages "
                               f"{[p.num_free for p in self.cache.pools]})")
        return plan

    def _schedule_decodes(self, plan: SchedulePlan, budget: int, scheduled: set[int]) -> int:
        """One token for every running request, as far as the budget goes; a request that needs a page when
        none is free preempts another (or itself).  Returns what is left of the budget."""
        for seq in list(self.running):
            if seq.status != SequenceStatus.RUNNING or budget == 0 or len(plan.seqs) >= self.max_num_seqs:
                continue
            n = len(seq)
            while not (self.cache.covers(seq.seq_id, n) or self.cache.can_allocate(seq.seq_id, n)):
                victim = self._pick_victim(scheduled, exclude=seq)
                if victim is None:
                    victim = seq
                self._preempt(victim, plan)
                if victim is seq:
                    break
            if seq.status != SequenceStatus.RUNNING:
                continue
            self.cache.allocate(seq.seq_id, n)
            seq.num_scheduled_tokens = 1
            plan.seqs.append(seq)
            scheduled.add(seq.seq_id)
            plan.num_decode_tokens += 1
            budget -= 1
        return budget

    def _pick_victim(self, scheduled: set[int], exclude: Sequence) -> Sequence | None:
        candidates = [s for s in self.running
                      if s is not exclude and s.seq_id not in scheduled and s.status == SequenceStatus.RUNNING]
        if not candidates:
            return None
        return min(candidates, key=lambda s: (s.num_cached_tokens, s.seq_id))

    def _preempt(self, seq: Sequence, plan: SchedulePlan) -> None:
        self.cache.free(seq.seq_id)
        self.num_preemptions += 1
        self.num_recomputed_tokens += seq.num_cached_tokens
        seq.num_preemptions += 1
        seq.num_cached_tokens = 0
        seq.num_scheduled_tokens = 0
        seq.status = SequenceStatus.WAITING
        self.running.remove(seq)
        self.waiting.append(seq)
        plan.preempted_seq_ids.append(seq.seq_id)

    # ------------------------------------------------------------------ a step whose tokens are read later
    def advance(self, seqs: list[Sequence]) -> list[int]:
        """Book a launched step whose chosen tokens are still on the device.  A request whose portion did not reach
        its end just moves on.  One that did gets a place for its token (``PENDING``) so that the next step can
        be planned; if it has reached its length it leaves ``running`` (its cache is kept until ``resolve`` sees its
        last token).  Returns, per request, the index of the place in its token list (-1: no token was chosen)."""
        places = []
        for seq in seqs:
            seq.num_cached_tokens += seq.num_scheduled_tokens
            seq.num_scheduled_tokens = 0
            if seq.num_cached_tokens < len(seq):
                places.append(-1)
                if self.cache.prefix_cache:
                    self.cache.commit(seq.seq_id, seq.token_ids, seq.num_cached_tokens)
                if self.cache.has_windows:
                    self.cache.release_behind_window(seq.seq_id, seq.num_cached_tokens)
                continue
            places.append(len(seq))
            seq.append_token(PENDING)
            if seq.num_completion_tokens >= seq.max_tokens or len(seq) >= self.max_model_len:
                seq.finishing = True
                self.running.remove(seq)
            elif self.cache.has_windows:
                self.cache.release_behind_window(seq.seq_id, seq.num_cached_tokens)
        return places

    def resolve(self, seqs: list[Sequence], places: list[int], token_ids: list[int]) -> None:
        """The tokens of a step booked with ``advance`` have arrived (one per request that has a place, in the order
        of the requests): they take their places; a request stops at
        the end-of-sequence token (whatever a later step, launched meanwhile, computed for it is dropped) or at
        its length."""
        tokens = iter(token_ids)
        for seq, place in zip(seqs, places):
            if place < 0:
                continue                                      # a portion that did not reach its request's end
            token = next(tokens)
            if seq.is_finished or place >= len(seq):
                continue                                      # it ended at an earlier token while this step ran
            seq.token_ids[place] = token
            if self.cache.prefix_cache and seq.seq_id in self.cache:
                known = min(seq.num_cached_tokens, place + 1)
                self.cache.commit(seq.seq_id, seq.token_ids, known)
            stop = not seq.ignore_eos and token == self.eos
            if stop or (seq.finishing and place == len(seq) - 1):
                del seq.token_ids[place + 1:]
                self._finish(seq)

    def _finish(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.FINISHED
        seq.finishing = False
        if seq.seq_id in self.cache:
            self.cache.free(seq.seq_id)
        if seq in self.running:
            self.running.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)

    # ------------------------------------------------------------------ after a step that is read at once
    def postprocess(self, seqs: list[Sequence], token_ids: list[int | None]) -> None:
        """``token_ids[i]`` is the token chosen for ``seqs[i]``, or None if its portion did not reach the
        end of the request (nothing was sampled for it): ``advance`` and ``resolve`` in one."""
        for seq, token in zip(seqs, token_ids):
            if token is None and seq.num_cached_tokens + seq.num_scheduled_tokens == len(seq):
                raise RuntimeError(f"request {seq.seq_id}: its last token was computed but no token was chosen")
        places = self.advance(seqs)
        self.resolve(seqs, places, [t for t, place in zip(token_ids, places) if place >= 0])
