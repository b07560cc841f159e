"""The engine behind ``LLM``: requests in, tokens out (nanovllm/engine/llm_engine.py:176-993).

``LLM(path, **options).generate(prompts, sampling_params)`` as in the reference:
prompts are strings (needs the folder's tokenizer) or lists of token ids; the result is a
list of ``{"text", "token_ids"}`` in the order of the prompts.  ``add_request``, ``step`` and
``is_finished`` are public for callers that feed requests while others run.  One ``step``
is one mixed batch: prompt portions beside decoded tokens.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from time import perf_counter

from ..config import Config
from ..sampling.params import SamplingParams
from .batch import StepItem
from .runner import ModelRunner
from .scheduler import Scheduler
from .sequence import PENDING, Sequence


@dataclass(slots=True)
class StepStats:
    """Token counts and time of one step (nanovllm/engine/llm_engine.py:27-62).  Prompt portions and
    decoded tokens run in one batch here, so both rates share the step's time."""
    num_decode_tokens: int = 0
    num_prefill_tokens: int = 0
    elapsed: float = 0.0

    @property
    def decode_throughput(self) -> float:
        return self.num_decode_tokens / self.elapsed if self.num_decode_tokens and self.elapsed else 0.0

    @property
    def prefill_throughput(self) -> float:
        return self.num_prefill_tokens / self.elapsed if self.num_prefill_tokens and self.elapsed else 0.0


@dataclass(slots=True)
class RequestMetrics:
    """A request's life in times (nanovllm/engine/llm_engine.py:64-174)."""
    seq_id: int
    num_prompt_tokens: int
    arrival_time: float
    first_scheduled_time: float | None = None
    first_token_time: float | None = None
    finish_time: float | None = None
    num_completion_tokens: int = 0

    @property
    def queue_ms(self):
        return None if self.first_scheduled_time is None else (self.first_scheduled_time - self.arrival_time) * 1e3

    @property
    def ttft_ms(self):
        return None if self.first_token_time is None else (self.first_token_time - self.arrival_time) * 1e3

    @property
    def tpot_ms(self):
        if self.first_token_time is None or self.finish_time is None:
            return None
        if self.num_completion_tokens <= 1:
            return 0.0
        return (self.finish_time - self.first_token_time) * 1e3 / (self.num_completion_tokens - 1)

    @property
    def e2e_ms(self):
        return None if self.finish_time is None else (self.finish_time - self.arrival_time) * 1e3


def validate_token_ids(token_ids) -> None:
    """nanovllm/inputs.py:29-56: a non-empty list of non-negative ints (bools are not ints here)."""
    if not isinstance(token_ids, list):
        raise TypeError("token_ids must be a list")
    if not token_ids:
        raise ValueError("token_ids must not be empty")
    for t in token_ids:
        if not isinstance(t, int) or isinstance(t, bool):
            raise TypeError("Every token ID must be an integer")
        if t < 0:
            raise ValueError("Token IDs must be non-negative")


class LLMEngine:
    def __init__(self, model, *, random_weights_seed: int | None = None, max_portion: int | None = None, **kwargs):
        unknown = set(kwargs) - Config.option_names()
        if unknown:
            raise TypeError(f"unknown engine options {sorted(unknown)}; known: {sorted(Config.option_names())}")
        self.config = config = Config(os.fspath(model), **kwargs)
        self.model_runner = ModelRunner(config, random_weights_seed=random_weights_seed)
        self.tokenizer = self._load_tokenizer(config.model)
        if config.eos == -1 and self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            config.eos = self.tokenizer.eos_token_id
        self.scheduler = Scheduler(self.model_runner.cache, max_num_seqs=config.max_num_seqs,
                                   max_num_batched_tokens=config.max_num_batched_tokens,
                                   max_model_len=config.max_model_len, eos=config.eos,
                                   policy=config.scheduler_policy, max_portion=max_portion)
        self.request_metrics: dict[int, RequestMetrics] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.last_sampled_ids: list[int] = []   # requests of the last step that chose a token, in the order of the
                                                # rows of ``model_runner.last_logits``
        # a launched decode step whose tokens the host has not read yet: (requests, their places, handle, time)
        self._inflight = None
        self.async_decode = bool(config.async_decode) and not config.enforce_eager

    @staticmethod
    def _load_tokenizer(model_dir: str):
        names = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "tokenizer.model")
        if not any(os.path.isfile(os.path.join(model_dir, n)) for n in names):
            return None
        from transformers import AutoTokenizer   # text in and out only; no model code
        return AutoTokenizer.from_pretrained(model_dir, use_fast=True)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt, sampling_params: SamplingParams) -> int:
        arrival = perf_counter()
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer, and the model folder has none; pass token ids")
            token_ids = self.tokenizer.encode(prompt)
        elif isinstance(prompt, list):
            validate_token_ids(prompt)
            token_ids = prompt.copy()
        else:
            raise TypeError("prompt must be a string or a list of token IDs")
        if max(token_ids) >= self.model_runner.vocab_size:
            raise ValueError(f"Token IDs must be below the vocabulary size {self.model_runner.vocab_size}")
        seq = Sequence(token_ids, sampling_params)
        if sampling_params.seed is None:
            seq.seed = (self.config.seed * 1000003 + seq.seq_id) & 0x7FFFFFFFFFFFFFFF
        self.scheduler.add(seq)
        self.request_metrics[seq.seq_id] = RequestMetrics(seq.seq_id, seq.num_prompt_tokens, arrival)
        return seq.seq_id

    def is_finished(self) -> bool:
        return self.scheduler.is_finished() and self._inflight is None

    # ------------------------------------------------------------------ one step
    def step(self):
        """Schedule, run one mixed batch, sample, book.  Returns (finished [(seq_id, token_ids)], StepStats).

        With ``async_decode`` a step is launched without waiting for it: the call returns what the step BEFORE it
        finished, and the tokens that the step in flight has chosen pass to this one on the device.  Only a plan that
        needs an unread token anywhere else than as a request's single next token (a preempted request that is
        recomputed) first waits for the step in flight.  Without it the step is read before the call returns.
        After a ``KernelError`` the requests of the failed step hold no valid tokens: ``abort_all()`` drops them."""
        t0 = perf_counter()
        outputs = []
        if self.scheduler.is_finished():
            if self._inflight is None:
                raise RuntimeError("nothing to do: no request is waiting, running or in flight")
            self.last_sampled_ids = []
            return self._drain(), StepStats(0, 0, perf_counter() - t0)
        try:
            plan = self.scheduler.schedule()
        except RuntimeError:
            # nothing fits: the step in flight may hold what is missing (requests at their length give their pages
            # back when their last token has been read)
            if self._inflight is None:
                raise
            outputs += self._drain()
            if self.scheduler.is_finished():
                self.last_sampled_ids = []
                return outputs, StepStats(0, 0, perf_counter() - t0)
            plan = self.scheduler.schedule()
        runner = self.model_runner
        # Which tokens of this plan has the host not read yet, and can the step in flight hand them over?  It can if
        # each is the single next token of a request that the step in flight chose a token for.
        flight = self._inflight
        source = {}
        if flight is not None:
            row = 0
            for s, place in zip(flight[0], flight[1]):
                if place >= 0:
                    source[s.seq_id] = (place, row)
                    row += 1
        feed = []
        for s in plan.seqs:
            start, n = s.num_cached_tokens, s.num_scheduled_tokens
            if PENDING not in s.token_ids[start:start + n]:
                feed.append(-1)
            elif n == 1 and s.seq_id in source and source[s.seq_id][0] == start:
                feed.append(source[s.seq_id][1])
            else:
                feed = None                                   # e.g. a preempted request recomputed from its first token
                break
        if feed is None:
            outputs += self._drain()
            flight = None
        seqs = [s for s in plan.seqs if not s.is_finished]    # a step just read may have ended some of them
        if len(seqs) != len(plan.seqs) or feed is None or all(f < 0 for f in feed):
            feed = None                                       # (requests end only when a step is read, and then nothing is fed)
        if not seqs:
            self.last_sampled_ids = []
            return outputs, StepStats(0, 0, perf_counter() - t0)
        items, sampled = [], []
        for s in seqs:
            start, n = s.num_cached_tokens, s.num_scheduled_tokens
            last = start + n == len(s)
            items.append(StepItem(s.seq_id, [0 if t == PENDING else t for t in s.token_ids[start:start + n]], start,
                                  [n - 1] if last else []))
            if last:
                sampled.append(s)
            m = self.request_metrics[s.seq_id]
            if m.first_scheduled_time is None:
                m.first_scheduled_time = t0
        self.last_sampled_ids = [s.seq_id for s in sampled]
        handle = runner.launch(items, [(s.temperature, s.seed, len(s)) for s in sampled],
                               feed_from=flight[2] if feed is not None else None, feed=feed)
        self.h2d_bytes += runner.builder.bytes_last_copy
        self.d2h_bytes += 4 * (len(sampled) + 1)              # the tokens and the step's health word
        n_decode = sum(1 for it in items if len(it.tokens) == 1 and it.want)
        stats = StepStats(n_decode, sum(len(it.tokens) for it in items) - n_decode, 0.0)
        places = self.scheduler.advance(seqs)
        previous, self._inflight = self._inflight, (seqs, places, handle)
        if previous is not None:
            outputs += self._resolve(previous)
        if not self.async_decode:
            outputs += self._drain()                          # every step is read before the next is planned
        stats.elapsed = perf_counter() - t0
        return outputs, stats

    def _book(self, sampled: list[Sequence], now: float) -> list:
        outputs = []
        for seq in sampled:
            m = self.request_metrics[seq.seq_id]
            m.num_completion_tokens = seq.num_completion_tokens
            if m.first_token_time is None:
                m.first_token_time = now
            if seq.is_finished and m.finish_time is None:
                m.finish_time = now
                outputs.append((seq.seq_id, seq.completion_token_ids))
        return outputs

    def _resolve(self, flight) -> list:
        """Read the tokens of a launched step and book them."""
        seqs, places, handle = flight
        self.scheduler.resolve(seqs, places, handle.read())
        return self._book([s for s, place in zip(seqs, places) if place >= 0], perf_counter())

    def abort_all(self) -> None:
        """Drop every request (waiting, running or in flight) and give back what they hold."""
        self._drain()
        for seq in list(self.scheduler.running) + list(self.scheduler.waiting):
            self.scheduler._finish(seq)

    def _drain(self) -> list:
        """Wait for the step in flight, if there is one."""
        if self._inflight is None:
            return []
        flight, self._inflight = self._inflight, None
        return self._resolve(flight)

    def get_completed_request_metrics(self) -> list[RequestMetrics]:
        return sorted((m for m in self.request_metrics.values() if m.finish_time is not None), key=lambda m: m.seq_id)

    # ------------------------------------------------------------------ the entry point
    def generate(self, prompts, sampling_params, use_tqdm: bool = True) -> list[dict]:
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt is needed")
        pbar = None
        if use_tqdm:
            from tqdm.auto import tqdm
            pbar = tqdm(total=len(prompts), desc="Generating", dynamic_ncols=True)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        outputs = {}
        prefill_tp = decode_tp = 0.0
        while not self.is_finished():
            finished, stats = self.step()
            if stats.num_prefill_tokens:
                prefill_tp = stats.prefill_throughput
            if stats.num_decode_tokens:
                decode_tp = stats.decode_throughput
            for seq_id, token_ids in finished:
                outputs[seq_id] = token_ids
                if pbar is not None:
                    pbar.set_postfix({"Prefill": f"{int(prefill_tp)}tok/s", "Decode": f"{int(decode_tp)}tok/s"})
                    pbar.update(1)
        if pbar is not None:
            pbar.close()
        result = []
        for seq_id in ids:
            token_ids = outputs[seq_id]
            text = self.tokenizer.decode(token_ids) if self.tokenizer is not None else ""
            result.append({"text": text, "token_ids": token_ids})
        return result


class LLM(LLMEngine):
    pass
