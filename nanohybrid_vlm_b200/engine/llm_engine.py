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
from .sequence import Sequence


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
        return self.scheduler.is_finished()

    # ------------------------------------------------------------------ one step
    def step(self):
        """Schedule, run one mixed batch, sample, book.  Returns (finished [(seq_id, token_ids)], StepStats)."""
        t0 = perf_counter()
        plan = self.scheduler.schedule()
        items, sampled = [], []
        for seq in plan.seqs:
            start, n = seq.num_cached_tokens, seq.num_scheduled_tokens
            last = start + n == len(seq)
            items.append(StepItem(seq.seq_id, seq.token_ids[start:start + n], start, [n - 1] if last else []))
            if last:
                sampled.append(seq)
            m = self.request_metrics[seq.seq_id]
            if m.first_scheduled_time is None:
                m.first_scheduled_time = t0
        runner = self.model_runner
        tokens = {}
        self.last_sampled_ids = [s.seq_id for s in sampled]
        if sampled:
            chosen = runner.run(items, [(s.temperature, s.seed, len(s)) for s in sampled])
            self.d2h_bytes += 4 * (len(sampled) + 1)        # the tokens and the step's health word
            tokens = {s.seq_id: t for s, t in zip(sampled, chosen)}
        else:
            runner.step(items)
        self.h2d_bytes += runner.builder.bytes_last_copy
        self.scheduler.postprocess(plan.seqs, [tokens.get(s.seq_id) for s in plan.seqs])
        now = perf_counter()
        outputs = []
        for seq in sampled:
            m = self.request_metrics[seq.seq_id]
            m.num_completion_tokens = seq.num_completion_tokens
            if m.first_token_time is None:
                m.first_token_time = now
            if seq.is_finished:
                m.finish_time = now
                outputs.append((seq.seq_id, seq.completion_token_ids))
        return outputs, StepStats(plan.num_decode_tokens, plan.num_prefill_tokens, now - t0)

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
