"""Sampling options of one request (nanovllm/sampling_params.py:5-15): ``temperature`` 0 means
greedy, a negative or non-finite one is an error; ``max_tokens``; ``ignore_eos``.  ``seed``
is this engine's addition: the request's random stream (None: derived from the engine's seed
and the request's number)."""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass(slots=True)
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False
    seed: int | None = None

    def __post_init__(self):
        if not math.isfinite(self.temperature):
            raise ValueError("temperature must be finite")
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
