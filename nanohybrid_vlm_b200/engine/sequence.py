"""One request's state on the host (nanovllm/engine/sequence.py:21-342, the text-only fields)."""
from __future__ import annotations

from enum import Enum, auto
from itertools import count

from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


PENDING = -1        # stands in a token list for a token that the GPU has chosen but the host has not read yet


class Sequence:
    counter = count()

    def __init__(self, token_ids: list[int], sampling_params: SamplingParams = SamplingParams(), seed: int | None = None):
        self.seq_id = next(Sequence.counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.num_prompt_tokens = len(token_ids)
        self.num_cached_tokens = 0          # tokens whose keys/values (and state) are in the cache
        self.num_scheduled_tokens = 0       # tokens of the step being run
        self.temperature = sampling_params.temperature
        self.max_tokens = sampling_params.max_tokens
        self.ignore_eos = sampling_params.ignore_eos
        self.seed = sampling_params.seed if sampling_params.seed is not None else (seed if seed is not None else self.seq_id)
        self.num_preemptions = 0
        self.finishing = False              # no further token is wanted (length), the last one is still on its way

    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def completion_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def is_prefill(self) -> bool:
        """More than one token of it is still to be computed."""
        return len(self.token_ids) - self.num_cached_tokens > 1

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(token_id)
