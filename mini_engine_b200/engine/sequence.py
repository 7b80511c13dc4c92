"""One request's state on the host (reference: engine/sequence.py:14-74)."""
from __future__ import annotations

from enum import Enum
from itertools import count
from time import perf_counter
from typing import Optional, Sequence as Seq

from ..cache.manager import CacheHolder
from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    WAITING = 1
    RUNNING = 2
    FINISHED = 3


class Sequence(CacheHolder):
    _counter = count()

    def __init__(self, token_ids: Seq[int], sampling_params: Optional[SamplingParams] = None,
                 priority: int = 0):
        super().__init__()
        if len(token_ids) == 0:
            raise ValueError("a request needs at least one prompt token")
        self.seq_id = next(Sequence._counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = [int(t) for t in token_ids]
        self.num_prompt_tokens = len(self.token_ids)
        self.num_scheduled_tokens = 0
        self.sampling_params = sampling_params if sampling_params is not None else SamplingParams()
        self.priority = priority
        self.arrival_time = perf_counter()

    def __len__(self):
        return len(self.token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def last_token(self) -> int:
        return self.token_ids[-1]

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED

    @property
    def num_completion_tokens(self) -> int:
        return self.num_tokens - self.num_prompt_tokens

    @property
    def prompt_token_ids(self) -> list[int]:
        return self.token_ids[:self.num_prompt_tokens]

    @property
    def completion_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_uncomputed_tokens(self) -> int:
        return self.num_tokens - self.num_computed_tokens

    @property
    def samples_this_step(self) -> bool:
        """The portion scheduled now reaches the request's last token (engine/sequence.py:65-66)."""
        return self.num_computed_tokens + self.num_scheduled_tokens == self.num_tokens

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(int(token_id))
