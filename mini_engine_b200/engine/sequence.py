"""A request as the host sees it: its tokens, its progress and what it holds of the cache.

The reference keeps the same facts in ``engine/sequence.py:14-74`` (token list, counters for computed,
cached, hashed and scheduled tokens, block table, priority, arrival time).  Here a request *is* a
``CacheHolder`` (block tables per cache group and a state slot), so the cache manager and the step function
take it as it is.
"""
from __future__ import annotations

import itertools
import time
from enum import Enum
from typing import Iterable, Optional

from ..cache.manager import CacheHolder
from ..sampling.params import SamplingParams

_ids = itertools.count()


class SequenceStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class Sequence(CacheHolder):
    """Prompt tokens followed by the tokens generated so far.

    ``num_computed_tokens`` (inherited) counts the tokens whose keys and values are in the cache;
    ``num_scheduled_tokens`` is the portion the current step computes.  A request owes
    ``num_tokens - num_computed_tokens`` tokens: its whole prompt at first, one token while it decodes, and
    prompt plus generated tokens again after it was preempted.
    """

    def __init__(self, token_ids: Iterable[int], sampling_params: Optional[SamplingParams] = None, priority: int = 0):
        super().__init__()
        self.token_ids: list[int] = [int(t) for t in token_ids]
        if not self.token_ids:
            raise ValueError("a request needs at least one prompt token")
        self.seq_id: int = next(_ids)
        self.num_prompt_tokens: int = len(self.token_ids)
        self.sampling_params: SamplingParams = sampling_params or SamplingParams()
        self.priority: int = priority
        self.arrival_time: float = time.perf_counter()
        self.status: SequenceStatus = SequenceStatus.WAITING
        self.num_scheduled_tokens: int = 0

    # ---- sizes --------------------------------------------------------------------------------------
    def __len__(self) -> int:
        return len(self.token_ids)

    num_tokens = property(__len__)

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_uncomputed_tokens(self) -> int:
        return len(self.token_ids) - self.num_computed_tokens

    # ---- views of the tokens ----------------------------------------------------------------------------
    @property
    def prompt_token_ids(self) -> list[int]:
        return self.token_ids[: self.num_prompt_tokens]

    @property
    def completion_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def last_token(self) -> int:
        return self.token_ids[-1]

    def scheduled_tokens(self) -> list[int]:
        """The tokens of the portion that the current step computes."""
        a = self.num_computed_tokens
        return self.token_ids[a:a + self.num_scheduled_tokens]

    # ---- progress -------------------------------------------------------------------------------------------
    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    @property
    def samples_this_step(self) -> bool:
        """True when the scheduled portion reaches the last token, so the step draws the next one
        (engine/sequence.py:65-66 in the reference)."""
        return self.num_computed_tokens + self.num_scheduled_tokens == len(self.token_ids)

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(int(token_id))

    def reached_limit(self, eos: Optional[int]) -> bool:
        """Finished by EOS (unless ignored) or by ``max_tokens``."""
        sp = self.sampling_params
        if not sp.ignore_eos and eos is not None and self.token_ids[-1] == eos and self.num_completion_tokens > 0:
            return True
        return self.num_completion_tokens >= sp.max_tokens
