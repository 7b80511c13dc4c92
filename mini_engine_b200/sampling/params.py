"""Per-request sampling options, as in the reference (sampling_params.py:3-11), plus a seed."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0      # 0 = greedy
    max_tokens: int = 64
    ignore_eos: bool = False
    seed: Optional[int] = None    # None: derived from the engine's seed and the request's number

    def __post_init__(self):
        if not self.temperature >= 0:
            raise ValueError("temperature must not be negative")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
