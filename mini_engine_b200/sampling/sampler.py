"""Greedy and temperature sampling on the device (the kernels of csrc/sampler.cu, called by the step function).

Reference (layers/sampler.py:5-11): logits in float32; greedy = argmax where the
temperature is 0; else ``argmax(softmax(logits / T) / E)`` with E ~ Exp(1) per entry (an
exponential race, the same law as adding Gumbel noise to ``logits / T``).  The reference
draws E from torch's global generator, so its tokens depend on how the batch was formed.
Here the noise of entry v comes from a counter-based hash of (request seed, position of
the sampled token, v), so a request's tokens do not depend on what else is in the batch or
on how its prompt was cut; ``noise_uniform`` restates the hash on the host for tests.
"""
from __future__ import annotations

import numpy as np


def _mix32(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.uint32)
    x ^= x >> np.uint32(16)
    x = (x * np.uint32(0x7FEB352D)).astype(np.uint32)
    x ^= x >> np.uint32(15)
    x = (x * np.uint32(0x846CA68B)).astype(np.uint32)
    x ^= x >> np.uint32(16)
    return x


def noise_uniform(seed: int, position: int, vocab_size: int) -> np.ndarray:
    """The uniform numbers in (0, 1) that the sampling kernel uses for one row (float64)."""
    with np.errstate(over="ignore"):
        v = np.arange(vocab_size, dtype=np.uint32)
        s = _mix32(np.asarray([seed & 0xFFFFFFFF], dtype=np.uint32) + np.uint32(0x9E3779B9))
        p = _mix32((s ^ np.uint32(position & 0xFFFFFFFF)) + np.uint32(0x85EBCA6B))
        h = _mix32((p ^ v) + np.uint32(0xC2B2AE35))
    return ((h >> np.uint32(9)).astype(np.float64) + 0.5) / 8388608.0
