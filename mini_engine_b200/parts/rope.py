"""Rotary position encoding, half-split ("neox") layout.

Reference (layers/rotary_embedding.py:5-25): ``inv_freq[i] = theta^(-2i/d)``, angle
``pos * inv_freq[i]``; for i < d/2: ``o[i] = x[i] cos - x[i+d/2] sin``,
``o[i+d/2] = x[i+d/2] cos + x[i] sin``.  The table is built in float32 exactly as the
reference builds it, and stays float32 (the reference rounds it to the working dtype,
layers/rotary_embedding.py:21-22); the rotation itself runs inside the fused
norm+rotate+cache-write kernel of the attention mixer.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


class RotaryEmbedding(PositionEncoding):
    capturable = True

    layout = "half_split"

    def __init__(self, rotary_dim: int, max_position: int, theta: float):
        super().__init__()
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim {rotary_dim} must be even")
        self.rotary_dim = rotary_dim                  # the leading elements of a head that are rotated
        self.max_position = max_position
        self.theta = float(theta)
        self.cos_sin: torch.Tensor | None = None      # [max_position, rotary_dim] = cos | sin halves

    def finalize(self, dtype, device):
        d = self.rotary_dim
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        t = torch.arange(self.max_position, dtype=torch.float32)
        freqs = torch.outer(t, inv_freq)                       # [P, d/2] float32
        self.cos_sin = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(device)


register_position_encoding("rope", RotaryEmbedding)
