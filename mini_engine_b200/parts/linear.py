"""Bias-free linear maps ``y = x W^T`` whose weight may be packed from several disk tensors.

Reference: layers/linear.py:4-45 (packed q|k|v rows and gate|up rows, ``F.linear``).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from .base import DiskSource, ParamDecl, Part


class Linear(Part):
    """``pieces``: (disk name relative to the owner, rows) for every packed piece."""

    capturable = True


    def __init__(self, in_features: int, pieces: Sequence[tuple[str, int]], name: str = "weight"):
        super().__init__()
        self.in_features = in_features
        self.pieces = list(pieces)
        self.out_features = sum(r for _, r in self.pieces)
        self.name = name

    def param_decls(self):
        sources, start = [], 0
        for disk, rows in self.pieces:
            sources.append(DiskSource(disk, start, rows))
            start += rows
        return [ParamDecl(self.name, (self.out_features, self.in_features), sources=sources)]

    @property
    def weight(self) -> torch.Tensor:
        return self.p(self.name)

    def forward(self, x: torch.Tensor, ctx, out_name: str, *, out_dtype: Optional[torch.dtype] = None,
                epilogue: str = "none", may_split: bool = False) -> torch.Tensor:
        """``x W^T``.  With ``may_split`` the result may come as float32 partial results [splits, T, N] of a
        split-K product; only a consumer that adds them (the next norm) may ask for that."""
        if may_split and epilogue == "none":
            part = ops.linear_partials(x, self.weight, ctx.buffer, out_name + "_partials")
            if part is not None:
                return part
        n_out = self.out_features // 2 if epilogue == "silu_mul" else self.out_features
        out = ctx.buffer(out_name, (x.shape[0], n_out), out_dtype or ctx.act_dtype)
        ops.linear(x, self.weight, out, epilogue=epilogue, workspace=ctx.buffer, err=ctx.error_flag)
        return out
