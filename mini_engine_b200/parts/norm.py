"""RMSNorm with the residual sum folded in.

Reference formula (layers/layernorm.py:11-23): ``y = x * rsqrt(mean(x^2) + eps)`` in
float32, cast to the working dtype, times the weight; with a residual the sum
``x + residual`` is normalised and also returned.  Here the residual stream itself is
kept in float32 in both precisions, so the sum, the statistics and the weight multiply
all happen in float32 and the result is rounded once.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import AddedToResidual, Norm, ParamDecl, PendingNorm
from .registry import register_norm


class RMSNorm(Norm):
    capturable = True

    def __init__(self, size: int, eps: float):
        super().__init__()
        self.size = size
        self.eps = float(eps)

    def param_decls(self):
        return [ParamDecl("weight", (self.size,), init="norm", role="vector")]

    def separable_weight(self):
        """y = x * rsqrt(mean(x^2) + eps) * w splits into an element-wise x * w and one factor per row, so the part
        in front may write x * w itself."""
        return self.p("weight")

    def forward(self, residual, delta, ctx, rows: Optional[torch.Tensor] = None, lazy: bool = False):
        if isinstance(delta, AddedToResidual):
            if lazy and rows is None and delta.preweighted is not None and delta.weight is self.p("weight"):
                return PendingNorm(residual, self.p("weight"), self.eps, delta.sumsq, delta.preweighted)
            delta = None                          # the residual already holds the sum
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer("norm_out", (n, self.size), ctx.act_dtype)
        ops.add_rmsnorm(residual, delta, self.p("weight"), self.eps, out, rows=rows)
        return out


register_norm("rmsnorm", RMSNorm)
