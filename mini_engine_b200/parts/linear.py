"""Bias-free linear maps ``y = x W^T`` whose weight may be packed from several disk tensors.

Reference: layers/linear.py:4-45 (packed q|k|v rows and gate|up rows, ``F.linear``).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from .base import AddedToResidual, DiskSource, ParamDecl, Part, PendingNorm


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

    def first_weight(self):
        return self.weight

    def forward(self, x, ctx, out_name: str, *, out_dtype: Optional[torch.dtype] = None,
                epilogue: str = "none", may_split: bool = False, residual: Optional[torch.Tensor] = None,
                next_norm=None, fetch_ahead: Optional[torch.Tensor] = None):
        """``x W^T``.

        ``x`` is a tensor or a ``PendingNorm`` (the product then applies the rows' factors to its results where
        its kernel takes the shape, else the norm is computed first).  With ``residual`` the product may add its
        result into that float32 tensor itself and return ``AddedToResidual``; ``next_norm`` is the norm that
        will read that residual next, whose element-wise half the same kernel then writes.  ``fetch_ahead`` is a
        tensor that a later kernel reads (the next product's weight): a decode product asks it into L2 while it
        runs, since the short dependent kernels of a decode step leave the memory system idle.  With ``may_split`` the
        result may come as float32 partial results [splits, T, N] of a split-K product; only a consumer that adds
        them (the next norm) may ask for that."""
        ops.tag = out_name
        pending = x if isinstance(x, PendingNorm) else None
        M = pending.residual.shape[0] if pending is not None else x.shape[0]
        fused = ctx.act_dtype == torch.bfloat16 and ops.decode_linear_takes(M, self.in_features, self.weight,
                                                                            residual is not None and epilogue == "none")
        row_scale = None
        if pending is not None:
            if fused:
                x, row_scale = pending.preweighted, (pending.sumsq, pending.eps)
            else:
                x = pending.materialize(ctx)
        fused = fused and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
        assert fused or row_scale is None, "a pre-weighted residual can only go through the kernel that finishes its norm"
        if fused and residual is not None and epilogue == "none":
            sumsq = ctx.buffer(out_name + "_sumsq", (ops.decode_linear_sumsq_parts(self.out_features, self.in_features), M), torch.float32)
            nw = next_norm.separable_weight() if next_norm is not None else None
            xw = ctx.buffer(out_name + "_preweighted", (M, self.out_features), torch.bfloat16) if nw is not None else None
            ops.decode_linear(self.weight, x, row_scale=row_scale, epilogue="residual", residual_out=residual,
                              sumsq_out=sumsq, next_norm=(nw, xw) if nw is not None else None, fetch_ahead=fetch_ahead,
                              err=ctx.error_flag)
            return AddedToResidual(sumsq, xw, nw)
        n_out = self.out_features // 2 if epilogue == "silu_mul" else self.out_features
        if may_split and epilogue == "none" and not fused:
            part = ops.linear_partials(x, self.weight, ctx.buffer, out_name + "_partials", err=ctx.error_flag)
            if part is not None:
                return part
        out = ctx.buffer(out_name, (M, n_out), out_dtype or ctx.act_dtype)
        if fused:
            ops.decode_linear(self.weight, x, out=out, epilogue=epilogue, row_scale=row_scale, fetch_ahead=fetch_ahead,
                              err=ctx.error_flag)
            return out
        ops.linear(x, self.weight, out, epilogue=epilogue, workspace=ctx.buffer, err=ctx.error_flag)
        return out
