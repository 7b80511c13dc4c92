"""Interfaces that every part of a layer implements.

A *part* (norm, position encoding, mixer, feed-forward, embedding, head) knows its own
sizes and constants, which it gets as constructor parameters, and nothing about the
model it sits in.  It declares

* its parameters (``param_decls``): shapes, how they are initialised at random and from
  which tensors on disk each one is filled (several disk tensors may be packed into one
  parameter, as the reference packs q/k/v and gate/up: layers/linear.py:4-45,
  models/qwen3.py:96-102);
* what it needs of the cache (``cache_needs``): pages of keys and values, all of them or
  a window, and/or a slot of fixed size per request.

and runs on the tokens of one step through ``forward``; everything a step knows (token
positions, which request a token belongs to, block tables, state slots, the cache
storage, work buffers) arrives in the ``StepContext``, never through a module global as
in the reference (utils/context.py:3-27).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import torch


@dataclass
class DiskSource:
    """Rows ``[row_start, row_start+rows)`` of a parameter come from one tensor on disk."""
    disk_name: str
    row_start: int
    rows: int


@dataclass
class ParamDecl:
    name: str                              # local name; the owner's prefix is put in front
    shape: tuple[int, ...]
    init: str = "normal"                   # "normal": N(0, 0.02); "norm": 1 + N(0, 0.1)
    sources: list[DiskSource] = field(default_factory=list)   # empty: one tensor, same name
    role: str = "matrix"                   # "matrix" | "vector" (vectors are held in float32)
    tied_to: Optional[str] = None          # full name of the parameter whose storage is shared


@dataclass(frozen=True)
class KVCacheNeed:
    """Paged keys and values: ``window=None`` keeps every key, else the last ``window``."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A slot of fixed size per request: ``shape`` elements of ``dtype`` (a torch dtype's name)."""
    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass
class AddedToResidual:
    """What a part returns instead of its output when its last kernel has already added that output into the
    float32 residual stream; ``sumsq`` [parts, T] holds the new residual's sums of squares per strip of
    columns, which the next normalisation needs.  If that kernel was told the next norm's weight it has also
    written ``preweighted`` = residual * ``weight`` (in the activations' dtype), the half of that norm that needs
    no statistics."""
    sumsq: "torch.Tensor"
    preweighted: "Optional[torch.Tensor]" = None
    weight: "Optional[torch.Tensor]" = None


@dataclass
class Upcoming:
    """What runs right after a mixer or feed-forward, as far as its last kernel can prepare for it: the norm that
    reads the residual stream next (its element-wise half may be written with the residual) and the first weight
    matrix used after that (it may be asked into the cache ahead of time).  Either may be None."""
    norm: "Any" = None
    weight: "Optional[torch.Tensor]" = None


@dataclass
class PendingNorm:
    """Rows that are ``norm(residual) * weight`` but have not been computed yet: ``preweighted`` holds
    residual * weight, and each row still lacks its factor rsqrt(sum of ``sumsq`` / width + eps).  A consumer
    whose product can apply that factor to its own results (``takes_pending_norm``) uses the pieces; any other
    gets a tensor from ``materialize``."""
    residual: "torch.Tensor"
    weight: "torch.Tensor"
    eps: float
    sumsq: "torch.Tensor"
    preweighted: "torch.Tensor"

    def materialize(self, ctx) -> "torch.Tensor":
        from .. import ops
        out = ctx.buffer("norm_out", tuple(self.residual.shape), ctx.act_dtype)
        ops.add_rmsnorm(self.residual, None, self.weight, self.eps, out)
        return out


class Part:
    """Base of all parts.  ``params`` is filled by the weight loader.

    ``capturable`` says that ``forward`` only launches kernels that read the step's shape from
    device memory, so a decode step may be recorded once in a CUDA graph and replayed.  A part
    that decides in Python on the step's host-side numbers leaves it False (the default), and a
    model with such a part runs every step eagerly."""

    capturable = False
    # A mixer or feed-forward whose first kernel can finish a PendingNorm, and whose last kernel can add into the
    # residual (``forward(..., residual=, upcoming=)``), says so; the block then hands it those.
    takes_pending_norm = False
    adds_to_residual = False

    def __init__(self):
        self.params: dict[str, torch.Tensor] = {}

    def first_weight(self) -> "Optional[torch.Tensor]":
        """The weight matrix that this part's first kernel reads, if the part wants the kernel before it to ask
        for it ahead of time; None otherwise."""
        return None

    def param_decls(self) -> list[ParamDecl]:
        return []

    def cache_needs(self) -> list[Any]:
        return []

    def sub_parts(self) -> list[tuple[str, "Part"]]:
        """(relative prefix, part) pairs of the parts this one is put together from."""
        return []

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        """Called once after the parameters are in place (build tables, check dtypes)."""

    def p(self, name: str) -> torch.Tensor:
        try:
            return self.params[name]
        except KeyError:
            raise RuntimeError(f"{type(self).__name__}: parameter {name!r} was never loaded") from None


class Mixer(Part):
    """Mixes information between the tokens of a request (attention, or a mixer with state)."""

    def forward(self, x: torch.Tensor, ctx: "Any", call: "Any") -> torch.Tensor:
        """``x`` [T, hidden] in the working dtype -> the mixer's output, same shape (or float32 split-K partial
        results [S, T, hidden]).  With ``adds_to_residual`` the block also passes ``residual=``, and the mixer may
        return ``AddedToResidual``; with ``takes_pending_norm`` ``x`` may be a ``PendingNorm``."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: "Any") -> torch.Tensor:
        """As ``Mixer.forward`` without the cache."""
        raise NotImplementedError


class Norm(Part):
    def separable_weight(self) -> "Optional[torch.Tensor]":
        """The weight w, if the norm is ``x * f(row) * w`` with one factor per row taken from the row's sum of
        squares (RMSNorm): the kernel that writes the residual may then write x * w beside it (``AddedToResidual``)
        and the product after the norm applies the factor.  None: the norm cannot be split that way."""
        return None

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: "Any",
                rows: Optional[torch.Tensor] = None, lazy: bool = False) -> torch.Tensor:
        """``residual += delta`` (if given), then the normalised rows in the working dtype.

        With ``rows`` only those rows are normalised and ``residual`` is left unchanged.  ``delta`` may be
        ``AddedToResidual`` (nothing to add); then, with ``lazy``, a ``PendingNorm`` may be returned.
        """
        raise NotImplementedError


class PositionEncoding(Part):
    """Position information applied to queries and keys before the cache write.

    What the attention mixer hands to its kernels, and so what a position encoding of the rotary family declares:

    * ``cos_sin``: float32 ``[max_position, rotary_dim]`` built in ``finalize``: for every absolute position the
      cosines of the ``rotary_dim / 2`` angles, then their sines;
    * ``rotary_dim``: how many leading elements of a head are rotated (even, at most the head size; the rest pass
      through unchanged);
    * ``layout``: how elements are paired, by name.  The kernels know ``"half_split"`` (element i with element
      i + rotary_dim / 2); any other name is refused with an error that says so, and needs a kernel branch.

    A token has ONE position (int32) in the step's metadata; an encoding with several position axes is not covered."""

    rotary_dim: int = 0
    layout: str = "half_split"
    cos_sin: "Optional[torch.Tensor]" = None
