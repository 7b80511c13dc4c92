"""A decoder model put together from a plan: embedding, blocks, final norm, head.

The plan is data.  ``blocks`` lists the layers that exist (each with its own mixer,
feed-forward and norm kinds, so layers may differ); ``schedule`` lists the order in which
they run: a ``LayerCall`` names the block, the cache slot its mixer uses and whether it
writes to it.  A block may be named twice (each call then has a cache slot of its own, or
shares one), and a call may read a slot that an earlier call wrote
(``writes_cache=False``).  The reference runs its ``ModuleList`` once in order
(models/qwen3.py:86-92); that is the schedule ``[(i, i, True) for i in range(L)]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterator, Optional

import torch

from .base import Part, ParamDecl
from .block import BlockSpec, SharedRef
from .embed import LMHead, TokenEmbedding
from .registry import PartSpec, build_block, build_part


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache_slot: int
    writes_cache: bool = True


@dataclass
class ModelPlan:
    vocab_size: int
    hidden_size: int
    blocks: list[BlockSpec]
    schedule: list[LayerCall]
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_position: int
    shared: dict[str, PartSpec] = field(default_factory=dict)   # key -> position encoding built once
    embed_prefix: str = "model.embed_tokens."
    block_prefix: str = "model.layers.{i}."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."


class DecoderModel(Part):
    capturable = True

    def __init__(self, plan: ModelPlan):
        super().__init__()
        self.plan = plan
        self.shared = {k: build_part("position_encoding", s) for k, s in plan.shared.items()}
        self.embed = TokenEmbedding(plan.vocab_size, plan.hidden_size)
        self.blocks = [build_block(s, self.shared) for s in plan.blocks]
        self.final_norm = build_part("norm", plan.final_norm)
        tied = plan.embed_prefix + "weight" if plan.tie_word_embeddings else None
        self.head = LMHead(plan.vocab_size, plan.hidden_size, tied)
        self.schedule = list(plan.schedule)
        n_slots = 1 + max((c.cache_slot for c in self.schedule), default=-1)
        # What each cache slot must hold, taken from the first call that uses it.
        self.slot_needs: list[list[Any]] = [[] for _ in range(n_slots)]
        written = set()
        for c in self.schedule:
            if not 0 <= c.block < len(self.blocks):
                raise ValueError(f"schedule names block {c.block}, the model has {len(self.blocks)}")
            needs = self.blocks[c.block].mixer.cache_needs()
            if not self.slot_needs[c.cache_slot]:
                self.slot_needs[c.cache_slot] = needs
            elif self.slot_needs[c.cache_slot] != needs:
                raise ValueError(f"cache slot {c.cache_slot} is used by mixers with different needs")
            if c.writes_cache:
                written.add(c.cache_slot)
            elif c.cache_slot not in written:
                raise ValueError(f"cache slot {c.cache_slot} is read before any call writes it")

    # ---- structure -----------------------------------------------------------------
    def sub_parts(self):
        parts = [(self.plan.embed_prefix, self.embed)]
        parts += [(self.plan.block_prefix.format(i=i), b) for i, b in enumerate(self.blocks)]
        parts += [(self.plan.final_norm_prefix, self.final_norm), (self.plan.head_prefix, self.head)]
        return parts

    def walk(self) -> Iterator[tuple[str, Part]]:
        """Every part once, with the prefix of its parameters (shared parts under their first owner)."""
        seen: set[int] = set()

        def rec(prefix: str, part: Part):
            if id(part) in seen:
                return
            seen.add(id(part))
            yield prefix, part
            for rel, sub in part.sub_parts():
                yield from rec(prefix + rel, sub)

        yield from rec("", self)

    def finalize_all(self, dtype, device):
        for _, part in self.walk():
            part.finalize(dtype, device)

    # ---- one step ------------------------------------------------------------------
    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        """Hidden states of the wanted rows, normalised: ``[len(ctx.logits_rows), hidden]``."""
        residual = self.embed.forward(token_ids, ctx)
        delta = None
        for i, call in enumerate(self.schedule):
            # the block learns what runs after it, so that its last kernel can prepare for it
            after = self.blocks[self.schedule[i + 1].block].upcoming() if i + 1 < len(self.schedule) else None
            delta = self.blocks[call.block].forward(residual, delta, ctx, call, upcoming=after)
        return self.final_norm.forward(residual, delta, ctx, rows=ctx.logits_rows)

    def compute_logits(self, hidden: torch.Tensor, ctx) -> torch.Tensor:
        return self.head.forward(hidden, ctx)
