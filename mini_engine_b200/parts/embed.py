"""Token embedding and output head.

Reference: layers/embed_head.py:5-23.  The embedding writes the float32 residual stream;
the head takes the rows that were asked for (already gathered and normalised) and returns
float32 logits.  A tied head shares the embedding's storage (models/qwen3.py:107-109).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import ParamDecl, Part


class TokenEmbedding(Part):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int):
        super().__init__()
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size

    def param_decls(self):
        return [ParamDecl("weight", (self.vocab_size, self.hidden_size))]

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        out = ctx.buffer("residual", (token_ids.shape[0], self.hidden_size), torch.float32)
        ops.embed(token_ids, self.p("weight"), out, ctx.error_flag, feedback=getattr(ctx, "token_feedback", None))
        return out


class LMHead(Part):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: str | None):
        super().__init__()
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to

    def param_decls(self):
        return [ParamDecl("weight", (self.vocab_size, self.hidden_size), tied_to=self.tied_to)]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        out = ctx.buffer("logits", (x.shape[0], self.vocab_size), torch.float32)
        ops.tag = "logits"
        ops.linear(x, self.p("weight"), out, workspace=ctx.buffer, err=ctx.error_flag)
        return out
