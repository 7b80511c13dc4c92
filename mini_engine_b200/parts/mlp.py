"""SwiGLU feed-forward: ``down( silu(gate(x)) * up(x) )``.

Reference: models/qwen3.py:42-51, layers/activation.py:4-7; gate and up are packed into
one weight (rows gate | up) so that one product reads x once, and SiLU-and-multiply runs in
that product's epilogue.
"""
from __future__ import annotations

from .base import FeedForward
from .linear import Linear
from .registry import register_feed_forward


class SwiGLU(FeedForward):
    capturable = True
    # The last projection adds its result into the residual stream in its own epilogue.  (Folding the norm in
    # front into the first projection was measured and lost: hundreds of blocks each re-read and convert the
    # residual; the kernel keeps that ability, the parts do not ask for it.)
    adds_to_residual = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_up_proj = Linear(hidden_size, [("gate_proj.weight", intermediate_size),
                                                 ("up_proj.weight", intermediate_size)],
                                   name="gate_up_proj.weight")
        self.down_proj = Linear(intermediate_size, [("down_proj.weight", hidden_size)],
                                name="down_proj.weight")

    def sub_parts(self):
        return [("", self.gate_up_proj), ("", self.down_proj)]

    def forward(self, x, ctx, residual=None):
        act = self.gate_up_proj.forward(x, ctx, "ffn_act", epilogue="silu_mul")
        return self.down_proj.forward(act, ctx, "ffn_out", may_split=True, residual=residual)


register_feed_forward("swiglu", SwiGLU)
