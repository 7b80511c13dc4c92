"""One decoder block: how norm, mixer and feed-forward are arranged around the residual.

Reference wiring (models/qwen3.py:65-74, layers/layernorm.py:19-23): pre-norm, with each
sub-layer's output added to the residual inside the next norm.  The same deferred add is
used here: a block receives the residual stream and the previous sub-layer's output
(``delta``, not yet added) and returns its own last output the same way.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import Part, Upcoming
from .registry import PartSpec, build_part


@dataclass
class BlockSpec:
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec                     # built twice: before the mixer and before the feed-forward
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."


class PreNormBlock(Part):
    capturable = True

    def __init__(self, spec: BlockSpec, shared: Optional[dict] = None):
        super().__init__()
        self.spec = spec
        mixer_spec = spec.mixer
        if shared:
            # Objects that several layers share (one rotary table for all of them).
            args = {k: shared.get(v.key, v) if isinstance(v, SharedRef) else v
                    for k, v in mixer_spec.args.items()}
            mixer_spec = PartSpec(mixer_spec.kind, args)
        self.mixer = build_part("mixer", mixer_spec)
        self.feed_forward = build_part("feed_forward", spec.feed_forward)
        self.mixer_norm = build_part("norm", spec.norm)
        self.feed_forward_norm = build_part("norm", spec.norm)

    def sub_parts(self):
        s = self.spec
        return [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer),
                (s.feed_forward_norm_prefix, self.feed_forward_norm),
                (s.feed_forward_prefix, self.feed_forward)]

    def upcoming(self) -> Upcoming:
        """What this block starts with, for the block that runs before it."""
        return Upcoming(self.mixer_norm, self.mixer.first_weight())

    def forward(self, residual, delta, ctx, call, upcoming=None):
        """``delta``: the output of the sub-layer before this block, not yet added to ``residual`` (or the mark
        that it has been).  Returns this block's last output the same way.  ``upcoming``: what runs after this
        block (``Upcoming``), if the caller knows it."""
        mixer, ffn = self.mixer, self.feed_forward
        x = self.mixer_norm.forward(residual, delta, ctx, lazy=mixer.takes_pending_norm)
        if mixer.adds_to_residual:
            mixed = mixer.forward(x, ctx, call, residual=residual,
                                  upcoming=Upcoming(self.feed_forward_norm, ffn.first_weight()))
        else:
            mixed = mixer.forward(x, ctx, call)
        x = self.feed_forward_norm.forward(residual, mixed, ctx, lazy=ffn.takes_pending_norm)
        if ffn.adds_to_residual:
            return ffn.forward(x, ctx, residual=residual, upcoming=upcoming)
        return ffn.forward(x, ctx)


@dataclass(frozen=True)
class SharedRef:
    """Stands in a PartSpec's args for an object that the model builds once and shares."""
    key: str
