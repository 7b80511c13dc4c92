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
from .registry import PartSpec, build_part, register_block


@dataclass
class BlockSpec:
    """One layer as data: the parts it is made of and (``kind``) how they are arranged.

    ``norm`` is the norm of both places; ``mixer_norm`` / ``feed_forward_norm`` give a place a norm of its own."""
    mixer: PartSpec
    feed_forward: PartSpec
    norm: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    kind: str = "pre_norm"             # a name registered with ``register_block``
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."

    def norm_of(self, place: str) -> PartSpec:
        spec = getattr(self, place) or self.norm
        if spec is None:
            raise ValueError(f"a block needs a norm for {place!r} (give ``norm`` or ``{place}``)")
        return spec


class Block(Part):
    """The arrangement of a layer's parts around the residual stream; built by the factory registered for
    ``BlockSpec.kind``.

    What the model asks of a block: ``mixer`` (its ``cache_needs()`` decide the layer's cache slot),
    ``sub_parts()`` (for the weights), ``upcoming()`` (what the block starts with, for the block before it; may be
    an empty ``Upcoming``) and ``forward(residual, delta, ctx, call, upcoming=None)``: ``residual`` is the float32
    stream [T, hidden], updated in place; ``delta`` is the output of the block before that is not added yet (a
    tensor, float32 split-K partial results, ``AddedToResidual``, or None); the return value is this block's own
    last output in the same form (None: everything is in ``residual`` already)."""

    mixer: Part

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
        self.mixer_norm = build_part("norm", spec.norm_of("mixer_norm"))
        self.feed_forward_norm = build_part("norm", spec.norm_of("feed_forward_norm"))

    def sub_parts(self):
        s = self.spec
        return [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer),
                (s.feed_forward_norm_prefix, self.feed_forward_norm),
                (s.feed_forward_prefix, self.feed_forward)]

    def upcoming(self) -> Upcoming:
        return Upcoming()

    def forward(self, residual, delta, ctx, call, upcoming=None):
        raise NotImplementedError


class PreNormBlock(Block):
    """``r += mixer(norm(r)); r += feed_forward(norm(r))`` with each sum deferred into the norm that follows
    (models/qwen3.py:65-74 in the reference)."""
    capturable = True

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


register_block("pre_norm", PreNormBlock)
