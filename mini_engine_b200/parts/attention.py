"""Grouped-query attention over the paged cache.

Reference (models/qwen3.py:12-38, layers/attention.py:52-76): packed q|k|v projection,
RMSNorm over head_dim of every q and k head with one weight vector each, rotary
embedding, keys and values written to their cache slots, softmax(scale * q.k) over the
request's cached keys j <= p with scale = head_dim^-0.5, query head h reading key/value
head h // (heads / kv_heads), then the output projection.

``window`` (not in the reference) restricts a query at position p to keys
p-window < j <= p; such a layer asks the cache for a window group, whose pages are given
back once the window has passed them.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import KVCacheNeed, Mixer, ParamDecl
from .linear import Linear
from .registry import PartSpec, build_part, register_mixer


class GQAAttention(Mixer):
    capturable = True
    # In a decode step the q|k|v projection finishes the norm in front of it (the rows' factors applied to its
    # results) and the output projection adds into the residual stream and starts the next norm, in their epilogues.
    takes_pending_norm = True
    adds_to_residual = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm_eps: Optional[float], position_encoding: Optional[PartSpec | object],
                 window: Optional[int] = None, scale: Optional[float] = None):
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are no multiple of {num_kv_heads} kv heads")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else head_dim ** -0.5   # models/qwen3.py:25
        ops.check_attention_sizes(head_dim, num_heads, num_kv_heads)
        self.qkv_proj = Linear(hidden_size, [("q_proj.weight", self.q_size),
                                             ("k_proj.weight", self.kv_size),
                                             ("v_proj.weight", self.kv_size)], name="qkv_proj.weight")
        self.o_proj = Linear(self.q_size, [("o_proj.weight", hidden_size)], name="o_proj.weight")
        # One position-encoding object may be shared by all layers (models/qwen3.py:81,83).
        if isinstance(position_encoding, PartSpec):
            position_encoding = build_part("position_encoding", position_encoding)
        self.rope = position_encoding

    def sub_parts(self):
        parts = [("", self.qkv_proj), ("", self.o_proj)]
        if self.rope is not None:
            parts.append(("rotary_emb.", self.rope))
        return parts

    def param_decls(self):
        if self.qk_norm_eps is None:
            return []
        return [ParamDecl("q_norm.weight", (self.head_dim,), init="norm", role="vector"),
                ParamDecl("k_norm.weight", (self.head_dim,), init="norm", role="vector")]

    def cache_needs(self):
        return [KVCacheNeed(self.num_kv_heads, self.head_dim, self.window)]

    def first_weight(self):
        return self.qkv_proj.weight

    def forward(self, x, ctx, call, residual=None, upcoming=None):
        qkv = self.qkv_proj.forward(x, ctx, "qkv", fetch_ahead=self.o_proj.weight)
        kv = ctx.kv_cache(call.cache_slot)
        meta = ctx.attn_meta
        has_norm = self.qk_norm_eps is not None
        prep = (self.p("q_norm.weight") if has_norm else None, self.p("k_norm.weight") if has_norm else None,
                self.qk_norm_eps if has_norm else 0.0, self.rope.cos_sin if self.rope is not None else None)
        rotary_dim = self.rope.rotary_dim if self.rope is not None else None
        layout = self.rope.layout if self.rope is not None else "half_split"
        slots = kv.slot_mapping if call.writes_cache else None
        # Requests that bring one token come first in the batch.  Where the decode kernel takes the shape it
        # prepares q and the newest key and value itself; the other rows get the separate pass.
        D = meta.num_decodes
        fused = D > 0 and layout == "half_split" and ops.decode_fused_takes(qkv, self.head_dim, kv.pool, kv.page_size, meta,
                                                                            rotary_dim)
        first = D if fused else 0
        if first < qkv.shape[0]:
            ops.qk_norm_rope_kv_write(qkv[first:], self.num_heads, self.num_kv_heads, self.head_dim, *prep,
                                      ctx.positions[first:], slots[first:] if slots is not None else None,
                                      kv.pool, kv.page_size, rotary_dim=rotary_dim, layout=layout)
        out = ctx.buffer("attn_out", (qkv.shape[0], self.q_size), ctx.act_dtype)
        if fused:
            ops.attention_decode_fused(qkv, out, self.num_heads, self.num_kv_heads, self.head_dim, kv.pool, kv.page_size,
                                       kv.block_tables, meta, self.scale, self.window, *prep, slots)
        ops.paged_attention(qkv, out, self.num_heads, self.num_kv_heads, self.head_dim,
                            kv.pool, kv.page_size, kv.block_tables, meta,
                            self.scale, self.window, decodes=not fused)
        return self.o_proj.forward(out, ctx, "mixer_out", may_split=True, residual=residual,
                                   next_norm=upcoming.norm if upcoming else None,
                                   fetch_ahead=upcoming.weight if upcoming else None)


register_mixer("gqa_attention", GQAAttention)
