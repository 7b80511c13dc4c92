"""Everything one step knows, handed to every part explicitly.

The reference passes this through a module global (utils/context.py:3-27: cu_seqlens_q,
slot_mapping, context_lens, block_tables, num_decodes, logits_indices, ...).  Here it is an
object: device tensors that kernels read, the same numbers on the host for parts that
decide in Python, the cache storage, and named work buffers that are reused from step to
step (a CUDA graph keeps a context of its own, so its buffers never move).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import weakref

import torch


@dataclass
class KVView:
    """One cache slot's pages as the mixer sees them in this step."""
    pool: torch.Tensor                 # [num_pages, 2, kv_heads, page_size, head_dim]
    page_size: int
    block_tables: torch.Tensor         # [B, max_pages] int32, -1 where there is no page
    slot_mapping: torch.Tensor         # [T] int32: page * page_size + offset, -1 = do not write
    group: int


@dataclass
class AttnMeta:
    """Batch shape for the attention kernels.  Requests [0, num_decodes) bring one token each."""
    num_reqs: int
    num_tokens: int
    num_decodes: int
    cu_seqlens: torch.Tensor           # [B+1] int32
    context_lens: torch.Tensor         # [B] int32: keys of the request after this step
    tile_lists: dict                   # tile size -> ([n, 2] int32 (request, first local query), n), requests >= num_decodes
    num_tiles: int                     # > 0 if any request brings several tokens
    max_context_len: int               # host upper bound of context_lens (sizes split-K scratch)
    workspace: Any                     # callable (name, shape, dtype) -> tensor
    error_flag: Any = None             # int32[4] on the device: kernels report bad input or a timed-out wait here
    scratch_context_len: int = 0       # if larger than max_context_len: size split-K scratch for this many keys (so it never has to grow)
    typical_context_len: int = 0       # what contexts a captured step will mostly see (0: max_context_len); picks kernel variants


@dataclass
class HostMeta:
    """The step's shape on the host, in batch order."""
    starts: list[int]                  # position of each request's first token in this step
    lengths: list[int]                 # tokens of each request in this step
    state_slots: list[int]
    holders: list[Any]


class StepContext:
    def __init__(self, runner, arena: Optional[dict] = None):
        self._runner = weakref.ref(runner)       # no cycle: a dropped runner frees its memory at once
        self.act_dtype: torch.dtype = runner.act_dtype
        self.device = runner.device
        self.error_flag: torch.Tensor = runner.error_flag
        self._arena: dict[str, torch.Tensor] = {} if arena is None else arena
        self._views: dict = {}
        self.frozen = False            # a captured graph's buffers must not be reallocated
        self.on_replace = None         # called with a buffer's name before a larger one takes its place
        self.token_feedback = getattr(runner, "token_feedback", None)   # int32 on the device: a token id ~j in a step means entry j of it
        # Filled per step:
        self.positions: torch.Tensor = None
        self.token_req: torch.Tensor = None
        self.state_slots: torch.Tensor = None
        self.logits_rows: torch.Tensor = None
        self.sample_temps: torch.Tensor = None
        self.sample_seeds: torch.Tensor = None
        self.sample_positions: torch.Tensor = None
        self.attn_meta: AttnMeta = None
        self.host: HostMeta = None
        self._bt: list[torch.Tensor] = []
        self._sm: list[torch.Tensor] = []

    @property
    def runner(self):
        return self._runner()

    def buffer(self, name: str, shape, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A work buffer by name: the same storage every step, grown when a step needs more.
        ``zero``: the storage is zeroed when it is made (for counters that kernels leave at zero)."""
        key = (name, tuple(shape), dtype)
        hit = self._views.get(key)
        if hit is not None and hit[0] is self._arena.get(name):
            return hit[1]
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(n * dtype.itemsize, 16)
        flat = self._arena.get(name)
        if flat is None or flat.numel() < nbytes:
            if self.frozen:
                raise RuntimeError(f"work buffer {name!r} would move under a captured graph")
            if flat is not None and self.on_replace is not None:
                self.on_replace(name)               # others that recorded the old storage must forget it
            flat = (torch.zeros if zero else torch.empty)(nbytes + (-nbytes) % 256, dtype=torch.uint8, device=self.device)
            self._arena[name] = flat
        view = flat[:n * dtype.itemsize].view(dtype).view(*shape)
        self._views[key] = (flat, view)              # the same tensor object until the storage is replaced
        return view

    def kv_cache(self, cache_slot: int) -> KVView:
        g, idx = self.runner.slot_location[cache_slot]
        return KVView(self.runner.kv_pools[g][idx], self.runner.page_size, self._bt[g], self._sm[g], g)

    def state(self, cache_slot: int) -> torch.Tensor:
        """Storage of a mixer's per-request state: [num_state_slots, *shape] of the dtype its ``StateNeed`` names."""
        return self.runner.state_storage[cache_slot]
