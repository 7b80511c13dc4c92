"""The cache manager: pages and block tables for every group of layers, and state slots.

What it takes from the reference (engine/block_manager.py:68-123): allocation for
``computed + new`` tokens that either succeeds as a whole or changes nothing; prefix reuse
by chained xxh64 hashes of full pages, verified against the tokens, never covering the last
token of a request (so at least one token is computed); pages hashed as soon as they fill;
release in reverse order so that a prefix's first pages are evicted last.

What it adds: several *groups*.  Layers whose mixers need the same thing of the cache
(every key, or a window of them; the same heads and head size) form a group with a page
pool and a block table of its own per request.  A window group gives a page back as soon
as every key in it lies behind the window of all tokens still to come; its table entry
becomes -1.  Prefix reuse is on only when every group keeps every key and no mixer has
state of its own, since a page that was given back, or a state, cannot be found again.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import xxhash

from .page_pool import PagePool
from .state_slots import StateSlotPool


@dataclass(frozen=True)
class GroupSpec:
    """One group of cache slots with the same needs."""
    window: Optional[int]            # None: every key is kept
    num_kv_heads: int
    head_dim: int
    cache_slots: tuple[int, ...]     # the model's cache slots that live in this group


class CacheHolder:
    """What a request holds of the cache; the scheduler's Sequence and replay's requests derive from it."""

    def __init__(self):
        self.block_tables: list[list[int]] = []     # one table per group; -1 = page given back
        self.num_released: list[int] = []           # leading pages already given back, per group
        self.state_slot: int = -1
        self.num_computed_tokens = 0
        self.num_cached_tokens = 0
        self.num_hashed_blocks = 0
        self.table_version = 0                      # bumped whenever a table changes other than by growing
        self._arrays: dict[int, tuple[int, np.ndarray]] = {}

    def table_array(self, g: int) -> np.ndarray:
        """Group ``g``'s block table as int32 (read only), kept up to date without converting the whole
        list at every step: pages are appended far more often than anything else happens to a table."""
        table = self.block_tables[g]
        ent = self._arrays.get(g)
        if ent is None or ent[0] != self.table_version or len(ent[1]) > len(table):
            arr = np.asarray(table, dtype=np.int32)
        else:
            arr = ent[1]
            if len(arr) < len(table):
                arr = np.concatenate((arr, np.asarray(table[len(arr):], dtype=np.int32)))
        self._arrays[g] = (self.table_version, arr)
        return arr


def compute_hash(token_ids: Sequence[int], prefix: int = -1) -> int:
    """xxh64 over the previous page's hash (8 bytes, little endian) and the page's tokens as int64
    (engine/block_manager.py:33-39)."""
    h = xxhash.xxh64()
    if prefix != -1:
        h.update(prefix.to_bytes(8, "little"))
    h.update(np.asarray(token_ids, dtype=np.int64).tobytes())
    return h.intdigest()


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], num_pages: int | Sequence[int], page_size: int,
                 num_state_slots: int = 0, enable_prefix_caching: bool = True, has_state: bool = False):
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.groups)
        self.pools = [PagePool(n) for n in num_pages]
        self.state_slots = StateSlotPool(num_state_slots)
        self.prefix_caching = bool(enable_prefix_caching and not has_state and self.groups
                                   and all(g.window is None for g in self.groups))
        self.num_prefix_hit_tokens = 0          # tokens that requests found in the cache instead of computing them

    # ---- sizes -----------------------------------------------------------------------
    @property
    def num_free_pages(self) -> list[int]:
        return [p.num_free for p in self.pools]

    def pages_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_size - 1) // self.page_size

    def fits_at_all(self, num_tokens: int, max_portion: Optional[int] = None) -> bool:
        """Could a request of this many tokens ever be held (with an empty pool)?

        A window group holds at most the window plus the portion being computed."""
        need = self.pages_for(num_tokens)
        portion = num_tokens if max_portion is None else min(num_tokens, max_portion)
        for g, pool in zip(self.groups, self.pools):
            n = need if g.window is None else min(need, self.pages_for(g.window + portion) + 1)
            if n > pool.num_pages:
                return False
        return True

    def _attach(self, holder: CacheHolder) -> None:
        if not holder.block_tables:
            holder.block_tables = [[] for _ in self.groups]
            holder.num_released = [0] * len(self.groups)

    # ---- prefix reuse ----------------------------------------------------------------
    def find_prefix_hit(self, token_ids: Sequence[int]) -> list[list[int]]:
        """Pages (per group) that already hold the leading full pages of ``token_ids``.

        Walks full pages up to ``(len-1)//page_size`` so that the last token is always left
        to compute (engine/block_manager.py:68-78)."""
        hits: list[list[int]] = [[] for _ in self.groups]
        if not self.prefix_caching:
            return hits
        ps = self.page_size
        h = -1
        for i in range((len(token_ids) - 1) // ps):
            toks = list(token_ids[i * ps:(i + 1) * ps])
            h = compute_hash(toks, h)
            pages = [pool.lookup(h, toks) for pool in self.pools]
            if any(p == -1 for p in pages):
                break
            for g, p in enumerate(pages):
                hits[g].append(p)
        return hits

    # ---- allocation ------------------------------------------------------------------
    def allocate(self, holder: CacheHolder, num_new_tokens: int,
                 hits: Optional[list[list[int]]] = None) -> bool:
        """Make room for ``num_new_tokens`` more tokens after the computed ones.

        All groups or none: returns False and changes nothing when any group is short
        (engine/block_manager.py:80-100).  ``hits`` may be given only for a holder without
        pages; the hit pages are shared and counted as computed."""
        self._attach(holder)
        ps = self.page_size
        n_hit = len(hits[0]) if hits and self.groups else 0
        if n_hit and any(holder.block_tables[g] for g in range(len(self.groups))):
            raise ValueError("prefix hits can only be given to a request that holds no pages")
        computed = holder.num_computed_tokens + n_hit * ps
        total = (computed + num_new_tokens + ps - 1) // ps
        fresh_needed = []
        for g, pool in enumerate(self.pools):
            have = len(holder.block_tables[g])
            fresh = max(0, total - have - n_hit)
            free_hits = sum(1 for p in (hits[g] if n_hit else []) if pool.ref_count[p] == 0)
            if fresh + free_hits > pool.num_free:
                return False
            fresh_needed.append(fresh)
        need_slot = holder.state_slot < 0 and self.state_slots.num_slots > 0
        if need_slot and self.state_slots.num_free == 0:
            return False
        for g, pool in enumerate(self.pools):
            table = holder.block_tables[g]
            if n_hit:
                for p in hits[g]:
                    pool.share(p)
                    table.append(p)
            for _ in range(fresh_needed[g]):
                table.append(pool.take_fresh())
        if n_hit:
            holder.num_computed_tokens = computed
            holder.num_cached_tokens += n_hit * ps
            self.num_prefix_hit_tokens += n_hit * ps
            holder.num_hashed_blocks += n_hit
        if need_slot:
            holder.state_slot = self.state_slots.acquire()
        return True

    def hash_full_pages(self, holder: CacheHolder, token_ids: Sequence[int]) -> None:
        """Hash the pages that have filled since the last call (engine/block_manager.py:102-113)."""
        if not self.prefix_caching:
            return
        ps = self.page_size
        end = holder.num_computed_tokens // ps
        for i in range(holder.num_hashed_blocks, end):
            toks = list(token_ids[i * ps:(i + 1) * ps])
            for g, pool in enumerate(self.pools):
                table = holder.block_tables[g]
                prefix = pool.page_hash[table[i - 1]] if i > 0 else -1
                if i > 0 and prefix == -1:
                    raise RuntimeError("a page is hashed before the page in front of it")
                pool.set_hash(table[i], compute_hash(toks, prefix), toks)
        holder.num_hashed_blocks = max(holder.num_hashed_blocks, end)

    def release_behind_window(self, holder: CacheHolder) -> int:
        """Give back the pages of window groups that no token still to come can see.

        A token at position p >= computed sees keys j > p - window, so a page whose last key
        lies at or before ``computed - window`` is behind every window to come."""
        released = 0
        ps = self.page_size
        for g, (spec, pool) in enumerate(zip(self.groups, self.pools)):
            if spec.window is None or not holder.block_tables:
                continue
            first_needed = holder.num_computed_tokens - spec.window + 1     # lowest key still visible
            table = holder.block_tables[g]
            i = holder.num_released[g]
            while i < len(table) and (i + 1) * ps <= first_needed:
                if table[i] >= 0:
                    pool.release(table[i])
                    table[i] = -1
                    holder.table_version += 1
                    released += 1
                i += 1
            holder.num_released[g] = i
        return released

    def free(self, holder: CacheHolder) -> None:
        """Give back everything the holder has (finish or preemption), last pages first
        (engine/block_manager.py:115-123)."""
        if holder.block_tables:
            for g, pool in enumerate(self.pools):
                for p in reversed(holder.block_tables[g]):
                    if p >= 0:
                        pool.release(p)
                holder.block_tables[g].clear()
                holder.num_released[g] = 0
            holder.table_version += 1
        if holder.state_slot >= 0:
            self.state_slots.release(holder.state_slot)
            holder.state_slot = -1
        holder.num_computed_tokens = 0
        holder.num_cached_tokens = 0
        holder.num_hashed_blocks = 0

    def check(self, holders: Sequence[CacheHolder] = ()) -> None:
        """Invariants over the pools and, if given, over all live holders: no page lost, no page
        held by more tables than its count says."""
        for pool in self.pools:
            pool.check()
        self.state_slots.check()
        if holders:
            for g, pool in enumerate(self.pools):
                counts = [0] * pool.num_pages
                for h in holders:
                    if h.block_tables:
                        for p in h.block_tables[g]:
                            if p >= 0:
                                counts[p] += 1
                if counts != pool.ref_count:
                    raise RuntimeError(f"group {g}: tables and reference counts disagree")
            slots = [h.state_slot for h in holders if h.state_slot >= 0]
            if len(slots) != len(set(slots)):
                raise RuntimeError("a state slot is held by two requests")
