"""The model runner: weights, cache storage and ONE step function.

Reference (engine/model_runner.py:24-145): ``run(seqs)`` flattens a ragged batch (single
decoded tokens first, then portions of prompts), copies the metadata to the device, runs
the model on exactly those tokens against the paged cache and computes logits only at the
rows that sample.  Here ``step(items)`` does the same for any caller (the engine's
scheduler, trace replay, tests): an item is (what the request holds of the cache, its next
tokens, the position of the first, the places whose logits are wanted) and the result is
the float32 logits of the wanted places, in the order of the items.  The metadata of a
step is built with numpy into one pinned buffer and reaches the device in one copy.
Steps that only decode replay a CUDA graph per batch-size bucket.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import gc

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheHolder, CacheManager, GroupSpec
from ..config.registry import get_architecture, load_model_config
from ..parts.base import KVCacheNeed, StateNeed
from ..parts.model import DecoderModel
from ..weights.loader import load_weights
from ..weights.random_init import init_random_on_device
from .step_context import AttnMeta, HostMeta, StepContext

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass
class StepItem:
    holder: CacheHolder            # block tables (per group) and state slot of the request
    tokens: Sequence[int]          # the request's next tokens
    start: int                     # position of tokens[0] in the request
    want: Sequence[int] = ()       # places among ``tokens`` whose logits are wanted
    sampling: Optional[tuple[float, int]] = None   # (temperature, seed) when tokens are to be drawn


@dataclass
class StepResult:
    logits: Optional[torch.Tensor]     # [wanted, vocab] float32, in the order of the items and their ``want``
    tokens: Optional[torch.Tensor]     # [wanted] int32, drawn on the device when the step was asked to sample


class _StepGraph:
    """A captured step of fixed shape: a decode step for a number of requests and a bound on their contexts, or one
    request's portion of a prompt.  It has its own context and metadata; the work buffers are shared by the decode
    graphs of one batch bucket (they never run at the same time), a prompt graph has its own."""

    def __init__(self, runner, bucket: int, arena: dict):
        self.bucket = bucket
        self.ctx = StepContext(runner, arena=arena)
        self.meta_dev: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.tokens: Optional[torch.Tensor] = None
        self.launches = 0
        self.form: Optional[str] = None          # the decode attention form the capture was tuned to, if it was


def plan_cache_groups(model: DecoderModel) -> tuple[list[GroupSpec], dict[int, tuple[int, int]], dict[int, StateNeed]]:
    """Group the model's cache slots by what they need; returns (groups, slot -> (group, index), slot -> state)."""
    keyed: dict[tuple, list[int]] = {}
    states: dict[int, StateNeed] = {}
    for slot, needs in enumerate(model.slot_needs):
        for need in needs:
            if isinstance(need, KVCacheNeed):
                keyed.setdefault((need.window, need.num_kv_heads, need.head_dim), []).append(slot)
            elif isinstance(need, StateNeed):
                states[slot] = need
            else:
                raise TypeError(f"cache slot {slot}: unknown kind of cache need {need!r}")
    groups, location = [], {}
    for (window, nkv, hd), slots in keyed.items():
        for i, s in enumerate(slots):
            location[s] = (len(groups), i)
        groups.append(GroupSpec(window, nkv, hd, tuple(slots)))
    return groups, location, states


class ModelRunner:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", page_size: int = 16,
                 num_pages: int = -1, max_num_seqs: int = 512, max_num_batched_tokens: int = 16384,
                 max_model_len: int = 4096, gpu_memory_utilization: float = 0.9,
                 use_cuda_graphs: bool = True, device: str = "cuda:0", model_config=None,
                 random_weights_seed: Optional[int] = None):
        ops.require_extension()                      # fails loudly when the kernels cannot be had
        self.device = torch.device(device)
        self.act_dtype = _TORCH_DTYPE[dtype]
        self.page_size = page_size
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.model_config = model_config or load_model_config(model_dir)
        self.max_model_len = min(max_model_len, self.model_config.max_position_embeddings)
        arch = get_architecture(self.model_config.architecture)
        self.model = DecoderModel(arch.plan(self.model_config))
        if random_weights_seed is None:
            load_weights(self.model, model_dir, self.act_dtype, self.device)
        else:                                        # the folder holds a config.json only
            init_random_on_device(self.model, random_weights_seed, self.act_dtype, self.device)
        self.model.finalize_all(self.act_dtype, self.device)
        self.vocab_size = self.model.plan.vocab_size

        self.groups, self.slot_location, self.state_needs = plan_cache_groups(self.model)
        self.error_flag = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.num_state_slots = max_num_seqs if self.state_needs else 0
        self.state_storage = {slot: torch.zeros(self.num_state_slots, *need.shape, dtype=getattr(torch, need.dtype),
                                                device=self.device)
                              for slot, need in self.state_needs.items()}
        # Four error flags and the tokens drawn by the last step whose results were staged here: one copy to the host,
        # and the place where a step launched ahead of the host finds the tokens it continues from (a token id ~j).
        self.result_dev = torch.zeros(4 + max_num_seqs, dtype=torch.int32, device=self.device)
        self.token_feedback = self.result_dev[4:]
        self._pins: list[Optional[torch.Tensor]] = [None, None]     # pinned host int32, used in turn
        self._pin_events: list[Any] = [None, None]
        self._pin_turn = 0
        self._staging_dev: Optional[torch.Tensor] = None
        self.last_h2d_bytes = 0
        # A decode step is replayed from a graph only if every part of the model allows it.
        self.use_cuda_graphs = (use_cuda_graphs and self.device.type == "cuda"
                                and all(part.capturable for _, part in self.model.walk()))
        self._graphs: dict[tuple[int, int], _StepGraph] = {}
        self._graph_arenas: dict[int, dict] = {}
        self.graph_buckets = [b for b in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256) if b <= max_num_seqs]
        # A portion of one prompt, alone in its step, is replayed from a graph as well once its shape (tokens, wanted
        # places) has come twice: the portions of a long prompt all have the step's token budget.  The host needs
        # longer to launch such a step's kernels one by one than the device to run them, up to some 1,500 tokens.
        self.prefill_graph_min_tokens = 128      # below, products go to the library and the step is short anyway
        self.prefill_graph_max = 4               # graphs kept (each has work buffers of its own); the oldest goes first
        self._prefill_graphs: dict[tuple, _StepGraph] = {}
        self._prefill_seen: dict[tuple, int] = {}
        self.graph_launches = 0          # kernels replayed from graphs (they bypass ops.launches)
        self.tune_decode_form = True     # a captured decode step keeps the fastest form of the decode attention kernel
        self.tune_decode_max_bucket = 32 # ... measured for batch buckets below this one; by rule from there on
        self.tune_decode_max_step_ms = 2.0   # ... and only while a step is shorter than this: a capture of 36 large layers
                                             # costs 0.1 s, which the few microseconds a layer between the forms never repay
        self.pool_sizing: dict = {}      # what the pool was sized from, when it was sized here
        self.num_pages = num_pages if num_pages > 0 else self._size_pool(gpu_memory_utilization)
        self.kv_pools = self._make_pools(self.num_pages)
        self.ctx = StepContext(self)

    # ---- sizes -----------------------------------------------------------------------
    def page_bytes(self) -> int:
        """Bytes of one page over all groups and their cache slots."""
        return sum(len(g.cache_slots) * 2 * g.num_kv_heads * self.page_size * g.head_dim
                   for g in self.groups) * self.act_dtype.itemsize

    def _make_pools(self, num_pages: int) -> list[torch.Tensor]:
        return [torch.zeros(len(g.cache_slots), num_pages, 2, g.num_kv_heads, self.page_size, g.head_dim,
                            dtype=self.act_dtype, device=self.device) for g in self.groups]

    def _size_pool(self, utilization: float) -> int:
        """Pages that fit into the share of device memory the engine may use, after the weights and the work
        buffers.  As the reference does (engine/model_runner.py:52-80), the work buffers are measured: with a pool
        of one page, and block tables that all point at it, the largest step of prompt portions and the largest
        step of single tokens are run once, kernel by kernel.  What the captured steps will take on top of that
        (an arena of work buffers per batch bucket, up to ``prefill_graph_max`` prompt graphs with buffers of
        their own) is counted from those two measurements."""
        from ..cache.manager import CacheHolder
        dev = self.device
        ps = self.page_size
        self.num_pages, self.kv_pools = 1, self._make_pools(1)
        self.ctx = StepContext(self)
        graphs, self.use_cuda_graphs = self.use_cuda_graphs, False

        def dummy(tokens: int) -> CacheHolder:
            h = CacheHolder()
            h.block_tables = [[0] * ((tokens + ps - 1) // ps) for _ in self.groups]
            h.num_released = [0] * len(self.groups)
            h.state_slot = 0 if self.state_needs else -1
            return h

        def used() -> int:
            torch.cuda.synchronize(dev)
            free, total = torch.cuda.mem_get_info(dev)
            return total - free

        def held() -> int:
            return torch.cuda.memory_allocated(dev)
        # What a step takes is the growth of the device's used memory, or, where the allocator served the step from
        # memory it held already (a process that has run other engines), the growth of what the allocator has given out.
        torch.cuda.empty_cache()
        base, base_held = used(), held()
        torch.cuda.reset_peak_memory_stats(dev)
        L = self.max_model_len
        m = min(L, self.max_num_batched_tokens)
        n = max(1, min(self.max_num_batched_tokens // m, self.max_num_seqs))
        self.step([StepItem(dummy(m), [0] * m, 0, [m - 1]) for _ in range(n)], sample=True)
        after_prompts, prompts_held = used(), held()
        prompt_bytes = max(after_prompts - base, torch.cuda.max_memory_allocated(dev) - base_held)
        torch.cuda.reset_peak_memory_stats(dev)
        self.step([StepItem(dummy(L), [0], L - 1, [0], (1.0, 0)) for _ in range(self.max_num_seqs)], sample=True)
        token_bytes = max(used() - after_prompts, torch.cuda.max_memory_allocated(dev) - prompts_held, 0)
        self.check_device_errors()
        allowance = 0
        if graphs:
            # the arena of a batch bucket grows with the bucket: all of them together, in units of the largest step
            share = sum(self.graph_buckets) / max(self.max_num_seqs, 1)
            allowance = int((prompt_bytes / max(n * m, 1) * self.max_num_seqs + token_bytes) * share) \
                + self.prefill_graph_max * prompt_bytes
        self.use_cuda_graphs = graphs
        free, total = torch.cuda.mem_get_info(dev)
        budget = int(total * utilization) - (total - free) - allowance
        self.pool_sizing = {"work_prompts": prompt_bytes, "work_tokens": token_bytes, "graphs": allowance, "budget": budget}
        n_pages = budget // max(self.page_bytes(), 1)
        # No request can use more than max_model_len tokens, so more pages than all requests
        # could fill are never touched.
        cap = self.max_num_seqs * ((self.max_model_len + self.page_size - 1) // self.page_size)
        n_pages = min(n_pages, cap)
        if n_pages < 1:
            raise RuntimeError("no device memory left for the cache pool: lower max_num_seqs / "
                               "max_num_batched_tokens or raise gpu_memory_utilization")
        self.kv_pools = []
        return int(n_pages)

    def make_cache_manager(self, enable_prefix_caching: bool = True) -> CacheManager:
        return CacheManager(self.groups, self.num_pages, self.page_size,
                            num_state_slots=self.num_state_slots,
                            enable_prefix_caching=enable_prefix_caching,
                            has_state=bool(self.state_needs))

    # ---- the step --------------------------------------------------------------------
    def _stage(self, n_ints: int, dev: Optional[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
        """A pinned host buffer whose last copy has finished, and the device buffer it goes to."""
        k = self._pin_turn = 1 - self._pin_turn
        if self._pin_events[k] is not None:
            self._pin_events[k].synchronize()
        if self._pins[k] is None or self._pins[k].numel() < n_ints:
            self._pins[k] = torch.empty(max(n_ints * 2, 1 << 16), dtype=torch.int32, pin_memory=True)
        if dev is None:
            if self._staging_dev is None or self._staging_dev.numel() < n_ints:
                self._staging_dev = torch.empty(max(n_ints * 2, 1 << 16), dtype=torch.int32, device=self.device)
            dev = self._staging_dev
        return self._pins[k], dev

    def build_batch(self, items: Sequence[StepItem], ctx: StepContext, *, pad_reqs: int = 0,
                    table_width: int = 0, dev: Optional[torch.Tensor] = None,
                    fill_ctx: bool = True, typical_context: int = 0) -> tuple[Optional[torch.Tensor], list[int]]:
        """Lay the step's metadata out in pinned memory, copy it once, fill ``ctx``.

        Requests that bring one token come first (as in engine/model_runner.py:88-89).
        ``pad_reqs``/``table_width`` give a fixed shape to steps replayed from a graph: padding
        requests have no keys and write nowhere.  Returns (token ids on the device, the batch
        order as indices into ``items``).  With ``fill_ctx`` False only the copy is made: a captured graph
        already knows where every array lies."""
        order = [i for i, it in enumerate(items) if len(it.tokens) == 1] + \
                [i for i, it in enumerate(items) if len(it.tokens) != 1]
        D = sum(1 for it in items if len(it.tokens) == 1)
        lens = [len(items[i].tokens) for i in order]
        if any(n < 1 for n in lens):
            raise ValueError("every item of a step must bring at least one token")
        B_real = len(order)
        B = max(B_real, pad_reqs)
        pad = B - B_real
        T_real = sum(lens)
        T = T_real + pad
        ps = self.page_size
        G = len(self.groups)
        starts = [items[i].start for i in order]
        ends = [s + n for s, n in zip(starts, lens)]
        if ends and max(ends) > self.model_config.max_position_embeddings:
            raise ValueError(f"position {max(ends) - 1} is beyond max_position_embeddings")
        widths = []
        for g in range(G):
            w = max([len(items[i].holder.block_tables[g]) for i in order] + [1, table_width])
            widths.append(w)
        want_rows: list[int] = []
        offsets = {}
        off = 0
        for k, i in enumerate(order):
            offsets[i] = off
            off += lens[k]
        for i, it in enumerate(items):
            for w in it.want:
                if not 0 <= w < len(it.tokens):
                    raise ValueError(f"wanted place {w} is outside the item's {len(it.tokens)} tokens")
                want_rows.append(offsets[i] + w)
        S_real = len(want_rows)
        if pad_reqs:                                  # fixed shape: as many rows as requests
            want_rows += [0] * (B - S_real)
        S = len(want_rows)
        tile_np = {}
        for tq in ops.ATTN_TILE_SIZES:
            per_req = [np.stack((np.full((lens[b] + tq - 1) // tq, b, dtype=np.int32),
                                 np.arange(0, lens[b], tq, dtype=np.int32)), axis=1) for b in range(D, B_real)]
            tile_np[tq] = np.concatenate(per_req).reshape(-1) if per_req else np.zeros(0, dtype=np.int32)
        n_tiles = sum(len(a) // 2 for a in tile_np.values())

        def al(n):                       # keep every array 16-byte aligned on the device
            return (n + 3) & ~3
        sizes = dict(tok=al(T), pos=al(T), req=al(T), cu=al(B + 1), ctxlen=al(B), slot=al(B),
                     rows=al(max(S, 1)), temp=al(max(S, 1)), seed=al(max(S, 1)), spos=al(max(S, 1)),
                     tiles=sum(al(max(len(a), 1)) for a in tile_np.values()))
        total = sum(sizes.values()) + sum(al(T) + al(B * widths[g]) for g in range(G))
        pin, dev = self._stage(total, dev)
        if dev.numel() < total:
            raise RuntimeError("a captured step's metadata outgrew its buffer")
        host = pin.numpy()
        cur = 0

        def take(n):
            nonlocal cur
            a, cur = cur, cur + n
            return a
        o_tok, o_pos, o_req = take(sizes["tok"]), take(sizes["pos"]), take(sizes["req"])
        o_cu, o_ctx, o_slot = take(sizes["cu"]), take(sizes["ctxlen"]), take(sizes["slot"])
        o_rows, o_temp, o_seed, o_spos = (take(sizes[k]) for k in ("rows", "temp", "seed", "spos"))
        o_tiles = take(sizes["tiles"])
        o_sm = [take(al(T)) for _ in range(G)]
        o_bt = [take(al(B * widths[g])) for g in range(G)]

        host[o_tok:o_tok + T] = 0
        host[o_pos:o_pos + T] = 0
        t = 0
        cu = [0]
        for k, i in enumerate(order):
            n = lens[k]
            if n == 1:                              # single tokens: plain integers beat array calls
                host[o_tok + t] = items[i].tokens[0]
                host[o_pos + t] = starts[k]
                host[o_req + t] = k
            else:
                host[o_tok + t:o_tok + t + n] = np.asarray(items[i].tokens, dtype=np.int32)
                host[o_pos + t:o_pos + t + n] = np.arange(starts[k], ends[k], dtype=np.int32)
                host[o_req + t:o_req + t + n] = k
            t += n
            cu.append(t)
        for k in range(pad):
            host[o_req + T_real + k] = B_real + k
            cu.append(T_real + k + 1)
        host[o_cu:o_cu + B + 1] = cu
        host[o_ctx:o_ctx + B] = ends + [0] * pad
        host[o_slot:o_slot + B] = [items[i].holder.state_slot for i in order] + [-1] * pad
        if S:
            host[o_rows:o_rows + S] = want_rows
            temps, seeds, spos = [], [], []
            for i, it in enumerate(items):
                t_, s_ = it.sampling if it.sampling is not None else (0.0, 0)
                for w in it.want:
                    temps.append(t_)
                    seeds.append(int(s_) & 0x7FFFFFFF)
                    spos.append(it.start + w + 1)      # position of the token that is drawn
            padn = S - S_real
            host[o_temp:o_temp + S] = np.asarray(temps + [0.0] * padn, dtype=np.float32).view(np.int32)
            host[o_seed:o_seed + S] = seeds + [0] * padn
            host[o_spos:o_spos + S] = spos + [0] * padn
        tile_off, cur_t = {}, o_tiles
        for tq, a in tile_np.items():
            tile_off[tq] = cur_t
            host[cur_t:cur_t + len(a)] = a
            cur_t += al(max(len(a), 1))
        for g in range(G):
            w = widths[g]
            bt = host[o_bt[g]:o_bt[g] + B * w].reshape(B, w)
            bt[:] = -1
            sm = host[o_sm[g]:o_sm[g] + T]
            sm[:] = -1
            t = 0
            for k, i in enumerate(order):
                holder = items[i].holder
                table = holder.table_array(g) if hasattr(holder, "table_array") else \
                    np.asarray(holder.block_tables[g], dtype=np.int32)
                bt[k, :len(table)] = table
                if lens[k] == 1:
                    pos = starts[k]
                    pi = pos // ps
                    if len(table) <= pi:
                        raise ValueError("a request's block table does not cover its new tokens")
                    page = int(table[pi])
                    if page < 0:
                        raise ValueError("a new token would be written to a page that was given back")
                    sm[t] = page * ps + (pos - pi * ps)
                    t += 1
                    continue
                pos = np.arange(starts[k], ends[k])
                page = pos // ps
                if len(table) <= int(page[-1]):
                    raise ValueError("a request's block table does not cover its new tokens")
                pages = table[page]
                if (pages < 0).any():
                    raise ValueError("a new token would be written to a page that was given back")
                sm[t:t + lens[k]] = pages * ps + pos % ps
                t += lens[k]
        dev[:total].copy_(pin[:total], non_blocking=True)
        ev = self._pin_events[self._pin_turn]
        if ev is None and self.device.type == "cuda":
            ev = self._pin_events[self._pin_turn] = torch.cuda.Event()
        if ev is not None:
            ev.record()
        self.last_h2d_bytes = total * 4
        self.last_num_wanted = S_real
        if not fill_ctx:
            return None, order

        ctx.positions = dev[o_pos:o_pos + T]
        ctx.token_req = dev[o_req:o_req + T]
        ctx.state_slots = dev[o_slot:o_slot + B]
        ctx.logits_rows = dev[o_rows:o_rows + S]
        ctx.sample_temps = dev[o_temp:o_temp + S].view(torch.float32)
        ctx.sample_seeds = dev[o_seed:o_seed + S]
        ctx.sample_positions = dev[o_spos:o_spos + S]
        ctx._bt = [dev[o_bt[g]:o_bt[g] + B * widths[g]].view(B, widths[g]) for g in range(G)]
        ctx._sm = [dev[o_sm[g]:o_sm[g] + T] for g in range(G)]
        ctx.attn_meta = AttnMeta(
            num_reqs=B, num_tokens=T, num_decodes=D + pad if pad_reqs else D,
            cu_seqlens=dev[o_cu:o_cu + B + 1], context_lens=dev[o_ctx:o_ctx + B],
            tile_lists={tq: (dev[tile_off[tq]:tile_off[tq] + max(len(a), 2)].view(-1, 2), len(a) // 2)
                        for tq, a in tile_np.items()},
            num_tiles=n_tiles,
            max_context_len=max(ends + [1]) if not table_width else table_width * ps,
            workspace=ctx.buffer, error_flag=self.error_flag,
            scratch_context_len=self.max_model_len if table_width else 0,
            typical_context_len=typical_context)
        ctx.host = HostMeta(starts=starts, lengths=lens,
                            state_slots=[items[i].holder.state_slot for i in order],
                            holders=[items[i].holder for i in order])
        return dev[o_tok:o_tok + T], order

    def _forward(self, token_ids: torch.Tensor, ctx: StepContext, sample: bool):
        hidden = self.model.forward(token_ids, ctx)
        if ctx.logits_rows.numel() == 0:
            return None, None
        logits = self.model.compute_logits(hidden, ctx)
        tokens = None
        if sample:
            tokens = ctx.buffer("sampled_tokens", (logits.shape[0],), torch.int32)
            ops.sample(logits, ctx.sample_temps, ctx.sample_seeds, ctx.sample_positions, tokens, workspace=ctx.buffer)
        return logits, tokens

    @torch.inference_mode()
    def step(self, items: Sequence[StepItem], sample: bool = False) -> StepResult:
        """Run exactly the tokens of ``items`` as one batch against the cache.

        Returns the float32 logits ``[wanted, vocab]`` in the order of the items and of each item's
        ``want`` and, with ``sample``, the tokens drawn from them on the device.  Both are work
        buffers that the next step overwrites."""
        if not items:
            return StepResult(None, None)
        if len(items) > self.max_num_seqs:
            raise ValueError(f"{len(items)} requests in one step, max_num_seqs is {self.max_num_seqs}")
        if self.use_cuda_graphs and all(len(it.tokens) == 1 for it in items):
            bucket = next((b for b in self.graph_buckets if b >= len(items)), None)
            if bucket is not None:
                return self._step_graph(items, bucket, sample)
        if (self.use_cuda_graphs and len(items) == 1 and len(items[0].tokens) >= self.prefill_graph_min_tokens
                and len(items[0].want) <= 8):            # (a graph keeps its own logits: not for replays that want every place)
            result = self._step_prefill_graph(items, sample)
            if result is not None:
                return result
        token_ids, _ = self.build_batch(items, self.ctx)
        logits, tokens = self._forward(token_ids, self.ctx, sample)
        return StepResult(logits, tokens)

    def _capture(self, g: _StepGraph, token_ids: torch.Tensor, sample: bool) -> None:
        """Run the step once eagerly (this allocates the graph's work buffers), then capture it; both runs do the
        step's real work."""
        g.ctx.frozen = False
        self._forward(token_ids, g.ctx, sample)
        torch.cuda.current_stream().synchronize()
        g.ctx.frozen = True
        before = ops.launches
        graph = torch.cuda.CUDAGraph()
        # Nothing may free device or pinned memory while the stream is capturing: Python's collector is
        # paused, and calls that have nothing to do with the capture do not invalidate it.
        gc.disable()
        try:
            with torch.cuda.graph(graph, capture_error_mode="relaxed"):
                g.logits, g.tokens = self._forward(token_ids, g.ctx, sample)
        finally:
            gc.enable()
        g.launches = ops.launches - before
        g.graph = graph

    def _capture_fastest_form(self, g: _StepGraph, token_ids: torch.Tensor) -> None:
        """Capture a decode step once for every form of the decode attention kernel that takes the shape, replay each a
        few times and keep the fastest.  Which form wins depends on the batch, the context and the GPU at hand (two B200
        boxes ranked them differently at a batch of 8), so it is measured where it matters instead of guessed; a replay
        of the same step writes the same values again, so the extra replays change nothing.

        Only small batches are measured (buckets below ``tune_decode_max_bucket``): there the step is a chain of short
        kernels and the forms lie close together; a large batch has many blocks an SM, where one form wins by rule, its
        graphs are many (narrow context buckets) and each measurement costs a tenth of a second: a workload of 256
        requests that end one after the other spent a third of its time measuring."""
        tune = self.tune_decode_form and ops.decode_form == "auto" and g.bucket < self.tune_decode_max_bucket
        forms = ops.decode_forms_for(self.page_size) if tune else [None]
        best = None
        try:
            for form in forms:
                ops.decode_form = form or "auto"
                self._capture(g, token_ids, True)
                if len(forms) == 1:
                    return
                for _ in range(2):
                    g.graph.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(4):
                    g.graph.replay()
                e1.record()
                e1.synchronize()
                t = e0.elapsed_time(e1)
                if best is None or t < best[0]:
                    best = (t, form, g.graph, g.logits, g.tokens, g.launches)
                if t / 4 > self.tune_decode_max_step_ms:
                    break                            # a long step (large layers): the forms differ by a per cent of it at most
        finally:
            ops.decode_form = "auto"
        _, g.form, g.graph, g.logits, g.tokens, g.launches = best

    def _step_prefill_graph(self, items: Sequence[StepItem], sample: bool) -> Optional[StepResult]:
        """One request's portion of a prompt from a graph; None while the shape has not come twice.

        Nothing that is launched for such a step depends on the request's context: the attention kernel's grid
        follows from the number of query tiles, its loops from the lengths on the device.  So the key is the number
        of tokens and of wanted places, and the block table has the width of the longest request there can be."""
        item = items[0]
        key = (len(item.tokens), len(item.want), bool(sample))
        g = self._prefill_graphs.get(key)
        if g is None:
            seen = self._prefill_seen[key] = self._prefill_seen.get(key, 0) + 1
            if seen < 2:
                return None
            while len(self._prefill_graphs) >= self.prefill_graph_max:
                self._prefill_graphs.pop(next(iter(self._prefill_graphs)))
            g = self._prefill_graphs[key] = _StepGraph(self, 0, {})
        width = (self.max_model_len + self.page_size - 1) // self.page_size
        if g.meta_dev is None:
            T = len(item.tokens)
            n = 8 * T + 64 + sum(T + width + 16 for _ in self.groups) + 8 * max(len(item.want), 1)
            g.meta_dev = torch.zeros(n + 64, dtype=torch.int32, device=self.device)
        token_ids, _ = self.build_batch(items, g.ctx, table_width=width, dev=g.meta_dev, fill_ctx=g.graph is None)
        if g.graph is None:
            self._capture(g, token_ids, sample)
        g.graph.replay()
        self.graph_launches += g.launches
        if g.logits is None:
            return StepResult(None, None)
        return StepResult(g.logits, g.tokens if sample else None)

    def _step_graph(self, items: Sequence[StepItem], bucket: int, sample: bool) -> StepResult:
        """Decode-only steps replay a graph captured for the bucket: metadata goes to fixed device
        addresses, padding requests have no keys, write nowhere and their rows are ignored."""
        # The graph's shape also fixes how many key partitions the attention kernel is launched for, so graphs
        # are kept per context bucket as well.  For large batches the buckets are narrow (steps of 256 tokens up
        # to 2,048, of 512 up to 8,192, of 2,048 beyond): a block for a partition that no request reaches costs
        # little, but with powers of two there are nearly as many of them as of the others (measured at batch
        # 256: 8.9 against 9.5 ms a step).  Small batches keep powers of two: fewer graphs, and the step was
        # not faster with narrow buckets (batch 8: 1.00 against 0.97 ms).
        longest = max(it.start for it in items) + 1
        if bucket >= 32:
            step = 256 if longest <= 2048 else (512 if longest <= 8192 else 2048)
            ctx_bucket = (longest + step - 1) // step * step
        else:
            ctx_bucket = 256
            while ctx_bucket < longest:
                ctx_bucket *= 2
        ctx_bucket = min(ctx_bucket, (self.max_model_len + self.page_size - 1) // self.page_size * self.page_size)
        if longest > ctx_bucket:
            raise ValueError(f"a request is at position {longest - 1}, beyond max_model_len {self.max_model_len}")
        width = (ctx_bucket + self.page_size - 1) // self.page_size
        g = self._graphs.get((bucket, ctx_bucket))
        if g is None:
            arena = self._graph_arenas.setdefault(bucket, {})
            g = self._graphs[(bucket, ctx_bucket)] = _StepGraph(self, bucket, arena)
            # a buffer that has to grow (scratch sized by the context bucket) takes the bucket's other graphs with it
            g.ctx.on_replace = lambda name, b=bucket, keep=(bucket, ctx_bucket): [
                self._graphs.pop(k) for k in list(self._graphs) if k[0] == b and k != keep]
            n = 16 * bucket + 64 + sum(4 * bucket + bucket * width + 8 for _ in self.groups)
            g.meta_dev = torch.zeros(n + 64, dtype=torch.int32, device=self.device)
        # the graph serves contexts from the bucket below up to this one: its kernels are chosen for the middle
        token_ids, _ = self.build_batch(items, g.ctx, pad_reqs=bucket, table_width=width, dev=g.meta_dev,
                                        fill_ctx=g.graph is None,
                                        typical_context=ctx_bucket * 3 // 4 if bucket < 32 else max(ctx_bucket - 128, 1))
        if g.graph is None:
            self._capture_fastest_form(g, token_ids)
        g.graph.replay()
        self.graph_launches += g.launches
        n = self.last_num_wanted
        if n == 0:
            return StepResult(None, None)
        return StepResult(g.logits[:n], g.tokens[:n] if sample else None)

    def check_device_errors(self) -> None:
        """Raise if a kernel flagged bad input (a token id outside the vocabulary) or gave up a bounded wait."""
        flags = self.error_flag.tolist()
        if any(flags):
            self.error_flag.zero_()
            ops.reset_stream_work_buffers()
            raise RuntimeError(f"a kernel reported an error: flags {flags} "
                               "(flag 0: token id outside the vocabulary; flag 1: a bounded wait ran out: a tensor-map load that "
                               "did not land, or a neighbouring block's sums that did not come)")
