"""Trace replay: given token ids, step by step, logits out; nothing is sampled.

The program behind ``bin/trace_run``.  It owns no model code: it builds the same
``ModelRunner`` that generation uses, holds each request's pages through the same cache
manager, and calls the same ``step``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional

import numpy as np

from ..cache.manager import CacheHolder
from ..config.registry import load_model_config


class TraceReplayer:
    """Feeds steps ``{"step", "entries": [{"id", "tokens", "want"}], "end"}`` to a model runner.

    ``prefix_caching``: a request that appears for the first time takes the leading full pages of its first portion
    from the cache when an earlier request left them there (looked up and hashed as the scheduler does it,
    engine/scheduler.py:120-131 and engine/block_manager.py:68-113 in the reference), and only the rest of the portion
    is run.  Pages are never taken for a place whose logits are wanted, nor for the portion's last token.
    ``poison`` (a debugging aid): the whole pool starts as NaN, a page is filled with NaN when it is handed out for
    new content and when its last holder lets go of it while nothing can find it again, so that any read of a key
    or value that this request did not write shows in the logits."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, prefix_caching: bool = False,
                 poison: bool = False, **runner_args):
        from .model_runner import ModelRunner
        unit = max(64, page_size)
        held = (max_tokens + unit - 1) // unit * unit
        num_pages = max(1, (held + page_size - 1) // page_size)
        cfg = load_model_config(model_dir)
        args = dict(max_num_seqs=8, max_num_batched_tokens=4096, max_model_len=cfg.max_position_embeddings)
        args.update(runner_args)
        self.runner = ModelRunner(model_dir, dtype=dtype, page_size=page_size, num_pages=num_pages,
                                  model_config=cfg, **args)
        self.cache = self.runner.make_cache_manager(enable_prefix_caching=prefix_caching)
        self.live: dict[str, CacheHolder] = {}
        self.poison = poison
        if poison:
            for pool in self.runner.kv_pools:
                pool.fill_(float("nan"))

    def _poison(self, group: int, pages) -> None:
        pages = [p for p in pages if p >= 0]
        if self.poison and pages:
            self.runner.kv_pools[group][:, pages] = float("nan")

    def _let_go(self, holder: CacheHolder, release) -> None:
        """Run ``release`` (which gives pages of ``holder`` back) and poison the pages that nobody holds or can find."""
        before = [list(t) for t in holder.block_tables]
        release()
        for g, (pool, pages) in enumerate(zip(self.cache.pools, before)):
            self._poison(g, [p for p in pages if p >= 0 and pool.ref_count[p] == 0 and pool.page_hash[p] == -1])

    def run_step(self, rec: dict) -> Optional[np.ndarray]:
        """Runs one step; returns the logits at the wanted places ([wanted, vocab] float32) or None."""
        from .model_runner import StepItem
        items, n_want = [], 0
        ps = self.cache.page_size
        for e in rec.get("entries", []):
            rid, toks = str(e["id"]), [int(t) for t in e["tokens"]]
            if not toks:
                continue
            want = [int(w) for w in e.get("want", [])]
            h = self.live.get(rid)
            hits, skip = None, 0
            if h is None:
                h = self.live[rid] = CacheHolder()
                h.tokens = []
                if self.cache.prefix_caching:
                    hits = self.cache.find_prefix_hit(toks)
                    keep = min([len(hits[0])] + [w // ps for w in want]) if hits else 0
                    hits = [pages[:keep] for pages in hits]
                    skip = keep * ps
            had = [len(t) for t in h.block_tables] or [0] * len(self.cache.pools)
            if not self.cache.allocate(h, len(toks) - skip, hits if skip else None):
                raise RuntimeError(f"step {rec.get('step')}: no pages left for request {rid!r} (free pages per "
                                   f"group: {self.cache.num_free_pages}); raise --max-tokens")
            for g, table in enumerate(h.block_tables):
                self._poison(g, table[had[g] + (skip // ps):])          # pages handed out for new content
            h.tokens += toks
            n_want += len(want)
            items.append(StepItem(h, toks[skip:], h.num_computed_tokens, [w - skip for w in want]))
        logits = self.runner.step(items).logits if items else None
        out = logits.cpu().numpy().astype("<f4", copy=True) if n_want else None
        for it in items:
            h = it.holder
            h.num_computed_tokens += len(it.tokens)
            self.cache.hash_full_pages(h, h.tokens)
            self._let_go(h, lambda h=h: self.cache.release_behind_window(h))
        self.runner.check_device_errors()
        for rid in rec.get("end", []):
            h = self.live.pop(str(rid), None)
            if h is not None:
                self._let_go(h, lambda h=h: self.cache.free(h))
        return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--prefix-caching", action="store_true",
                    help="a new request takes leading pages that an earlier request left in the cache (off: every "
                         "step runs exactly the tokens it brings)")
    ap.add_argument("--poison", action="store_true", help="debugging: unowned pages of the cache hold NaN")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    replayer = TraceReplayer(args.model, args.dtype, args.max_tokens, args.page_size,
                             prefix_caching=args.prefix_caching, poison=args.poison)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        logits = replayer.run_step(rec)
        if logits is not None:
            logits.tofile(os.path.join(args.out, f"{rec['step']}.f32"))
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
