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
    """Feeds steps ``{"step", "entries": [{"id", "tokens", "want"}], "end"}`` to a model runner."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, **runner_args):
        from .model_runner import ModelRunner
        unit = max(64, page_size)
        held = (max_tokens + unit - 1) // unit * unit
        num_pages = max(1, (held + page_size - 1) // page_size)
        cfg = load_model_config(model_dir)
        args = dict(max_num_seqs=8, max_num_batched_tokens=4096, max_model_len=cfg.max_position_embeddings)
        args.update(runner_args)
        self.runner = ModelRunner(model_dir, dtype=dtype, page_size=page_size, num_pages=num_pages,
                                  model_config=cfg, **args)
        self.cache = self.runner.make_cache_manager(enable_prefix_caching=False)
        self.live: dict[str, CacheHolder] = {}

    def run_step(self, rec: dict) -> Optional[np.ndarray]:
        """Runs one step; returns the logits at the wanted places ([wanted, vocab] float32) or None."""
        from .model_runner import StepItem
        items, n_want = [], 0
        for e in rec.get("entries", []):
            rid, toks = str(e["id"]), [int(t) for t in e["tokens"]]
            if not toks:
                continue
            h = self.live.get(rid)
            if h is None:
                h = self.live[rid] = CacheHolder()
            if not self.cache.allocate(h, len(toks)):
                raise RuntimeError(f"step {rec.get('step')}: no pages left for request {rid!r} (free pages per "
                                   f"group: {self.cache.num_free_pages}); raise --max-tokens")
            want = [int(w) for w in e.get("want", [])]
            n_want += len(want)
            items.append(StepItem(h, toks, h.num_computed_tokens, want))
        logits = self.runner.step(items).logits if items else None
        out = logits.cpu().numpy().astype("<f4", copy=True) if n_want else None
        for it in items:
            it.holder.num_computed_tokens += len(it.tokens)
            self.cache.release_behind_window(it.holder)
        self.runner.check_device_errors()
        for rid in rec.get("end", []):
            h = self.live.pop(str(rid), None)
            if h is not None:
                self.cache.free(h)
        return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    replayer = TraceReplayer(args.model, args.dtype, args.max_tokens, args.page_size)
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
