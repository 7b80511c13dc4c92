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

import numpy as np

from ..cache.manager import CacheHolder
from ..config.registry import load_model_config


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

    from .model_runner import ModelRunner, StepItem
    page = args.page_size
    unit = max(64, page)
    num_pages = max(1, ((args.max_tokens + unit - 1) // unit * unit + page - 1) // page)
    cfg = load_model_config(args.model)
    runner = ModelRunner(args.model, dtype=args.dtype, page_size=page, num_pages=num_pages,
                         max_num_seqs=8, max_num_batched_tokens=4096,
                         max_model_len=cfg.max_position_embeddings, model_config=cfg)
    cache = runner.make_cache_manager(enable_prefix_caching=False)
    live: dict[str, CacheHolder] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        items, n_want = [], 0
        for e in rec.get("entries", []):
            rid, toks = str(e["id"]), [int(t) for t in e["tokens"]]
            if not toks:
                continue
            h = live.get(rid)
            if h is None:
                h = live[rid] = CacheHolder()
            if not cache.allocate(h, len(toks)):
                raise RuntimeError(f"step {step}: no pages left for request {rid!r} "
                                   f"(free pages per group: {cache.num_free_pages}); raise --max-tokens")
            want = [int(w) for w in e.get("want", [])]
            n_want += len(want)
            items.append(StepItem(h, toks, h.num_computed_tokens, want))
        logits = runner.step(items) if items else None
        if n_want:
            arr = logits.cpu().numpy().astype("<f4", copy=False)
            arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for it in items:
            it.holder.num_computed_tokens += len(it.tokens)
            cache.release_behind_window(it.holder)
        runner.check_device_errors()
        for rid in rec.get("end", []):
            h = live.pop(str(rid), None)
            if h is not None:
                cache.free(h)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
