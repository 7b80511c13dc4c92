#!/usr/bin/env python3
"""The reference arm of bench.py: ankur110/mini_engine, unmodified, through its own ``LLM`` on the same workload.

Run as a child process by ``bench.py --impl reference``.  Nothing of mini_engine_b200 is imported here: the
process puts the reference tree (a plain copy of its folders, ``baseline/_ref``) first on ``sys.path`` and drives
its stock path, ``LLM(folder, ...)``, ``add_request`` and ``step()`` (engine/llm_engine.py:13-36 there).  The
reference is a set of top-level packages that run from their folder, not an installable distribution, so the
"install" is that copy.  Its CUDA extension is built by its own ``layers/ops.py`` at import; that file pins the
architecture with ``os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "8.0")`` (layers/ops.py:6), so setting the
variable before the import builds the same sources for this GPU.

The model folder is given by the caller: ``config.json`` and ``model.safetensors`` (random weights) plus the two
input files the reference's constructor asks for, ``"model_type": "qwen3"`` for ``AutoConfig`` and a word-level
``tokenizer.json`` (engine/llm_engine.py:18-19 only loads it and reads ``eos_token_id``).

Prints one JSON object: decode tokens a second at the given batch (device time between two CUDA events around K
``step()`` calls, and the same by wall clock), decode at batch 1 and 64, and one 2,048-token prompt.
"""
import argparse
import json
import os
import sys
import time


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="the reference tree")
    ap.add_argument("--model", required=True)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--vocab", type=int, default=10000)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--points", default="1,64")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    args = ap.parse_args()

    os.environ["TORCH_CUDA_ARCH_LIST"] = os.environ.get("MINI_ENGINE_REF_ARCH", "10.0")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    ref = os.path.abspath(args.ref)
    sys.path.insert(0, ref)
    os.chdir(ref)
    real_stdout = sys.stdout
    sys.stdout = sys.stderr                     # the reference prints while it builds and sizes its pool
    import torch
    from llm import LLM                          # the reference's (llm.py:1-4)
    from sampling_params import SamplingParams

    max_seqs = max([args.batch] + [int(x) for x in args.points.split(",") if x])
    budget = max(2048, args.prefill_tokens)
    llm = LLM(args.model, max_num_seqs=max_seqs, max_model_len=args.context, max_num_batched_tokens=budget)
    g = torch.Generator().manual_seed(args.seed + 1)

    def prompts(n, length):
        return [torch.randint(0, args.vocab, (length,), generator=g).tolist() for _ in range(n)]

    def decode(batch, steps, warmup):
        # requests whose prompt is done decode while the others' prompts are still computed: room for those tokens too
        ahead = batch * args.prompt_len // budget + batch
        sp = SamplingParams(temperature=0.6, max_tokens=steps + warmup + 8 + ahead, ignore_eos=True)
        for p in prompts(batch, args.prompt_len):
            llm.add_request(p, sp)
        sched = llm.scheduler
        while sched.waiting or any(s.num_uncomputed_tokens > 1 for s in sched.running):
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        n = 0
        for _ in range(steps):
            _, _, _, emitted = llm.step()
            n += len(emitted)
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1)
        while not llm.is_finished():
            llm.step()
        assert n == batch * steps, (n, batch, steps)
        return n / (ms * 1e-3), n / wall, ms / steps

    def prefill(tokens, reps, warmup):
        times = []
        for k in range(reps + warmup):
            (p,) = prompts(1, tokens)            # another prompt every time: the reference reuses cached prefixes
            llm.add_request(p, SamplingParams(temperature=0.6, max_tokens=1, ignore_eos=True))
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            llm.step()
            e1.record()
            torch.cuda.synchronize()
            assert llm.is_finished()
            if k >= warmup:
                times.append(e0.elapsed_time(e1))
        return sum(times) / len(times)

    value, e2e, ms_step = decode(args.batch, args.steps, args.warmup)
    points = {}
    for b in [int(x) for x in args.points.split(",") if x]:
        v, _, _ = decode(b, max(10, args.steps // 2), max(3, args.warmup))
        points[f"decode_b{b}"] = round(v, 1)
    ms_prefill = prefill(args.prefill_tokens, 5, 3) if args.prefill_tokens else None
    out = {"value": round(value, 1), "e2e": round(e2e, 1), "ms_per_step": round(ms_step, 4), "points": points,
           "prefill_ms": None if ms_prefill is None else round(ms_prefill, 4),
           "num_kvcache_blocks": llm.scheduler.block_manager.blocks.__len__(),
           "preemptions": llm.scheduler.num_preemptions, "torch": torch.__version__,
           "arch": os.environ["TORCH_CUDA_ARCH_LIST"]}
    real_stdout.write(json.dumps(out) + "\n")
    real_stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
