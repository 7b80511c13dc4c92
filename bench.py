#!/usr/bin/env python3
"""Decode and prefill throughput of mini_engine_b200 at the Qwen3-0.6B layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens a second at batch 8 (prompts of 1,024 random
token ids, engine context 4,096), timed on the device with CUDA events around exactly K decode
steps after W warm-up steps; every step reads all weights (1.19 GB, larger than the 126 MB L2) so
no L2 flush is needed.  ``e2e`` is the same through ``LLM.step()``: host token ids in (one pinned
host-to-device copy a step) and drawn token ids out (one device-to-host copy a step).  ``prefill``
is one 2,048-token prompt in one step; ``points`` holds decode at batch 1 and 64; ``roofline``
relates the decode step to the bytes it must read.  The reference (ankur110/mini_engine) cannot
be installed offline (it has neither setup.py nor pyproject.toml), so ``--impl reference`` prints
an ``unavailable`` line.  The engine runs on one GPU: for ``--gpus N`` with N > 1 one line says so
and the exit code is 2.

The options of the reference's own bench.py (bench.py:8-19 there) that apply to this engine are
kept for its workload: ``--mode offline --num-seqs 256 --budget 16384 --chunked 1 --threshold 0
--out results/bench.jsonl --label x --expect-gpu B200`` runs 256 random requests through
``LLM.generate`` and appends a JSON row like the reference's.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_0_6B = {   # layer sizes of the Qwen3-0.6B shape
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 1024, "num_hidden_layers": 28,
    "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960, "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16",
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--mode", choices=["step", "offline"], default="step")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--prompt-len", type=int, default=1024)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                   help="run one part only (small runs for profilers); the JSON line then holds that part")
    p.add_argument("--no-graphs", action="store_true", help="run decode steps eagerly instead of replaying CUDA graphs")
    p.add_argument("--no-pdl", action="store_true", help="launch kernels without programmatic dependent launch")
    p.add_argument("--seed", type=int, default=0)
    # the reference's own options (its bench.py:8-19), used by --mode offline
    p.add_argument("--model", default="", help="model folder; empty: random weights of the 0.6B shape")
    p.add_argument("--num-seqs", type=int, default=256)
    p.add_argument("--out", default="results/bench.jsonl")
    p.add_argument("--label", default="")
    p.add_argument("--chunked", type=int, default=1)
    p.add_argument("--budget", type=int, default=16384)
    p.add_argument("--threshold", type=int, default=0)
    p.add_argument("--expect-gpu", default="")
    return p.parse_args()


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out = dict(FALLBACK_PEAKS, source="measured")
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(raw.get(k), (int, float)) and raw[k] > 0:
                    out[k] = float(raw[k])
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


def model_folder(cfg: dict, seed: int) -> str:
    """A folder with random weights of the configuration, made once per machine under the temp dir."""
    from mini_engine_b200.weights import write_random_model
    key = hashlib.sha256(json.dumps([cfg, seed], sort_keys=True).encode()).hexdigest()[:16]
    folder = os.path.join(tempfile.gettempdir(), f"mini_engine_b200_bench_{os.getuid()}", key)
    if not os.path.isfile(os.path.join(folder, "done")):
        t = time.time()
        write_random_model(folder, cfg, seed)
        with open(os.path.join(folder, "done"), "w") as f:
            f.write("ok")
        print(f"[bench] wrote random weights to {folder} in {time.time() - t:.0f} s", file=sys.stderr)
    return folder


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while a timed region runs (read only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int = 0, period: float = 0.05):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:                                       # no NVML: the line says so
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def random_prompts(n: int, length: int, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, min(vocab, 10000), (length,), generator=g).tolist() for _ in range(n)]


def weight_bytes_per_step(cfg: dict, layers: int, itemsize: int) -> int:
    """Every weight a decode step uses, once: the layers' matrices and norms, the final norm and the head."""
    H, nh, nkv, hd, I, V = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                             "head_dim", "intermediate_size", "vocab_size"))
    per_layer = ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I) * itemsize + (2 * H + 2 * hd) * 4
    return layers * per_layer + V * H * itemsize + H * 4


def kv_bytes_per_token(cfg: dict, layers: int, itemsize: int) -> int:
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * itemsize


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    H, nh, nkv, hd, I, V = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                             "head_dim", "intermediate_size", "vocab_size"))
    linear = 2.0 * T * layers * ((nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I)
    attention = layers * 2.0 * nh * hd * T * T            # QK^T and PV over the causal half
    return linear + attention + 2.0 * V * H


def decode_on_device(runner, cache, prompts, steps: int, warmup: int):
    """W + K decode steps of a batch timed with CUDA events; the context grows by one token a step."""
    import torch
    from mini_engine_b200 import ops
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import StepItem
    holders = []
    for p in prompts:
        h = CacheHolder()
        assert cache.allocate(h, len(p) + steps + warmup + 1), "cache pool too small for the benchmark"
        holders.append(h)
    budget = runner.max_num_batched_tokens
    for h, p in zip(holders, prompts):                          # prefill in portions under the budget
        for a in range(0, len(p), budget):
            runner.step([StepItem(h, p[a:a + budget], a, [])])
    pos = [len(p) for p in prompts]
    tok = [7 + i for i in range(len(prompts))]

    def one():
        items = [StepItem(h, [tok[i]], pos[i], [0], (0.6, i)) for i, h in enumerate(holders)]
        runner.step(items, sample=True)
        for i in range(len(pos)):
            pos[i] += 1
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    l0, g0 = ops.launches, runner.graph_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx0 = pos[0]
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = (ops.launches - l0) + (runner.graph_launches - g0)
    for h in holders:
        cache.free(h)
    return ms / steps, launches, (ctx0 + pos[0]) / 2.0


def decode_e2e(llm, prompts, steps: int, warmup: int):
    """K decode steps through ``LLM.step()``: pinned host-to-device metadata in, drawn ids out, every step."""
    import torch
    from mini_engine_b200 import SamplingParams
    sp = SamplingParams(temperature=0.6, max_tokens=steps + warmup + 8, ignore_eos=True)
    for p in prompts:
        llm.add_request(p, sp)
    while any(s.num_uncomputed_tokens > 1 for s in llm.scheduler.running) or llm.scheduler.waiting:
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    h0, d0 = llm.h2d_bytes, llm.d2h_bytes
    t0 = time.perf_counter()
    n = 0
    for _ in range(steps):
        _, _, n_dec, emitted = llm.step()
        n += len(emitted)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d, d2h = (llm.h2d_bytes - h0) // steps, (llm.d2h_bytes - d0) // steps
    while not llm.is_finished():
        llm.step()
    return n / dt, h2d, d2h


def prefill_on_device(runner, cache, prompt, reps: int, warmup: int):
    import torch
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import StepItem
    h = CacheHolder()
    assert cache.allocate(h, len(prompt))
    item = [StepItem(h, prompt, 0, [len(prompt) - 1])]
    for _ in range(max(warmup, 2)):          # the engine captures a graph when a shape comes the second time: not in the timed part
        runner.step(item)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        runner.step(item)
    e1.record()
    torch.cuda.synchronize()
    cache.free(h)
    return e0.elapsed_time(e1) / reps


def run_step_mode(args) -> int:
    import torch
    from mini_engine_b200 import LLM, ops
    if args.no_pdl:
        ops.set_programmatic_launch(False)
    cfg = dict(QWEN3_0_6B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    folder = args.model or model_folder(cfg, args.seed)
    pk = peaks()
    itemsize = 2 if args.dtype in ("bfloat16", "bf16") else 4
    pages = (max(64, args.batch) * (args.prompt_len + args.steps + args.warmup + 64) + 4096) // 16 + 64
    llm = LLM(folder, dtype=args.dtype, kvcache_block_size=16, num_kvcache_blocks=pages, max_num_seqs=max(64, args.batch),
              max_num_batched_tokens=2048, max_model_len=args.context, enable_prefix_caching=False, seed=args.seed,
              use_cuda_graphs=not args.no_graphs)
    runner, cache = llm.model_runner, llm.cache
    vocab = cfg["vocab_size"]
    prompts = random_prompts(max(64, args.batch), args.prompt_len, vocab, args.seed + 1)

    T = 2048
    if args.only == "prefill":
        ms_prefill = prefill_on_device(runner, cache, random_prompts(1, T, vocab, args.seed + 2)[0], reps=args.steps, warmup=args.warmup)
        print(json.dumps({"only": "prefill", "tokens": T, "ms": round(ms_prefill, 4), "value": round(T * 1000.0 / ms_prefill, 1),
                          "frac": round(prefill_flops(cfg, layers, T) / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0
    with ClockSampler() as clocks:
        ms_step, launches, mean_ctx = decode_on_device(runner, cache, prompts[:args.batch], args.steps, args.warmup)
    if args.only == "decode":
        b = weight_bytes_per_step(cfg, layers, itemsize) + args.batch * mean_ctx * kv_bytes_per_token(cfg, layers, itemsize)
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(ms_step, 4),
                          "value": round(args.batch * 1000.0 / ms_step, 1), "gpu_launches": int(launches),
                          "hbm_frac": round(b / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}))
        return 0
    value = args.batch * 1000.0 / ms_step
    points = {}
    for b, k in ((1, max(20, args.steps // 2)), (64, max(20, args.steps // 4))):
        ms_b, _, _ = decode_on_device(runner, cache, prompts[:b], k, max(3, args.warmup))
        points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
    e2e_value, h2d, d2h = decode_e2e(llm, prompts[:args.batch], args.steps, max(3, args.warmup))
    ms_prefill = prefill_on_device(runner, cache, random_prompts(1, T, vocab, args.seed + 2)[0], reps=5, warmup=3)
    flops = prefill_flops(cfg, layers, T)
    bytes_step = weight_bytes_per_step(cfg, layers, itemsize) + args.batch * mean_ctx * kv_bytes_per_token(cfg, layers, itemsize)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s @ batch 8 (Qwen3-0.6B shape, 1,024-token prompts)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if itemsize == 2 else "fp32", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen3-0.6B shape, random weights N(0,0.02)", "layers": layers, "layers_of_config": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
                   "tied_embeddings": cfg["tie_word_embeddings"], "global_batch": args.batch,
                   "prompt_len": args.prompt_len, "seq_len": args.context, "kv_block": 16, "parallelism": "1 gpu",
                   "cuda_graphs": bool(runner.use_cuda_graphs),
                   "l2": "every step reads all weights (1.19 GB > 126 MB L2); no flush"},
        "clocks": clocks.summary(),
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(T * 1000.0 / ms_prefill, 1), "tokens": T, "ms": round(ms_prefill, 4),
                    "frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def run_offline_mode(args) -> int:
    """The reference's own workload (its bench.py:38-66): N random requests at once through generate()."""
    import subprocess
    from datetime import datetime
    from random import randint, seed
    import torch
    from mini_engine_b200 import LLM, SamplingParams
    gpu = subprocess.run(["nvidia-smi", "--query-gpu=name", "--format=csv,noheader"], capture_output=True,
                         text=True).stdout.strip().splitlines()[0]
    assert args.expect_gpu in gpu, f"wrong GPU: got {gpu}, expected *{args.expect_gpu}*"
    seed(0)
    N = args.num_seqs
    prompts = [[randint(0, 10000) for _ in range(randint(100, 1024))] for _ in range(N)]
    max_tokens = [randint(100, 1024) for _ in range(N)]
    folder = args.model or model_folder(dict(QWEN3_0_6B), args.seed)
    llm = LLM(folder, max_num_seqs=256, max_model_len=2048, max_num_batched_tokens=args.budget,
              enable_chunked_prefill=bool(args.chunked), long_prefill_token_threshold=args.threshold, dtype=args.dtype)
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=m) for m in max_tokens]
    llm.generate([[1, 2, 3]], SamplingParams(), use_tqdm=False)
    t = time.time()
    llm.generate(prompts, sps, use_tqdm=False)
    t = time.time() - t
    total = sum(max_tokens)
    row = {"engine": "mini_engine_b200", "label": args.label, "gpu": gpu, "torch": torch.__version__, "num_seqs": N,
           "input_tokens": sum(len(x) for x in prompts), "output_tokens": total, "time_s": round(t, 2),
           "throughput_tok_s": round(total / t, 1), "chunked": bool(args.chunked), "budget": args.budget,
           "threshold": args.threshold, "preemptions": llm.scheduler.num_preemptions,
           "time": datetime.now().isoformat(timespec="seconds")}
    print(json.dumps(row))
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    with open(args.out, "a") as f:
        f.write(json.dumps(row) + "\n")
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "ankur110/mini_engine has neither setup.py nor pyproject.toml: "
                          "pip cannot install it offline ('Directory is not installable')"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: mini_engine_b200 is a one-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    return run_offline_mode(args) if args.mode == "offline" else run_step_mode(args)


if __name__ == "__main__":
    sys.exit(main())
