#!/usr/bin/env python3
"""Decode and prefill throughput of mini_engine_b200 at the Qwen3 layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 0.6b|8b|32b] [--mode ...]

With no options it prints ONE JSON line for the Qwen3-0.6B shape.  ``value`` is decoded tokens a second at
batch 8 (prompts of 1,024 random token ids, engine context 4,096), timed on the device with CUDA events around
exactly K decode steps after W warm-up steps; every step reads all weights (1.19 GB, larger than the 126 MB L2)
so no L2 flush is needed.  ``e2e`` is the same through ``LLM.step()``: host token ids in (one pinned
host-to-device copy a step) and drawn token ids out (one device-to-host copy a step).  ``prefill`` is one
2,048-token prompt in one step; ``roofline`` relates the decode step to the bytes it must read; ``kernels``
gives, for each kind of kernel of one decode step and one prefill step run kernel by kernel between CUDA events,
its mean time, its bytes or flops and the fraction of the measured peak.  ``points`` holds decode at batch 1 and
64, the reference's offline workload (256 random requests through ``LLM.generate``), and the two larger shapes:
the 8B shape's mixed workload (64 random requests, prompts of 100 to 2,048 tokens, 100 to 512 tokens out, token
budget 8,192, through ``LLM.generate``), the 8B and 32B shapes' decode at batch 1, 8 and 64 after 2,048-token
prompts, each with its fraction of the memory roofline, and prompts of 8,192 and 16,384 tokens in portions of 2,048.  ``--extras 0`` leaves the offline workload and the
larger shapes out.

Every size comes from the configuration that is loaded: ``--shape`` picks one of the three built-in ones (its
weights are drawn at random: written to a folder for 0.6b, drawn on the device for 8b and 32b), ``--model DIR``
loads a folder, and the bytes and flops of the roofline figures are computed from that configuration.

``--impl reference`` runs ankur110/mini_engine itself, unmodified, on the same workload in a child process
(``baseline/run_reference.py``) and prints the same line with ``"impl": "reference"``.  The engine runs on one
GPU: for ``--gpus N`` with N > 1 one line says so and the exit code is 2.

Modes: ``step`` (the line above), ``offline`` (the reference's own bench.py:38-66 with its options ``--num-seqs
--budget --chunked --threshold --out --label --expect-gpu``; a JSON row like the reference's is appended to
``--out``), ``mixed`` (the 8B workload above, at any shape), ``decode`` (decode at batches ``--batches`` after
``--prompt-len`` prompts), ``prefill`` (one prompt of ``--prompt-len`` tokens in portions of ``--budget``).
"""
from __future__ import annotations

import argparse
import gc
import hashlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _qwen3(layers, hidden, heads, kv_heads, inter, tied, **kw):
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": hidden, "num_hidden_layers": layers,
           "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128, "intermediate_size": inter,
           "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": tied,
           "max_position_embeddings": 40960, "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"}
    cfg.update(kw)
    return cfg


SHAPES = {   # layer sizes of the Qwen3 dense models
    "0.6b": _qwen3(28, 1024, 16, 8, 3072, True),
    "8b": _qwen3(36, 4096, 32, 8, 12288, False),
    "32b": _qwen3(64, 5120, 64, 8, 25600, False),
}
SHAPE_NAMES = {"0.6b": "Qwen3-0.6B", "8b": "Qwen3-8B", "32b": "Qwen3-32B"}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--mode", choices=["step", "offline", "mixed", "decode", "prefill"], default="step")
    p.add_argument("--shape", choices=sorted(SHAPES), default="0.6b", help="layer sizes, when no --model is given")
    p.add_argument("--extras", type=int, default=1,
                   help="step mode: also run the offline workload, the 8B mixed workload and the 32B decode points")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--batches", default="1,8,64", help="decode mode: the batch sizes")
    p.add_argument("--prompt-len", type=int, default=0, help="0: 1,024 (2,048 for the 32B decode points and prefill mode)")
    p.add_argument("--context", type=int, default=0, help="engine context length; 0: 4,096 (8,192 for 8b and 32b)")
    p.add_argument("--page-size", type=int, default=16, help="tokens a page of the cache")
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                   help="step mode: run one part only (small runs for profilers); the JSON line then holds that part")
    p.add_argument("--no-graphs", action="store_true", help="run decode steps eagerly instead of replaying CUDA graphs")
    p.add_argument("--no-pdl", action="store_true", help="launch kernels without programmatic dependent launch")
    p.add_argument("--no-kernels", action="store_true", help="step mode: leave the per-kernel table out")
    p.add_argument("--seed", type=int, default=0)
    # the reference's own options (its bench.py:8-19), used by --mode offline (and --budget by mixed / prefill)
    p.add_argument("--model", default="", help="model folder; empty: random weights of --shape")
    p.add_argument("--num-seqs", type=int, default=0, help="requests of the offline (256) and mixed (64) workloads")
    p.add_argument("--out", default="results/bench.jsonl")
    p.add_argument("--label", default="")
    p.add_argument("--chunked", type=int, default=1)
    p.add_argument("--budget", type=int, default=0, help="token budget of a step; 0: 16,384 offline, 8,192 mixed, 2,048 else")
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


# ---- models ----------------------------------------------------------------------------------------------------
def _bench_dir() -> str:
    return os.path.join(tempfile.gettempdir(), f"mini_engine_b200_bench_{os.getuid()}")


def model_folder(cfg: dict, seed: int, weights: bool = True) -> str:
    """A folder with the configuration and, with ``weights``, random weights of it; made once per machine under
    the temp dir."""
    from mini_engine_b200.weights import write_random_model
    key = hashlib.sha256(json.dumps([cfg, seed, weights], sort_keys=True).encode()).hexdigest()[:16]
    folder = os.path.join(_bench_dir(), key)
    if not os.path.isfile(os.path.join(folder, "done")):
        t = time.time()
        os.makedirs(folder, exist_ok=True)
        if weights:
            write_random_model(folder, cfg, seed)
        else:
            with open(os.path.join(folder, "config.json"), "w") as f:
                json.dump(cfg, f, indent=1)
        with open(os.path.join(folder, "done"), "w") as f:
            f.write("ok")
        if weights:
            print(f"[bench] wrote random weights to {folder} in {time.time() - t:.0f} s", file=sys.stderr)
    return folder


class Model:
    """What a run loads: the folder, its configuration as a dict, and how the engine gets the weights."""

    def __init__(self, args, shape: str = ""):
        from_folder = bool(args.model) and not shape
        shape = shape or args.shape
        if from_folder:
            self.folder = os.path.expanduser(args.model)
            with open(os.path.join(self.folder, "config.json")) as f:
                self.cfg = json.load(f)
            self.name = os.path.basename(os.path.normpath(self.folder))
            self.engine_args = {}
        else:
            self.cfg = dict(SHAPES[shape])
            self.name = f"{SHAPE_NAMES[shape]} shape, random weights N(0,0.02)"
            on_device = shape != "0.6b"                      # 16 and 65 GB of files would take minutes to write and read
            if args.layers:
                self.cfg["num_hidden_layers"] = args.layers
            self.folder = model_folder(self.cfg, args.seed, weights=not on_device)
            self.engine_args = {"random_weights": True} if on_device else {}
        self.full_layers = self.cfg["num_hidden_layers"] if from_folder else SHAPES[shape]["num_hidden_layers"]
        self.layers = self.cfg["num_hidden_layers"]
        self.vocab = self.cfg["vocab_size"]
        self.default_context = 4096 if self.cfg["hidden_size"] <= 1024 else 8192


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


# ---- bytes and flops from the configuration ------------------------------------------------------------------------
def _sizes(cfg: dict):
    return (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                             "intermediate_size", "vocab_size"))


def product_shapes(cfg: dict) -> dict:
    """(rows of the weight, K) of the four products of a layer and of the head."""
    H, nh, nkv, hd, I, V = _sizes(cfg)
    return {"qkv": ((nh + 2 * nkv) * hd, H), "mixer_out": (H, nh * hd), "ffn_act": (2 * I, H), "ffn_out": (H, I),
            "logits": (V, H)}


def weight_bytes_per_step(cfg: dict, layers: int, itemsize: int) -> int:
    """Every weight a decode step uses, once: the layers' matrices and norms, the final norm and the head."""
    H, nh, nkv, hd, I, V = _sizes(cfg)
    shapes = product_shapes(cfg)
    per_layer = sum(n * k for name, (n, k) in shapes.items() if name != "logits") * itemsize + (2 * H + 2 * hd) * 4
    return layers * per_layer + V * H * itemsize + H * 4


def kv_bytes_per_token(cfg: dict, layers: int, itemsize: int) -> int:
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * itemsize


def prefill_flops(cfg: dict, layers: int, T: int, start: int = 0) -> float:
    """Flops of a step that computes tokens [start, start + T) of one prompt and the logits of its last token."""
    H, nh, nkv, hd, I, V = _sizes(cfg)
    linear = 2.0 * T * layers * sum(n * k for name, (n, k) in product_shapes(cfg).items() if name != "logits")
    attention = layers * 2.0 * nh * hd * (T * T + 2.0 * T * start)      # QK^T and PV over the keys each query sees
    return linear + attention + 2.0 * V * H


def decode_bytes(cfg: dict, layers: int, itemsize: int, batch: int, mean_ctx: float) -> float:
    return weight_bytes_per_step(cfg, layers, itemsize) + batch * mean_ctx * kv_bytes_per_token(cfg, layers, itemsize)


# ---- timed pieces ------------------------------------------------------------------------------------------------
def make_engine(model: Model, args, *, max_seqs: int, budget: int, context: int, pages: int = -1, **kw):
    from mini_engine_b200 import LLM
    opts = dict(dtype=args.dtype, kvcache_block_size=args.page_size, num_kvcache_blocks=pages, max_num_seqs=max_seqs,
                max_num_batched_tokens=budget, max_model_len=context, seed=args.seed, use_cuda_graphs=not args.no_graphs)
    opts.update(model.engine_args)
    opts.update(kw)
    return LLM(model.folder, **opts)


def release_memory() -> None:
    """After the caller has dropped its engine: give the device memory back before the next engine is built."""
    import torch
    from mini_engine_b200 import ops
    ops.forget_tensors()
    gc.collect()
    torch.cuda.empty_cache()


def prefill_requests(runner, cache, prompts, extra_tokens: int):
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import StepItem
    holders = []
    for p in prompts:
        h = CacheHolder()
        assert cache.allocate(h, len(p) + extra_tokens), "cache pool too small for the benchmark"
        holders.append(h)
    budget = runner.max_num_batched_tokens
    for h, p in zip(holders, prompts):                          # prefill in portions under the budget
        for a in range(0, len(p), budget):
            runner.step([StepItem(h, p[a:a + budget], a, [])])
    return holders


def decode_on_device(runner, cache, prompts, steps: int, warmup: int):
    """W + K decode steps of a batch timed with CUDA events; the context grows by one token a step."""
    import torch
    from mini_engine_b200 import ops
    from mini_engine_b200.engine.model_runner import StepItem
    holders = prefill_requests(runner, cache, prompts, steps + warmup + 1)
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
    runner.check_device_errors()
    return ms / steps, launches, (ctx0 + pos[0]) / 2.0


def decode_e2e(llm, prompts, steps: int, warmup: int):
    """K decode steps through ``LLM.step()``: pinned host-to-device metadata in, drawn ids out, every step."""
    import torch
    from mini_engine_b200 import SamplingParams
    # requests whose prompt is done decode while the others' prompts are still computed: room for those tokens too
    ahead = sum(len(p) for p in prompts) // llm.config.max_num_batched_tokens + len(prompts)
    sp = SamplingParams(temperature=0.6, max_tokens=steps + warmup + 8 + ahead, ignore_eos=True)
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


def prefill_on_device(runner, cache, prompt, reps: int, warmup: int, portion: int = 0):
    """One prompt, whole or in portions of ``portion`` tokens, ``reps`` times into the same pages; ms per prompt."""
    import torch
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import StepItem
    h = CacheHolder()
    assert cache.allocate(h, len(prompt))
    portion = portion or len(prompt)
    items = [[StepItem(h, prompt[a:a + portion], a, [len(prompt) - 1 - a] if a + portion >= len(prompt) else [])]
             for a in range(0, len(prompt), portion)]

    def once():
        for it in items:
            runner.step(it)
    for _ in range(max(warmup, 2)):          # the engine captures a graph when a shape comes the second time: not in the timed part
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        once()
    e1.record()
    torch.cuda.synchronize()
    cache.free(h)
    runner.check_device_errors()
    return e0.elapsed_time(e1) / reps


def kernel_table(model: Model, runner, cache, args, pk: dict, batch: int, prompt_len: int, T: int) -> dict:
    """One decode step of ``batch`` requests and one prefill step of ``T`` tokens launched kernel by kernel, every
    launch between two CUDA events: per kind of kernel the median microseconds of a launch (less what an empty event
    pair measures, ``event_pair_us``), the bytes (decode) or flops (prefill) it has to move or do, and the fraction
    of the measured peak that makes.  Kernels run one after the other here; in the step itself each starts under its
    predecessor, so these add up to more than the step."""
    import torch
    from mini_engine_b200 import ops
    from mini_engine_b200.cache.manager import CacheHolder
    from mini_engine_b200.engine.model_runner import StepItem
    cfg, L = model.cfg, model.layers
    item = 2 if args.dtype in ("bfloat16", "bf16") else 4
    H, nh, nkv, hd, I, V = _sizes(cfg)
    shapes = product_shapes(cfg)
    graphs, runner.use_cuda_graphs = runner.use_cuda_graphs, False

    def collect(run):
        run()                                           # once untimed: buffers, tensor maps
        torch.cuda.synchronize()
        ops.timeline = []
        try:
            # The host needs longer to issue a launch and its two events than the device to run a small kernel, and an
            # event pair around a kernel that the device is waiting for also times that wait.  So the device is kept
            # busy first, while the host queues the whole step; then it runs launch after launch with no gaps.
            busy = torch.empty(1 << 28, dtype=torch.float32, device="cuda")         # 1 GiB
            for _ in range(24):
                busy.add_(1.0)                           # some 8 ms of work ahead of the step
            gc.disable()                                 # (a collection in the middle of the queueing starves the device: one
            try:                                         # launch then "took" 72 ms)
                run()
            finally:
                gc.enable()
            torch.cuda.synchronize()
            del busy
            got = {}
            for tag, name, e0, e1 in ops.timeline:
                key = tag if name.startswith(("me_gemm", "library_mm")) else name[3:] if name.startswith("me_") else name
                got.setdefault(key, []).append(e0.elapsed_time(e1) * 1e3)
        finally:
            ops.timeline = None
        return got

    # What two events around NOTHING measure, in the same setting (device kept busy, commands queued): an event pair
    # costs the stream a few microseconds by itself, which is not the kernel's time.  It is taken off every figure.
    def event_overhead_us() -> float:
        busy = torch.empty(1 << 28, dtype=torch.float32, device="cuda")
        for _ in range(8):
            busy.add_(1.0)
        pairs = []
        for _ in range(200):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            e1.record()
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in pairs) * 1e3
    overhead = event_overhead_us()
    out = {"event_pair_us": round(overhead, 2)}
    # decode
    prompts = random_prompts(batch, prompt_len, model.vocab, args.seed + 3)
    holders = prefill_requests(runner, cache, prompts, 4)
    ctx = prompt_len + 1
    got = collect(lambda: runner.step([StepItem(h, [11 + i], prompt_len, [0], (0.6, i)) for i, h in enumerate(holders)],
                                      sample=True))
    for h in holders:
        cache.free(h)
    work = {name: n * k * item for name, (n, k) in shapes.items()}
    work["attn_decode_fused"] = work["attn_decode"] = batch * ctx * 2 * nkv * hd * item
    for key, us in sorted(got.items()):
        mean = max(statistics.median(us) - overhead, 0.1)
        row = {"us": round(mean, 2), "launches": len(us)}
        if key in work:
            row["bytes"] = int(work[key])
            row["frac"] = round(work[key] / (mean * 1e-6) / 1e9 / pk["hbm_gbs"], 4)
        out[f"decode_b{batch}.{key}"] = row
    # prefill
    (prompt,) = random_prompts(1, T, model.vocab, args.seed + 4)
    h = CacheHolder()
    assert cache.allocate(h, T)
    got = collect(lambda: runner.step([StepItem(h, prompt, 0, [T - 1])]))
    cache.free(h)
    flops = {name: 2.0 * T * n * k for name, (n, k) in shapes.items() if name != "logits"}
    flops["attn_prefill_tcgen05"] = flops["attn_prefill"] = flops["attn_chunk"] = 2.0 * nh * hd * T * T
    for key, us in sorted(got.items()):
        mean = max(statistics.median(us) - overhead, 0.1)
        row = {"us": round(mean, 2), "launches": len(us)}
        if key in flops:
            row["flops"] = flops[key]
            row["frac"] = round(flops[key] / (mean * 1e-6) / (pk["bf16_tflops"] * 1e12), 4)
        out[f"prefill_{T}.{key}"] = row
    runner.use_cuda_graphs = graphs
    return out


# ---- workloads through LLM.generate ----------------------------------------------------------------------------------
def generate_workload(model: Model, args, num_seqs: int, prompt_range, out_range, budget: int, max_model_len: int,
                      max_num_seqs: int) -> dict:
    """Seeded random requests, all at once, through ``LLM.generate``; output tokens over wall time, as the
    reference measures it (its bench.py:38-66)."""
    from random import randint, seed
    import torch
    from mini_engine_b200 import SamplingParams
    seed(0)
    prompts = [[randint(0, 10000) for _ in range(randint(*prompt_range))] for _ in range(num_seqs)]
    max_tokens = [randint(*out_range) for _ in range(num_seqs)]
    llm = make_engine(model, args, max_seqs=max_num_seqs, budget=budget, context=max_model_len,
                      enable_chunked_prefill=bool(args.chunked), long_prefill_token_threshold=args.threshold)
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=m) for m in max_tokens]
    llm.generate([[1, 2, 3]], SamplingParams(), use_tqdm=False)
    torch.cuda.synchronize()
    steps0 = llm.num_steps
    t = time.time()
    llm.generate(prompts, sps, use_tqdm=False)
    torch.cuda.synchronize()
    t = time.time() - t
    total = sum(max_tokens)
    row = {"num_seqs": num_seqs, "input_tokens": sum(len(x) for x in prompts), "output_tokens": total,
           "time_s": round(t, 2), "throughput_tok_s": round(total / t, 1), "steps": llm.num_steps - steps0,
           "chunked": bool(args.chunked), "budget": budget, "threshold": args.threshold,
           "preemptions": llm.scheduler.num_preemptions, "pages": llm.model_runner.num_pages}
    del llm
    release_memory()
    return row


def run_offline_mode(args) -> int:
    """The reference's own workload (its bench.py:38-66): N random requests at once through generate()."""
    from datetime import datetime
    import torch
    gpu = subprocess.run(["nvidia-smi", "--query-gpu=name", "--format=csv,noheader"], capture_output=True,
                         text=True).stdout.strip().splitlines()[0]
    assert args.expect_gpu in gpu, f"wrong GPU: got {gpu}, expected *{args.expect_gpu}*"
    model = Model(args)
    if args.mode == "offline":
        row = generate_workload(model, args, args.num_seqs or 256, (100, 1024), (100, 1024), args.budget or 16384, 2048, 256)
    else:
        row = generate_workload(model, args, args.num_seqs or 64, (100, 2048), (100, 512), args.budget or 8192,
                                args.context or model.default_context, 64)
    row = {"engine": "mini_engine_b200", "label": args.label, "gpu": gpu, "torch": torch.__version__, "model": model.name,
           "workload": args.mode, **row, "time": datetime.now().isoformat(timespec="seconds")}
    print(json.dumps(row))
    os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
    with open(args.out, "a") as f:
        f.write(json.dumps(row) + "\n")
    return 0


# ---- decode points and prefill of any shape ------------------------------------------------------------------------
def decode_points(model: Model, args, batches, prompt_len: int, steps: int, warmup: int, pk: dict) -> dict:
    """Decode at the given batch sizes after ``prompt_len``-token prompts: tokens a second and the fraction of the
    memory roofline."""
    item = 2 if args.dtype in ("bfloat16", "bf16") else 4
    context = args.context or model.default_context
    top = max(batches)
    pages = top * ((prompt_len + steps + warmup + 64) // 16 + 2) + 64
    llm = make_engine(model, args, max_seqs=max(top, 1), budget=max(2048, top), context=context, pages=pages,
                      enable_prefix_caching=False)
    prompts = random_prompts(top, prompt_len, model.vocab, args.seed + 1)
    out = {}
    for b in batches:
        k = max(10, steps // (4 if b >= 64 else 1))
        ms, _, mean_ctx = decode_on_device(llm.model_runner, llm.cache, prompts[:b], k, max(3, warmup))
        gbs = decode_bytes(model.cfg, model.layers, item, b, mean_ctx) / (ms * 1e-3) / 1e9
        out[b] = {"tok_s": round(b * 1000.0 / ms, 1), "ms_per_step": round(ms, 4), "hbm_frac": round(gbs / pk["hbm_gbs"], 4)}
    del llm
    release_memory()
    return out


def run_decode_mode(args) -> int:
    model, pk = Model(args), peaks()
    batches = [int(b) for b in args.batches.split(",") if b]
    prompt_len = args.prompt_len or (2048 if model.cfg["hidden_size"] > 1024 else 1024)
    pts = decode_points(model, args, batches, prompt_len, args.steps, args.warmup, pk)
    print(json.dumps({"mode": "decode", "model": model.name, "layers": model.layers, "layers_of_config": model.full_layers,
                      "prompt_len": prompt_len, "peaks": pk["source"],
                      "points": {f"decode_b{b}": v for b, v in pts.items()}}))
    return 0


def run_prefill_mode(args) -> int:
    model, pk = Model(args), peaks()
    T = args.prompt_len or 2048
    portion = min(args.budget or 2048, T)
    llm = make_engine(model, args, max_seqs=4, budget=portion, context=max(args.context or model.default_context, T + 16),
                      pages=T // 16 + 64, enable_prefix_caching=False)
    (prompt,) = random_prompts(1, T, model.vocab, args.seed + 2)
    ms = prefill_on_device(llm.model_runner, llm.cache, prompt, reps=max(3, min(args.steps, 10)), warmup=args.warmup, portion=portion)
    flops = sum(prefill_flops(model.cfg, model.layers, min(portion, T - a), a) for a in range(0, T, portion))
    print(json.dumps({"mode": "prefill", "model": model.name, "layers": model.layers, "tokens": T, "portion": portion,
                      "ms": round(ms, 4), "value": round(T * 1000.0 / ms, 1),
                      "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "peaks": pk["source"]}))
    return 0


# ---- the contract line -----------------------------------------------------------------------------------------------
def run_step_mode(args) -> int:
    from mini_engine_b200 import ops
    if args.no_pdl:
        ops.set_programmatic_launch(False)
    model, pk = Model(args), peaks()
    cfg, layers = model.cfg, model.layers
    itemsize = 2 if args.dtype in ("bfloat16", "bf16") else 4
    prompt_len = args.prompt_len or 1024
    context = args.context or model.default_context
    top = max(64, args.batch)
    pages = (top * (prompt_len + args.steps + args.warmup + 64) + 4096) // 16 + 64
    llm = make_engine(model, args, max_seqs=top, budget=2048, context=context, pages=pages, enable_prefix_caching=False)
    runner, cache = llm.model_runner, llm.cache
    vocab = model.vocab
    prompts = random_prompts(top, prompt_len, vocab, args.seed + 1)

    T = 2048
    if args.only == "prefill":
        ms_prefill = prefill_on_device(runner, cache, random_prompts(1, T, vocab, args.seed + 2)[0], reps=args.steps, warmup=args.warmup)
        print(json.dumps({"only": "prefill", "tokens": T, "ms": round(ms_prefill, 4), "value": round(T * 1000.0 / ms_prefill, 1),
                          "frac": round(prefill_flops(cfg, layers, T) / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0
    with ClockSampler() as clocks:
        ms_step, launches, mean_ctx = decode_on_device(runner, cache, prompts[:args.batch], args.steps, args.warmup)
    if args.only == "decode":
        b = decode_bytes(cfg, layers, itemsize, args.batch, mean_ctx)
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": round(ms_step, 4),
                          "value": round(args.batch * 1000.0 / ms_step, 1), "gpu_launches": int(launches),
                          "hbm_frac": round(b / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}))
        return 0
    value = args.batch * 1000.0 / ms_step
    points = {}
    for b, k in ((1, max(20, args.steps // 2)), (64, max(20, args.steps // 4))):
        ms_b, _, ctx_b = decode_on_device(runner, cache, prompts[:b], k, max(3, args.warmup))
        points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
        points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, layers, itemsize, b, ctx_b) / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    e2e_value, h2d, d2h = decode_e2e(llm, prompts[:args.batch], args.steps, max(3, args.warmup))
    ms_prefill = prefill_on_device(runner, cache, random_prompts(1, T, vocab, args.seed + 2)[0], reps=5, warmup=3)
    kernels = {} if args.no_kernels else kernel_table(model, runner, cache, args, pk, args.batch, prompt_len, T)
    flops = prefill_flops(cfg, layers, T)
    bytes_step = decode_bytes(cfg, layers, itemsize, args.batch, mean_ctx)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    wb = weight_bytes_per_step(cfg, layers, itemsize)
    del llm, runner, cache
    release_memory()
    if args.extras and not args.model:
        points.update(extra_points(args, pk))
    line = {
        "metric": f"decode tok/s @ batch {args.batch} ({model.name.split(',')[0]}, {prompt_len:,}-token prompts)",
        "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if itemsize == 2 else "fp32", "data": "synthetic", "impl": "ours",
        "config": {"model": model.name, "layers": layers, "layers_of_config": model.full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
                   "tied_embeddings": bool(cfg.get("tie_word_embeddings", False)), "global_batch": args.batch,
                   "prompt_len": prompt_len, "seq_len": context, "kv_block": 16, "parallelism": "1 gpu",
                   "cuda_graphs": not args.no_graphs,
                   "l2": f"every step reads all weights ({wb / 1e9:.2f} GB > 126 MB L2); no flush"},
        "clocks": clocks.summary(),
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(T * 1000.0 / ms_prefill, 1), "tokens": T, "ms": round(ms_prefill, 4),
                    "frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
        "kernels": kernels,
    }
    print(json.dumps(line))
    return 0


def extra_points(args, pk: dict) -> dict:
    """The workloads beyond the headline: the reference's offline workload at the 0.6B shape, the 8B shape's mixed
    workload and the 32B shape's decode points.  A part that fails says so in its place and the line still comes."""
    out = {}

    def attempt(name, fn):
        t = time.time()
        try:
            fn()
        except Exception as e:                      # the headline must not be lost to an extra
            out[name + "_error"] = f"{type(e).__name__}: {e}"[:300]
        print(f"[bench] {name}: {time.time() - t:.0f} s", file=sys.stderr)

    def offline():
        row = generate_workload(Model(args, "0.6b"), args, 256, (100, 1024), (100, 1024), 16384, 2048, 256)
        out["offline_tok_s"] = row["throughput_tok_s"]
        out["offline_time_s"] = row["time_s"]

    def mixed_8b():
        m = Model(args, "8b")
        row = generate_workload(m, args, 64, (100, 2048), (100, 512), 8192, 8192, 64)
        out["8b_mixed64_tok_s"] = row["throughput_tok_s"]
        out["8b_mixed64_time_s"] = row["time_s"]
        out["8b_mixed64_steps"] = row["steps"]
        out["8b_layers"] = m.layers

    def decode_32b():
        m = Model(args, "32b")
        pts = decode_points(m, args, [1, 8, 64], 2048, 20, 3, pk)
        for b, v in pts.items():
            out[f"32b_decode_b{b}"] = v["tok_s"]
            out[f"32b_decode_b{b}_hbm_frac"] = v["hbm_frac"]
        out["32b_layers"] = m.layers

    def long_prompts():
        # one prompt of 8,192 and of 16,384 tokens at the 0.6B shape, in portions of 2,048 (each portion attends to all before it)
        m = Model(args, "0.6b")
        llm = make_engine(m, args, max_seqs=4, budget=2048, context=16384 + 64, pages=16384 // 16 + 64, enable_prefix_caching=False)
        for T in (8192, 16384):
            (prompt,) = random_prompts(1, T, m.vocab, args.seed + 5)
            ms = prefill_on_device(llm.model_runner, llm.cache, prompt, reps=3, warmup=2, portion=2048)
            flops = sum(prefill_flops(m.cfg, m.layers, 2048, a) for a in range(0, T, 2048))
            out[f"prefill_{T}_tok_s"] = round(T * 1000.0 / ms, 1)
            out[f"prefill_{T}_frac"] = round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        del llm
        release_memory()

    def decode_8b():
        m = Model(args, "8b")
        pts = decode_points(m, args, [1, 8, 64], 2048, 20, 3, pk)
        for b, v in pts.items():
            out[f"8b_decode_b{b}"] = v["tok_s"]
            out[f"8b_decode_b{b}_hbm_frac"] = v["hbm_frac"]

    attempt("long_prompts", long_prompts)
    attempt("offline", offline)
    attempt("8b_mixed64", mixed_8b)
    attempt("8b_decode", decode_8b)
    attempt("32b_decode", decode_32b)
    return out


# ---- the reference arm ---------------------------------------------------------------------------------------------
def reference_model_folder(cfg: dict, seed: int) -> str:
    """The random-weights folder plus the input files that the reference's constructor reads: ``model_type`` in
    config.json (there already) for transformers' AutoConfig, and a word-level tokenizer over the vocabulary
    (the reference loads it and reads ``eos_token_id``, engine/llm_engine.py:18-19)."""
    folder = model_folder(cfg, seed)
    if not os.path.isfile(os.path.join(folder, "tokenizer.json")):
        from tokenizers import Tokenizer, models, pre_tokenizers
        V = cfg["vocab_size"]
        tok = Tokenizer(models.WordLevel({f"t{i}": i for i in range(V)}, unk_token="t0"))
        tok.pre_tokenizer = pre_tokenizers.Whitespace()
        tok.save(os.path.join(folder, "tokenizer.json"))
        with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
            json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": f"t{V - 1}", "unk_token": "t0"}, f)
    return folder


def run_reference(args) -> int:
    """ankur110/mini_engine, unmodified, on the headline workload: a child process that imports nothing of this
    package (baseline/run_reference.py)."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:600]}))
        return 0
    if args.gpus != 1:
        return unavailable("ankur110/mini_engine is a one-GPU engine (no distributed code)")
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref, "llm.py")):
        src = os.environ.get("MINI_ENGINE_REF", "")
        if src and os.path.isfile(os.path.join(src, "llm.py")):
            import shutil
            shutil.copytree(src, ref, dirs_exist_ok=True)
        else:
            return unavailable("the reference tree is not at baseline/_ref (copy ankur110/mini_engine there, or name it in $MINI_ENGINE_REF)")
    if args.shape != "0.6b" or args.model:
        return unavailable("the reference's kernels are compiled for head_dim 128, KV block 16 and 2 query heads per KV head "
                           "(csrc/paged_decode.cu:12-15): only the 0.6B shape fits")
    cfg = dict(SHAPES["0.6b"])
    try:
        folder = reference_model_folder(cfg, args.seed)
    except Exception as e:
        return unavailable(f"could not write the model folder: {type(e).__name__}: {e}")
    prompt_len, context = args.prompt_len or 1024, args.context or 4096
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "run_reference.py"), "--ref", ref, "--model", folder,
           "--batch", str(args.batch), "--prompt-len", str(prompt_len), "--context", str(context),
           "--steps", str(args.steps), "--warmup", str(args.warmup), "--seed", str(args.seed)]
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    with ClockSampler() as clocks:
        proc = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=1500)
    sys.stderr.write(proc.stderr[-4000:])
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    if proc.returncode != 0 or not lines:
        tail = [ln for ln in proc.stderr.strip().splitlines() if ln.strip()][-3:]
        return unavailable(f"the reference failed here (exit code {proc.returncode}): " + " | ".join(tail))
    r = json.loads(lines[-1])
    pk = peaks()
    T = 2048
    line = {
        "metric": f"decode tok/s @ batch {args.batch} (Qwen3-0.6B shape, {prompt_len:,}-token prompts)",
        "value": r["value"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "Qwen3-0.6B shape, random weights N(0,0.02)", "layers": cfg["num_hidden_layers"],
                   "layers_of_config": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied_embeddings": True,
                   "global_batch": args.batch, "prompt_len": prompt_len, "seq_len": context, "kv_block": 16,
                   "parallelism": "1 gpu", "cuda_graphs": False,
                   "how": f"ankur110/mini_engine unmodified from baseline/_ref, TORCH_CUDA_ARCH_LIST={r['arch']}, its LLM.step()"},
        "clocks": clocks.summary(),
        "e2e": {"value": r["e2e"], "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
        "prefill": {"value": round(T * 1000.0 / r["prefill_ms"], 1), "tokens": T, "ms": r["prefill_ms"],
                    "frac": round(prefill_flops(cfg, cfg["num_hidden_layers"], T) / (r["prefill_ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "points": r["points"],
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: mini_engine_b200 is a one-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    if args.mode in ("offline", "mixed"):
        return run_offline_mode(args)
    if args.mode == "decode":
        return run_decode_mode(args)
    if args.mode == "prefill":
        return run_prefill_mode(args)
    return run_step_mode(args)


if __name__ == "__main__":
    sys.exit(main())
