"""Shared helpers of the GPU tests: model folders, traces in four cuttings, comparisons."""
from __future__ import annotations

import functools
import os
import tempfile

import numpy as np
import torch

import plain_model
from mini_engine_b200.weights import write_random_model

# Largest absolute difference of logits (random tiny models give logits up to about 1.3).
# float32: only the order of sums differs.  bfloat16: activations are rounded to 8 bits of
# mantissa between the parts; the weights are the same bfloat16 numbers on both sides.
TOL = {"float32": 5e-5, "bfloat16": 3e-2}


# "A" is the tiny configuration A with the usual random weights N(0, 0.02).  "A!" is the same configuration with
# matrices N(0, 0.1): what the layers add to the residual stream then outweighs a token's own embedding and the
# logits spread over several units, so a wrong input token, a stale page or a wrong key changes the next token.
def _std_of(name: str) -> float:
    return 0.1 if name.endswith("!") else 0.02


def config_of(name: str):
    from tiny_configs import ALL
    return ALL[name.rstrip("!")]


@functools.lru_cache(maxsize=None)
def model_folder(name: str, dtype: str = "bfloat16") -> str:
    """A temporary model folder for a tiny configuration (made once per session, never committed)."""
    cfg, seed, _ = config_of(name)
    d = tempfile.mkdtemp(prefix=f"me_tiny_{name.rstrip('!')}_")
    return write_random_model(d, cfg, seed, dtype={"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype],
                              matrix_std=_std_of(name))


@functools.lru_cache(maxsize=None)
def plain_weights(name: str):
    return plain_model.load_folder(model_folder(name), torch.float64)


def random_requests(vocab: int, lengths, seed: int) -> list[list[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


@functools.lru_cache(maxsize=None)
def _plain_logits_cached(name: str, ids: tuple) -> np.ndarray:
    cfg, w = plain_weights(name)
    return plain_model.forward_logits(cfg, w, list(ids)).numpy()


def plain_logits(name: str, ids) -> np.ndarray:
    return _plain_logits_cached(name, tuple(ids))


# ---- traces: lists of steps for TraceReplayer / bin/trace_run --------------------------------
def trace_whole(reqs, first_step=0, tag="w"):
    """Each request alone and whole."""
    return [{"step": first_step + i, "entries": [{"id": f"{tag}{i}", "tokens": r, "want": list(range(len(r)))}],
             "end": [f"{tag}{i}"]} for i, r in enumerate(reqs)]


def trace_decode_tail(reqs, first_step=0, tail=32, tag="d"):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps, s = [], first_step
    for i, r in enumerate(reqs):
        head = max(1, len(r) - tail)
        steps.append({"step": s, "entries": [{"id": f"{tag}{i}", "tokens": r[:head], "want": list(range(head))}], "end": []})
        s += 1
        for p in range(head, len(r)):
            steps.append({"step": s, "entries": [{"id": f"{tag}{i}", "tokens": [r[p]], "want": [0]}],
                          "end": [f"{tag}{i}"] if p == len(r) - 1 else []})
            s += 1
        if head == len(r):
            steps[-1]["end"] = [f"{tag}{i}"]
    return steps


def trace_portions(reqs, sizes=(7, 2, 19, 3, 16, 2, 33, 5, 1, 64), first_step=0, tag="p"):
    """Portions of changing size, down to two tokens (and one)."""
    steps, s = [], first_step
    for i, r in enumerate(reqs):
        pos, k = 0, i                       # every request starts elsewhere in the size list
        while pos < len(r):
            n = min(sizes[k % len(sizes)], len(r) - pos)
            k += 1
            steps.append({"step": s, "entries": [{"id": f"{tag}{i}", "tokens": r[pos:pos + n], "want": list(range(n))}],
                          "end": [f"{tag}{i}"] if pos + n == len(r) else []})
            pos += n
            s += 1
    return steps


def trace_mixed(reqs, max_live=4, seed=0, first_step=0, tag="m", decode_tail=12):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others;
    requests may sit out a step; new requests start when others end, so pages are used again."""
    rng = np.random.RandomState(seed)
    steps, s = [], first_step
    waiting = list(range(len(reqs)))
    pos = {}
    live = []
    while waiting or live:
        while waiting and len(live) < max_live:
            i = waiting.pop(0)
            live.append(i)
            pos[i] = 0
        entries, ended = [], []
        for i in list(live):
            if len(live) > 1 and rng.rand() < 0.2:
                continue                                     # left out of this step
            r = reqs[i]
            left = len(r) - pos[i]
            n = 1 if left <= decode_tail else int(min(left - decode_tail, rng.choice([2, 3, 5, 8, 13, 21, 40])))
            entries.append({"id": f"{tag}{i}", "tokens": r[pos[i]:pos[i] + n], "want": list(range(n))})
            pos[i] += n
            if pos[i] == len(r):
                ended.append(f"{tag}{i}")
                live.remove(i)
        if entries:
            steps.append({"step": s, "entries": entries, "end": ended})
            s += 1
    return steps


def trace_mixed_shared(reqs, shared, max_live=4, seed=0, first_step=0, tag="s", decode_tail=12):
    """As ``trace_mixed``, with requests that repeat the start of another.  ``shared``: {i: (j, n, when)}: request i
    begins with request j's first n tokens and starts only once j has computed at least n tokens and still lives
    (when = "alive"), or once j has ended (when = "ended").  Its first portion holds those n tokens and a few more,
    and its logits are wanted from place n on, so that a replayer with prefix reuse may take the n tokens' pages
    from the cache."""
    rng = np.random.RandomState(seed)
    steps, s = [], first_step
    waiting = list(range(len(reqs)))
    pos, live, ended = {}, [], set()

    def may_start(i):
        if i not in shared:
            return True
        j, n, when = shared[i]
        return j in ended if when == "ended" else (j in live and pos[j] >= n)
    while waiting or live:
        for i in list(waiting):
            if len(live) < max_live and may_start(i):
                waiting.remove(i)
                live.append(i)
                pos[i] = 0
        assert live, "a request waits for one that never comes"
        entries, done = [], []
        for i in list(live):
            r = reqs[i]
            if len(live) > 1 and pos[i] > 0 and rng.rand() < 0.2:
                continue                                     # left out of this step
            left = len(r) - pos[i]
            if pos[i] == 0 and i in shared:
                n = shared[i][1] + int(rng.choice([1, 3, 6]))
                want = list(range(shared[i][1], n))
            else:
                n = 1 if left <= decode_tail else int(min(left - decode_tail, rng.choice([2, 3, 5, 8, 13, 21, 40])))
                want = list(range(n))
            assert n <= left
            entries.append({"id": f"{tag}{i}", "tokens": r[pos[i]:pos[i] + n], "want": want})
            pos[i] += n
            if pos[i] == len(r):
                done.append(i)
        for i in done:
            live.remove(i)
            ended.add(i)
        if entries:
            steps.append({"step": s, "entries": entries, "end": [f"{tag}{i}" for i in done]})
            s += 1
    return steps


def collect(steps, outputs) -> dict[str, np.ndarray]:
    """Per request id, the logits of all its positions in order ([len, vocab])."""
    rows: dict[str, list[np.ndarray]] = {}
    for st, out in zip(steps, outputs):
        k = 0
        for e in st["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(out[k])
                k += 1
        assert out is None or k == out.shape[0]
    return {rid: np.stack(v) for rid, v in rows.items()}


def max_live_tokens(steps) -> int:
    """Most tokens held at once, each request rounded up to 64 (what --max-tokens must cover)."""
    held, worst = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum((n + 63) // 64 * 64 for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return worst
