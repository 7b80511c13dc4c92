"""Trace replay against the plain implementation, in every way of cutting the work."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"A": (70, 45, 100, 33, 64, 129), "B": (37, 88, 50, 112, 41, 65), "C": (90, 47, 130, 36, 80, 52),
           "D": (150, 33, 97, 64, 200, 41)}


def _requests(name):
    return helpers.random_requests(ALL[name][0]["vocab_size"], LENGTHS[name], seed=11 + ALL[name][1])


def _replay(name, dtype, steps, max_tokens=None, **kw):
    from mini_engine_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(helpers.model_folder(name), dtype, max_tokens or helpers.max_live_tokens(steps),
                       page_size=helpers.config_of(name)[2], **kw)
    outs = [rp.run_step(st) for st in steps]
    assert not rp.live
    rp.cache.check([])
    assert rp.cache.num_free_pages == [p.num_pages for p in rp.cache.pools]
    return helpers.collect(steps, outs), rp


def _check(name, dtype, reqs, got, tag):
    tol = helpers.TOL[dtype]
    for i, r in enumerate(reqs):
        ref = helpers.plain_logits(name, r)
        mine = got[f"{tag}{i}"]
        assert mine.shape == ref.shape
        diff = np.abs(mine - ref).max(axis=1)
        bad = np.nonzero(diff > tol)[0]
        assert bad.size == 0, (f"config {name} {dtype} cutting {tag!r} request {i}: first wrong token at position "
                               f"{bad[0]} (diff {diff[bad[0]]:.3e}, tol {tol})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(name, dtype):
    reqs = _requests(name)
    got, _ = _replay(name, dtype, helpers.trace_whole(reqs))
    _check(name, dtype, reqs, got, "w")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_last_32_tokens_one_by_one(name, dtype):
    reqs = _requests(name)
    got, _ = _replay(name, dtype, helpers.trace_decode_tail(reqs))
    _check(name, dtype, reqs, got, "d")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_changing_size(name, dtype):
    reqs = _requests(name)
    got, _ = _replay(name, dtype, helpers.trace_portions(reqs))
    _check(name, dtype, reqs, got, "p")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_with_pages_used_again(name, dtype):
    reqs = _requests(name) + _requests(name)[:3]
    steps = helpers.trace_mixed(reqs, max_live=4, seed=3)
    assert max(len(st["entries"]) for st in steps) >= 3
    assert any(len(e["tokens"]) == 1 for st in steps for e in st["entries"] if len(st["entries"]) > 1)
    need = helpers.max_live_tokens(steps)
    assert need < sum((len(r) + 63) // 64 * 64 for r in reqs)          # fewer pages than all requests: reuse
    got, rp = _replay(name, dtype, steps, max_tokens=need)
    _check(name, dtype, reqs, got, "m")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "A!", "B!"])
def test_mixed_batches_with_prefix_hits_and_poisoned_pages(name, dtype):
    """The mixed cutting with two requests that repeat the first two pages (and three tokens) of request 0: one starts
    while request 0 lives, one after it has ended and its pages are free; both must find the pages instead of
    computing them.  Every page that no live request wrote holds NaN (the pool at the start, pages handed out,
    pages let go), so a key or value read from the wrong place shows in the logits."""
    cfg, _, page = helpers.config_of(name)
    reqs = _requests(name.rstrip("!")) + _requests(name.rstrip("!"))[:2]
    n = 2 * page + 3
    reqs[2] = reqs[0][:n] + reqs[2]
    reqs[6] = reqs[0][:n] + reqs[6][:40]
    shared = {2: (0, n, "alive"), 6: (0, n, "ended")}
    steps = helpers.trace_mixed_shared(reqs, shared, max_live=4, seed=5)
    need = helpers.max_live_tokens(steps)
    assert need < sum((len(r) + 63) // 64 * 64 for r in reqs)
    got, rp = _replay(name, dtype, steps, max_tokens=need + 64, prefix_caching=True, poison=True)
    assert rp.cache.num_prefix_hit_tokens == 2 * (2 * page)                   # both found their two pages
    tol = helpers.TOL[dtype] * (1.0 if not name.endswith("!") else 4.0)
    for i, r in enumerate(reqs):
        ref = helpers.plain_logits(name, r)
        first = shared[i][1] if i in shared else 0
        mine = got[f"s{i}"]
        assert mine.shape == ref[first:].shape and not np.isnan(mine).any()
        diff = np.abs(mine - ref[first:]).max(axis=1)
        bad = np.nonzero(diff > tol * max(1.0, np.abs(ref).max() if name.endswith("!") else 1.0))[0]
        assert bad.size == 0, f"config {name} {dtype} request {i}: first wrong token at position {first + bad[0]} (diff {diff[bad[0]]:.3e})"
    # the same trace without reuse computes the shared pages again and gives the same logits
    got2, rp2 = _replay(name, dtype, steps, max_tokens=need + 64, prefix_caching=False, poison=True)
    assert rp2.cache.num_prefix_hit_tokens == 0
    for k in got:
        assert np.abs(got[k] - got2[k]).max() <= 2 * tol * max(1.0, np.abs(got2[k]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype):
    name = "B"
    (r,) = helpers.random_requests(ALL[name][0]["vocab_size"], (300,), seed=5)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": r[:1], "want": [0]}], "end": []}]
    steps += [{"step": p, "entries": [{"id": "x", "tokens": [r[p]], "want": [0]}], "end": ["x"] if p == 299 else []}
              for p in range(1, 300)]
    got, _ = _replay(name, dtype, steps)
    _check(name, dtype, [r], {"x0": got["x"]}, "x")
    # the first tokens of a sequence, each as its own whole request
    for n in (1, 2, 3):
        got, _ = _replay(name, dtype, helpers.trace_whole([r[:n]]))
        _check(name, dtype, [r[:n]], got, "w")


@pytest.mark.parametrize("tiles", [2, 3])
def test_long_decoding_with_several_key_tiles_a_block(tiles):
    # the decode attention kernel in the form that large batches take (a block walks several tiles of 128 keys with a
    # running softmax), forced on one request: contexts from 100 to 420 tokens cross the tiles' and the partitions'
    # edges one token at a time, in a layer that sees all keys and in one with a window of 40 (config D)
    from mini_engine_b200 import ops
    name = "D"
    (r,) = helpers.random_requests(ALL[name][0]["vocab_size"], (420,), seed=7)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": r[:100], "want": list(range(100))}], "end": []}]
    steps += [{"step": p - 99, "entries": [{"id": "x", "tokens": [r[p]], "want": [0]}], "end": ["x"] if p == 419 else []}
              for p in range(100, 420)]
    old = ops.decode_form, ops.decode_tiles
    ops.decode_form, ops.decode_tiles = "one_tile", tiles
    try:
        got, _ = _replay(name, "bfloat16", steps)
    finally:
        ops.decode_form, ops.decode_tiles = old
    _check(name, "bfloat16", [r], {"x0": got["x"]}, "x")


def test_page_exhaustion_is_a_clear_error():
    reqs = _requests("A")
    steps = helpers.trace_whole(reqs[:1])
    steps[0]["end"] = []
    steps.append({"step": 1, "entries": [{"id": "other", "tokens": reqs[2], "want": []}], "end": []})
    with pytest.raises(RuntimeError, match="no pages left"):
        _replay("A", "float32", steps, max_tokens=128)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """The program itself, as a child process, step by step with the 'done' handshake."""
    name = "A"
    reqs = _requests(name)[:3]
    steps = helpers.trace_portions(reqs[:1]) + helpers.trace_mixed(reqs, max_live=3, seed=1, first_step=100)
    for k, st in enumerate(steps):
        st["step"] = k
    out = tmp_path / "out"
    env = dict(os.environ)
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", helpers.model_folder(name),
                             "--dtype", dtype, "--out", str(out), "--max-tokens", str(helpers.max_live_tokens(steps))],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    outs = []
    for st in steps:
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {st['step']}"
        n = sum(len(e["want"]) for e in st["entries"])
        path = out / f"{st['step']}.f32"
        outs.append(np.fromfile(path, dtype="<f4").reshape(n, -1) if n else None)
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    got = helpers.collect(steps, outs)
    _check(name, dtype, reqs[:1], got, "p")
    _check(name, dtype, reqs, got, "m")
