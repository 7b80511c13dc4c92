"""The engine at the layer sizes of Qwen3-0.6B, 8B and 32B (head size 128), in every way of cutting the work.

Few layers (two at the 0.6B sizes, one at the others) keep the plain implementation cheap; everything else is the
real shape: hidden 1,024 / 4,096 / 5,120, groups of 2 / 4 / 8 query heads, products with K up to 25,600, and at the
0.6B sizes the real vocabulary with a tied head.  These are the shapes where bfloat16 steps run the tcgen05
attention and product kernels, the tensor-map decode kernel with the q/k norm and rotary embedding folded in, the
small-batch products with norm and residual in their epilogues (0.6B) or the library and split-K products (8B, 32B),
and decode steps replayed from graphs.  The cuttings: each request alone and whole; its last 32 tokens one by one;
portions that cross 16/17, 127/128/129 and 1,024/1,025 rows (the row counts at which products change kernels); and
mixed steps of up to four live requests with so few pages that they are used again, with two requests that find
their first pages in the cache, every page that no live request wrote holding NaN.

Logits are wanted at a thinned set of places (all decoded tokens, every fifth place of a portion and its last), which
keeps the outputs small at a vocabulary of 151,936.  The plain implementation runs in float64 on the GPU (the same
torch code as on the host).
"""
import functools
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_model
from mini_engine_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

SIZES = {
    "0.6B": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                 num_hidden_layers=2, vocab_size=151936, tie_word_embeddings=True),
    "8B": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
               num_hidden_layers=1, vocab_size=2000, tie_word_embeddings=False),
    "32B": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=25600,
                num_hidden_layers=1, vocab_size=2000, tie_word_embeddings=False),
}
LENGTHS = {"0.6B": (1300, 260, 150, 400, 180, 330), "8B": (400, 260, 150, 330, 180), "32B": (400, 260, 150, 330, 180)}
TOL = {"float32": 2e-4, "bfloat16": 4e-2}          # times the largest logit (about 3 at these sizes)
PAGE = 16


@functools.lru_cache(maxsize=None)
def _model(name):
    cfg = dict(architectures=["Qwen3ForCausalLM"], rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=2048,
               **SIZES[name])
    folder = write_random_model(tempfile.mkdtemp(prefix=f"me_large_{name}_"), cfg, seed=4)
    c, w = plain_model.load_folder(folder, torch.float32)
    reqs = helpers.random_requests(min(cfg["vocab_size"], 10000), LENGTHS[name], seed=6)
    return folder, c, w, reqs


@functools.lru_cache(maxsize=None)
def _plain(name, ids: tuple, positions: tuple):
    _, c, w, _ = _model(name)
    return plain_model.forward_logits(c, w, list(ids), dtype=torch.float64, device="cuda", positions=list(positions)).numpy()


def thin_wants(steps, every=5):
    """Keeps, of each entry's wanted places, the decoded tokens, every ``every``-th place and the portion's last;
    returns {request: positions in the request whose logits the trace still wants, in order}."""
    pos, kept = {}, {}
    for st in steps:
        for e in st["entries"]:
            a, n = pos.get(e["id"], 0), len(e["tokens"])
            e["want"] = [w for w in e["want"] if n == 1 or w == n - 1 or (a + w) % every == 0]
            kept.setdefault(e["id"], []).extend(a + w for w in e["want"])
            pos[e["id"]] = a + n
    return kept


def _run(name, dtype, steps, max_tokens, **kw):
    from mini_engine_b200.engine.replay import TraceReplayer
    folder = _model(name)[0]
    kept = thin_wants(steps)
    rp = TraceReplayer(folder, dtype, max_tokens, page_size=PAGE, **kw)
    got = helpers.collect(steps, [rp.run_step(st) for st in steps])
    assert not rp.live and rp.cache.num_free_pages == [p.num_pages for p in rp.cache.pools]
    rp.runner.check_device_errors()
    graphs = sum(g.launches > 0 for g in rp.runner._graphs.values())
    hits = rp.cache.num_prefix_hit_tokens
    del rp
    torch.cuda.empty_cache()
    return got, kept, graphs, hits


def _check(name, dtype, reqs, got, kept, tag, what):
    for i, r in enumerate(reqs):
        rid = f"{tag}{i}"
        ref = _plain(name, tuple(r), tuple(kept[rid]))
        mine = got[rid]
        assert mine.shape == ref.shape and not np.isnan(mine).any()
        diff = np.abs(mine - ref).max(axis=1)
        tol = TOL[dtype] * max(1.0, float(np.abs(ref).max()))
        bad = np.nonzero(diff > tol)[0]
        assert bad.size == 0, (f"{name} {dtype} {what}, request {i}: first wrong token at position {kept[rid][bad[0]]} "
                               f"(diff {diff[bad[0]]:.3e}, tolerance {tol:.1e})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["0.6B", "8B", "32B"])
def test_whole_requests(name, dtype):
    reqs = list(_model(name)[3][:3])
    steps = helpers.trace_whole(reqs)
    got, kept, _, _ = _run(name, dtype, steps, helpers.max_live_tokens(steps))
    _check(name, dtype, reqs, got, kept, "w", "whole")


@pytest.mark.parametrize("name", ["0.6B", "8B"])
def test_a_prompt_of_so_many_rows_that_a_block_of_the_products_walks_tiles(name):
    # 1,900 tokens in one step: q|k|v and gate|up have two tiles an SM and more and run the persistent form of the tcgen05
    # product (at the 8B sizes the other two as well)
    from mini_engine_b200 import ops
    _, cfg, _, _ = _model(name)
    T = 1900
    assert ops.tcgen05_persistent_pays(T, cfg["intermediate_size"], cfg["hidden_size"], 1)
    (r,) = helpers.random_requests(2000, (T,), seed=12)
    steps = helpers.trace_whole([r])
    got, kept, _, _ = _run(name, "bfloat16", steps, helpers.max_live_tokens(steps))
    _check(name, "bfloat16", [r], got, kept, "w", "one long prompt")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["0.6B", "8B", "32B"])
def test_last_32_tokens_one_by_one(name, dtype):
    reqs = list(_model(name)[3][1:4])
    steps = helpers.trace_decode_tail(reqs)
    got, kept, graphs, _ = _run(name, dtype, steps, helpers.max_live_tokens(steps))
    assert graphs > 0                                    # the single tokens were replayed from a captured step
    _check(name, dtype, reqs, got, kept, "d", "last 32 tokens one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["0.6B", "8B", "32B"])
def test_portions_that_cross_the_row_counts_where_kernels_change(name, dtype):
    reqs = list(_model(name)[3][:3])
    sizes = (17, 127, 129, 1025, 2) if name == "0.6B" else (17, 127, 129, 16, 2, 128, 1)
    steps = helpers.trace_portions(reqs, sizes=sizes)
    if name == "0.6B":
        assert [len(st["entries"][0]["tokens"]) for st in steps[:5]] == [17, 127, 129, 1025, 2]
    got, kept, _, _ = _run(name, dtype, steps, helpers.max_live_tokens(steps))
    _check(name, dtype, reqs, got, kept, "p", "portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["0.6B", "8B", "32B"])
def test_mixed_steps_with_pages_used_again_and_prefix_hits(name, dtype):
    reqs = [list(r) for r in _model(name)[3][1:]] + [list(r)[:120] for r in _model(name)[3][1:4]]
    n = 2 * PAGE + 3
    reqs[2] = reqs[0][:n] + reqs[2]
    reqs[-1] = reqs[0][:n] + reqs[-1]
    shared = {2: (0, n, "alive"), len(reqs) - 1: (0, n, "ended")}
    steps = helpers.trace_mixed_shared(reqs, shared, max_live=4, seed=2, decode_tail=10)
    assert max(len(st["entries"]) for st in steps) == 4
    assert any(len(e["tokens"]) == 1 for st in steps for e in st["entries"] if any(len(o["tokens"]) > 1 for o in st["entries"]))
    need = helpers.max_live_tokens(steps)
    assert need < sum((len(r) + 63) // 64 * 64 for r in reqs)          # fewer pages than all requests: reuse
    got, kept, _, hits = _run(name, dtype, steps, need + 64, prefix_caching=True, poison=True)
    assert hits == 2 * (2 * PAGE)
    _check(name, dtype, reqs, got, kept, "s", "mixed")
