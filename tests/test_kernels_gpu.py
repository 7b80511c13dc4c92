"""Each CUDA kernel alone against its plain twin (tests/plain_ops.py), at many sizes."""
import math

import numpy as np
import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from mini_engine_b200 import ops as o
    o.require_extension()
    return o


_ERR = None


def errword():
    """The error word handed to products (the tcgen05 kernel reports a wait that ran out there)."""
    global _ERR
    if _ERR is None:
        _ERR = torch.zeros(4, dtype=torch.int32, device=DEV)
    return _ERR


@pytest.fixture(autouse=True)
def no_kernel_reported_an_error():
    yield
    if _ERR is not None:
        assert _ERR.tolist() == [0, 0, 0, 0]


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(a, b, dtype, scale=1.0):
    tol = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}[dtype] * scale
    d = (a.float() - b.float()).abs().max().item()
    assert d <= tol, f"max abs diff {d:.3e} > {tol:.3e}"


# ---- embedding ------------------------------------------------------------------------------
@pytest.mark.parametrize("wd", ["float32", "bfloat16"])
def test_embed(ops, wd):
    V, H, T = 333, 96, 37
    table = rnd(V, H, dtype=DT[wd])
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    out = torch.full((T, H), float("nan"), device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.embed(ids, table, out, err)
    assert torch.equal(out, table[ids.long()].float()) and err.tolist() == [0, 0, 0, 0]
    ids[5] = V
    ops.embed(ids, table, out, err)
    assert err[0].item() == 1 and torch.all(out[5] == 0)


# ---- residual add + RMSNorm --------------------------------------------------------------------
@pytest.mark.parametrize("H", [64, 96, 1000, 1001, 1024, 2048, 4104, 8200, 9001])
@pytest.mark.parametrize("od", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [19, 333])
def test_add_rmsnorm(ops, H, od, T):
    # (from 64 rows on and up to 2,048 columns a warp takes a row: another kernel than for a handful of rows)
    for delta_dt in (None, od, "float32"):
        res = rnd(T, H, seed=1)
        delta = None if delta_dt is None else rnd(T, H, dtype=DT[delta_dt], seed=2)
        w = 1 + 0.1 * rnd(H, seed=3)
        out, ref_out = torch.empty(T, H, dtype=DT[od], device=DEV), torch.empty(T, H, dtype=DT[od], device=DEV)
        ref_res = res.clone()
        plain_ops.add_rmsnorm(ref_res, delta, w, 1e-5, ref_out)
        ops.add_rmsnorm(res, delta, w, 1e-5, out)
        assert torch.allclose(res, ref_res, atol=1e-6)
        close(out, ref_out, DT[od], scale=4)
    # partial results of a product split along K: [splits, T, H] float32, added in order
    res, parts = rnd(T, H, seed=6), rnd(3, T, H, seed=7)
    ref_res = res.clone()
    plain_ops.add_rmsnorm(ref_res, parts, w, 1e-5, ref_out)
    ops.add_rmsnorm(res, parts, w, 1e-5, out)
    assert torch.allclose(res, ref_res, atol=2e-6)
    close(out, ref_out, DT[od], scale=4)
    # gathered rows: the residual is read, not written
    res, delta = rnd(T, H, seed=4), rnd(T, H, dtype=DT[od], seed=5)
    rows = torch.tensor([3, 0, 18, 3], dtype=torch.int32, device=DEV)
    keep = res.clone()
    out, ref_out = torch.empty(4, H, dtype=DT[od], device=DEV), torch.empty(4, H, dtype=DT[od], device=DEV)
    ops.add_rmsnorm(res, delta, w, 1e-6, out, rows=rows)
    plain_ops.add_rmsnorm(keep.clone(), delta, w, 1e-6, ref_out, rows=rows)
    assert torch.equal(res, keep)
    close(out, ref_out, DT[od], scale=4)


def test_silu_mul(ops):
    for dt in (torch.float32, torch.bfloat16):
        x = rnd(23, 2 * 200, dtype=dt, scale=2.0)
        out, ref = torch.empty(23, 200, dtype=dt, device=DEV), torch.empty(23, 200, dtype=dt, device=DEV)
        ops.silu_mul(x, out)
        plain_ops.silu_mul(x, ref)
        close(out, ref, dt, scale=4)


# ---- matrix products ------------------------------------------------------------------------
@pytest.mark.parametrize("M, N, K", [(1, 96, 64), (37, 224, 96), (130, 333, 72), (5, 1000, 513), (64, 64, 16), (8, 4096, 1024)])
@pytest.mark.parametrize("kinds", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "bfloat16"),
                                   ("bfloat16", "bfloat16", "float32"), ("bfloat16", "float32", "bfloat16")])
def test_linear(ops, M, N, K, kinds):
    xd, wd, od = (DT[k] for k in kinds)
    x, w = rnd(M, K, dtype=xd, seed=1), rnd(N, K, dtype=wd, seed=2, scale=K ** -0.5)
    out, ref = torch.empty(M, N, dtype=od, device=DEV), torch.empty(M, N, dtype=od, device=DEV)
    ops.linear(x, w, out, err=errword())
    plain_ops.linear(x, w, ref)
    close(out, ref, od, scale=4)


@pytest.mark.parametrize("M, N, K", [(128, 1024, 2048), (300, 1000, 3072), (1024, 96, 1024), (520, 1024, 584)])
def test_products_split_along_k(ops, M, N, K):
    # the tcgen05 product with K shared out over several blocks a tile: float32 partial results that sum to the product
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=K ** -0.5)
    ref = torch.empty(M, N, device=DEV)
    plain_ops.linear(x, w, ref)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    for bn in (64, 128, 256):
        for want in (2, 3, 4):
            n = ops.tcgen05_splits(K, want)
            part = torch.full((n, M, N), float("nan"), device=DEV)
            ops.linear_tcgen05(x, w, part, "none", err, tile_n=bn, splits=want if n == want else n)
            close(part.sum(0), ref, torch.float32, scale=4)
    assert err.tolist() == [0, 0, 0, 0]
    # the engine's choice, through the call that a feed-forward or attention output makes
    ws = {}
    part = ops.linear_partials(x, w, lambda name, shape, dt: ws.setdefault(name, torch.full(shape, float("nan"), dtype=dt, device=DEV)), "p", err=err)
    bn, parts = ops.tcgen05_split_plan(M, N, K)
    assert (part is None) == (parts < 2)
    if part is not None:
        assert part.shape == (parts, M, N)
        close(part.sum(0), ref, torch.float32, scale=4)


@pytest.mark.parametrize("M, I, K", [(1, 128, 64), (37, 224, 96), (70, 200, 72), (8, 3072, 1024)])
@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
def test_linear_silu_mul(ops, M, I, K, dt):
    x, w = rnd(M, K, dtype=DT[dt], seed=1), rnd(2 * I, K, dtype=DT[dt], seed=2, scale=K ** -0.5)
    out, ref = torch.empty(M, I, dtype=DT[dt], device=DEV), torch.empty(M, I, dtype=DT[dt], device=DEV)
    ops.linear(x, w, out, epilogue="silu_mul", err=errword())
    plain_ops.linear(x, w, ref, epilogue="silu_mul")
    close(out, ref, DT[dt], scale=4)


@pytest.mark.parametrize("M", [1, 3, 8, 16])
@pytest.mark.parametrize("N, K", [(96, 64), (1000, 200), (4096, 1024), (1024, 2048), (1030, 3072), (200, 4096 + 72)])
def test_small_batch_products(ops, M, N, K):
    # the decode kernel: bfloat16 and float32 results, split-K partial results, SiLU-and-multiply
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=K ** -0.5)
    splits = ops.skinny_splits(M, K, x, w)
    assert splits == (K + 1023) // 1024
    ref = torch.empty(M, N, dtype=torch.float32, device=DEV)
    plain_ops.linear(x, w, ref)
    ws = {}

    def workspace(name, shape, dt):
        return ws.setdefault(name, torch.full(tuple(shape), float("nan"), dtype=dt, device=DEV))
    part = ops.linear_partials(x, w, workspace, "p", err=errword())
    if splits == 1:
        assert part is None
        for od in (torch.bfloat16, torch.float32):
            before = ops.library_calls
            out = torch.full((M, N), float("nan"), dtype=od, device=DEV)
            ops.linear(x, w, out, err=errword())
            assert ops.library_calls == before                     # our kernel, not the library
            close(out, ref, od, scale=4)
    else:
        assert part.shape == (splits, M, N) and part.dtype == torch.float32
        close(part.sum(0), ref, torch.float32, scale=50)            # bfloat16 inputs, float32 sums
        res = rnd(M, N, seed=5)
        wn = 1 + 0.1 * rnd(N, seed=6)
        out, ref_out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV), torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        res2 = res.clone()
        ops.add_rmsnorm(res, part, wn, 1e-6, out)
        plain_ops.add_rmsnorm(res2, part, wn, 1e-6, ref_out)
        assert torch.allclose(res, res2, atol=1e-5)
        close(out, ref_out, torch.bfloat16, scale=4)
    if K <= 1024 and N % 2 == 0:
        I = N // 2
        out, ref2 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV), torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        before = ops.library_calls
        ops.linear(x, w, out, epilogue="silu_mul", workspace=workspace, err=errword())
        assert ops.library_calls == before
        plain_ops.linear(x, w, ref2, epilogue="silu_mul")
        close(out, ref2, torch.bfloat16, scale=4)


@pytest.mark.parametrize("M, N, K", [(128, 64, 64), (128, 128, 64), (129, 200, 136), (300, 4096, 1024), (2048, 1024, 2048),
                                     (1000, 1032, 3072), (64, 151936 // 16, 1024), (3000, 9000, 264), (300, 1002, 264)])
@pytest.mark.parametrize("tile_n, persistent", [(64, False), (128, False), (256, False), (128, True), (256, True)])
def test_tcgen05_products(ops, M, N, K, tile_n, persistent):
    # the tcgen05 kernels by name: every tile width, edges in M, N and K, bfloat16 and float32 results, SiLU epilogue;
    # one tile a block, and the persistent form (a block walks tiles: none, one, or half a dozen with the shape before the
    # last); the last shape's rows of results are not 16-byte aligned and leave element by element
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=K ** -0.5)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    for od in (torch.bfloat16, torch.float32):
        out, ref = torch.full((M, N), float("nan"), dtype=od, device=DEV), torch.empty(M, N, dtype=od, device=DEV)
        ops.linear_tcgen05(x, w, out, "none", err, tile_n=tile_n, persistent=persistent)
        plain_ops.linear(x, w, ref)
        assert err.tolist() == [0, 0, 0, 0]
        close(out, ref, od, scale=4)
    if N % 2 == 0:
        I = N // 2
        out, ref = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV), torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        ops.linear_tcgen05(x, w, out, "silu_mul", err, tile_n=tile_n, persistent=persistent)
        plain_ops.linear(x, w, ref, epilogue="silu_mul")
        assert err.tolist() == [0, 0, 0, 0]
        close(out, ref, torch.bfloat16, scale=4)


@pytest.mark.parametrize("M, N, K", [(128, 256, 64), (129, 200, 136), (300, 4096, 1024), (256, 512, 8192), (1000, 1032, 3072),
                                     (2048, 5000, 520), (3000, 9000, 264), (40000, 256, 64), (300, 1002, 264)])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_tcgen05_products_with_the_work_shared_out_evenly(ops, M, N, K, tile_n):
    # the stages of the last rounds' tiles cut into one range an SM: a tile shared by two blocks and by six, tiles that
    # no block shares, fewer stages than SMs, a block with whole tiles before its share, edges in M, N and K; twice, so that
    # the second run finds the flags as the first left them
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=K ** -0.5)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    for od in (torch.bfloat16, torch.float32, torch.bfloat16):
        out, ref = torch.full((M, N), float("nan"), dtype=od, device=DEV), torch.empty(M, N, dtype=od, device=DEV)
        ops.linear_tcgen05(x, w, out, "none", err, tile_n=tile_n, share=True)
        plain_ops.linear(x, w, ref)
        assert err.tolist() == [0, 0, 0, 0]
        close(out, ref, od, scale=4)
    I = N // 2
    out, ref = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV), torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    ops.linear_tcgen05(x, w, out, "silu_mul", err, tile_n=tile_n, share=True)
    plain_ops.linear(x, w, ref, epilogue="silu_mul")
    assert err.tolist() == [0, 0, 0, 0]
    close(out, ref, torch.bfloat16, scale=4)
    assert all(int(f.sum()) == 0 for _, f in ops._shared_ws.values())


def test_which_tcgen05_products_share_their_work(ops):
    sms = ops.sm_count()
    assert ops.tcgen05_share_pays(1024, 6144, 4096, 0) == (sms == 148)          # 192 tiles: a second round a third full
    assert not ops.tcgen05_share_pays(1024, 6144, 4096, 1)                      # never with the SiLU epilogue
    assert not ops.tcgen05_share_pays(8192, 6144, 4096, 0)                      # 1,536 tiles: the last round hardly matters
    assert not ops.tcgen05_share_pays(256, 4096, 1024, 0)                       # few tiles, short K: nothing to share
    assert not ops.tcgen05_share_pays(1280, 4096, 1024, 0)                      # a short K: handing sums over costs what a tile takes
    assert not ops.tcgen05_share_pays(1024, 4096, 12288, 0)                     # eight tiles to a tile of W, at different places along K
    assert ops.tcgen05_share_pays(512, 4096, 12288, 0) == (sms == 148)          # 64 tiles, a long K


def test_which_tcgen05_products_get_a_block_an_sm_for_one_round(ops):
    if ops.sm_count() != 148:
        pytest.skip("the rule's examples are for 148 SMs")
    assert ops.tcgen05_one_round_width(2048, 1024) == 128          # 16 x 8 tiles of 128 columns
    assert ops.tcgen05_one_round_width(4096, 1024) == 256          # 32 x 4 tiles of 256 columns
    assert ops.tcgen05_one_round_width(512, 1024) == 0             # a third of the SMs either way


@pytest.fixture
def decode_kernel(ops, request):
    """Which of the two decode product kernels ``ops.decode_linear`` runs: one block over all of K (csrc/gemm_decode.cu)
    or blocks that walk their rows along any K (csrc/gemm_stream.cu)."""
    old, ops.decode_kernel = ops.decode_kernel, request.param
    yield request.param
    ops.decode_kernel = old


@pytest.mark.parametrize("M", [1, 5, 8, 16])
@pytest.mark.parametrize("decode_kernel, N, K", [
    ("decode", 96, 64), ("decode", 1000, 200), ("decode", 4096, 1024), ("decode", 1024, 2048), ("decode", 1032, 3072),
    ("stream", 96, 64), ("stream", 1000, 200), ("stream", 4096, 1024), ("stream", 1032, 3072), ("stream", 1000, 4096 + 72),
    ("stream", 5120, 5120), ("stream", 2600, 2056), ("auto", 520, 12288)], indirect=["decode_kernel"])
def test_decode_products_with_norm_and_residual_folded_in(ops, decode_kernel, M, N, K):
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=K ** -0.5)
    assert ops.decode_linear_takes(M, K, w)
    ref = torch.empty(M, N, dtype=torch.float32, device=DEV)
    plain_ops.linear(x, w, ref)
    # plain input, float32 and bfloat16 output
    for od in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), dtype=od, device=DEV)
        ops.decode_linear(w, x, err=errword(), out=out)
        close(out, ref, od, scale=4)
    # residual epilogue: residual += x W^T, the sums of squares of the new residual per strip of 16 columns, and
    # the new residual times the next norm's weight
    res = rnd(M, N, seed=3)
    want = res + ref
    parts = ops.decode_linear_sumsq_parts(N, K)
    if decode_kernel == "decode":
        width = 16 if parts == (N + 15) // 16 else 8         # narrow strips where 16 columns would make few blocks
        assert parts == (N + width - 1) // width
        edges = [min(N, p * width) for p in range(parts + 1)]
    else:        # a part a block: block b adds the columns of the groups (of 128) whose first piece of K lies in its share
        groups, its = (N + 127) // 128, (K + 127) // 128
        assert parts == min(groups * its, ops.sm_count())
        ends = [-(-(groups * its * b // parts) // its) for b in range(parts + 1)]   # groups begun before block b starts
        edges = [min(N, 128 * e) for e in ends]
    sumsq = torch.full((parts, M), float("nan"), device=DEV)
    next_w = 1 + 0.3 * rnd(N, seed=6)
    xw = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.decode_linear(w, x, err=errword(), epilogue="residual", residual_out=res, sumsq_out=sumsq, next_norm=(next_w, xw))
    close(res, want, torch.float32, scale=50)
    want_sq = torch.stack([res[:, a:b].pow(2).sum(-1) for a, b in zip(edges, edges[1:])])
    assert torch.allclose(sumsq, want_sq, rtol=1e-4, atol=1e-5)
    assert torch.equal(xw, (res * next_w).to(torch.bfloat16))
    res2, sumsq2 = rnd(M, N, seed=3), torch.empty_like(sumsq)
    later = rnd(777, 40, dtype=torch.bfloat16, seed=9)                                       # asked into L2 on the way
    ops.decode_linear(w, x, err=errword(), epilogue="residual", residual_out=res2, sumsq_out=sumsq2, fetch_ahead=later)    # no next norm
    assert torch.equal(res2, res) and torch.equal(sumsq2, sumsq)
    # the other half of that norm: a product over a pre-weighted residual applies the rows' factors to its results
    K_parts = (K + 15) // 16
    resk = rnd(M, K, seed=4, scale=3.0)
    sq_in = torch.nn.functional.pad(resk, (0, K_parts * 16 - K)).view(M, K_parts, 16).pow(2).sum(-1).t().contiguous()
    nw = 1 + 0.1 * rnd(K, seed=5)
    pre = (resk * nw).to(torch.bfloat16)
    xn = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    plain_ops.add_rmsnorm(resk.clone(), None, nw, 1e-5, xn)
    refn = torch.empty(M, N, dtype=torch.float32, device=DEV)
    plain_ops.linear(xn, w, refn)
    # (the same arithmetic in float64 for the tight comparison, the plain norm-then-product for the meaning)
    factor = (resk.double().pow(2).mean(-1, keepdim=True) + 1e-5).rsqrt()
    sharp = ((pre.double() @ w.double().t()) * factor).float()
    for od in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), dtype=od, device=DEV)
        ops.decode_linear(w, pre, err=errword(), out=out, row_scale=(sq_in, 1e-5))
        close(out, sharp, od, scale=4)
        close(out, refn, torch.bfloat16, scale=4)
    res3, sumsq3 = rnd(M, N, seed=7), torch.empty_like(sumsq)
    want3 = res3 + sharp
    ops.decode_linear(w, pre, err=errword(), epilogue="residual", residual_out=res3, sumsq_out=sumsq3, row_scale=(sq_in, 1e-5))
    close(res3, want3, torch.float32, scale=50)
    if N % 2 == 0:
        I = N // 2
        out2, ref2 = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV), torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        ops.decode_linear(w, pre, err=errword(), out=out2, epilogue="silu_mul", row_scale=(sq_in, 1e-5))
        plain_ops.linear(xn, w, ref2, epilogue="silu_mul")
        close(out2, ref2, torch.bfloat16, scale=4)


@pytest.mark.parametrize("M", [1, 7, 16])
@pytest.mark.parametrize("N, K", [(17001, 1000), (8300, 2048 + 24)])
def test_vocabulary_sized_products_of_few_rows(ops, M, N, K):
    # a weight of 32 MB and more under up to 16 rows (the LM head in decode) streams through csrc/gemm_stream.cu:
    # our kernel, both output types, rows beyond N and columns beyond K filled with zeros by the tensor maps
    assert N * K >= ops.STREAM_MIN_WEIGHT_ELEMENTS
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2, scale=K ** -0.5)
    w[N - 3] *= 400                                                 # one row that stands out, near the ragged end
    ref = torch.empty(M, N, dtype=torch.float32, device=DEV)
    plain_ops.linear(x, w, ref)
    for od in (torch.float32, torch.bfloat16):
        before, launched = ops.library_calls, ops.launches
        out = torch.full((M, N), float("nan"), dtype=od, device=DEV)
        ops.linear(x, w, out, err=errword())
        assert ops.library_calls == before and ops.launches == launched + 1
        assert (out.float().abs().argmax(dim=1) == N - 3).all()
        shrink = torch.ones(N, device=DEV)
        shrink[N - 3] = 1 / 400                                         # (that column at the others' magnitude)
        close(out.float() * shrink, ref * shrink, od, scale=4)


def test_linear_rows_do_not_depend_on_the_batch(ops):
    x, w = rnd(70, 96, seed=1), rnd(224, 96, seed=2)
    full, one = torch.empty(70, 224, device=DEV), torch.empty(1, 224, device=DEV)
    ops.linear(x, w, full, err=errword())
    ops.linear(x[41:42], w, one, err=errword())
    assert torch.equal(full[41:42], one)


def test_remembered_launches_follow_their_tensors(ops):
    # a product or norm called again with the same tensors launches with last time's arguments: the result must
    # follow the tensors' contents, and tensors of other shapes, kinds or places must not be taken for them
    bf = torch.bfloat16
    w = rnd(96, 64, dtype=bf, seed=2, scale=0.125)
    x, out, ref = rnd(130, 64, dtype=bf, seed=1), torch.empty(130, 96, dtype=bf, device=DEV), torch.empty(130, 96, dtype=bf, device=DEV)
    for seed in (1, 5, 9):                                   # same tensors, new contents: twice remembered
        x.copy_(rnd(130, 64, dtype=bf, seed=seed))
        ops.linear(x, w, out, err=errword())
        plain_ops.linear(x, w, ref)
        close(out, ref, bf, scale=4)
    before = ops.launches
    ops.linear(x, w, out, err=errword())
    assert ops.launches == before + 1
    for M, dt in ((130, torch.float32), (7, bf), (131, bf)):  # other kinds and sizes, some at the same addresses as before
        del x, out, ref
        x, w2 = rnd(M, 64, dtype=dt, seed=3), w.to(dt)
        out, ref = torch.empty(M, 96, dtype=dt, device=DEV), torch.empty(M, 96, dtype=dt, device=DEV)
        for _ in range(2):
            out.fill_(float("nan"))
            ops.linear(x, w2, out, err=errword())
            plain_ops.linear(x, w2, ref)
            close(out, ref, dt, scale=4)
    res, delta = rnd(70, 96, seed=4), rnd(70, 96, dtype=bf, seed=5)
    nw, y, y_ref = 1 + 0.1 * rnd(96, seed=6), torch.empty(70, 96, dtype=bf, device=DEV), torch.empty(70, 96, dtype=bf, device=DEV)
    res_ref = res.clone()
    for _ in range(3):                                       # the residual grows each time: a stale launch would show
        ops.add_rmsnorm(res, delta, nw, 1e-6, y)
        plain_ops.add_rmsnorm(res_ref, delta, nw, 1e-6, y_ref)
        close(res, res_ref, torch.float32, scale=8)
        close(y, y_ref, bf, scale=4)
    ops.remember_launches = False
    try:
        ops.add_rmsnorm(res, delta, nw, 1e-6, y)
        plain_ops.add_rmsnorm(res_ref, delta, nw, 1e-6, y_ref)
        close(y, y_ref, bf, scale=4)
    finally:
        ops.remember_launches = True


# ---- q/k norm + rotary + cache write --------------------------------------------------------------
@pytest.mark.parametrize("nh, nkv, hd", [(4, 2, 16), (8, 2, 32), (6, 3, 48), (16, 8, 128), (5, 5, 80), (2, 1, 256)])
@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
@pytest.mark.parametrize("norm, rope", [(True, True), (False, True), (True, False)])
def test_qk_norm_rope_kv_write(ops, nh, nkv, hd, dt, norm, rope):
    T, page, pages = 29, 8, 9
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=DT[dt], seed=1)
    qw = (1 + 0.1 * rnd(hd, seed=2)) if norm else None
    kw = (1 + 0.1 * rnd(hd, seed=3)) if norm else None
    pos = torch.randint(0, 200, (T,), dtype=torch.int32, device=DEV)
    inv = 1.0 / (5000.0 ** (torch.arange(0, hd, 2).float() / hd))
    fr = torch.outer(torch.arange(200).float(), inv)
    cs = torch.cat((fr.cos(), fr.sin()), -1).to(DEV) if rope else None
    slots = torch.randperm(pages * page)[:T].to(torch.int32).to(DEV)
    slots[7] = -1
    pool = torch.full((pages, 2, nkv, page, hd), float("nan"), dtype=DT[dt], device=DEV)
    ref_qkv, ref_pool = qkv.clone(), pool.clone()
    ops.qk_norm_rope_kv_write(qkv, nh, nkv, hd, qw, kw, 1e-5, cs, pos, slots, pool, page)
    plain_ops.qk_norm_rope_kv_write(ref_qkv, nh, nkv, hd, qw, kw, 1e-5, cs, pos, slots, ref_pool, page)
    close(qkv, ref_qkv, DT[dt], scale=4)
    assert torch.equal(pool.isnan(), ref_pool.isnan())                  # exactly the given slots were written
    close(pool.nan_to_num(0), ref_pool.nan_to_num(0), DT[dt], scale=4)
    # v is copied bit for bit (csrc/kv_cache.cu in the reference is bit-exact too)
    s = int(slots[0])
    assert torch.equal(pool[s // page, 1, :, s % page].reshape(-1), qkv[0, (nh + nkv) * hd:])
    # without a slot mapping nothing is written
    pool2 = torch.zeros_like(pool)
    ops.qk_norm_rope_kv_write(ref_qkv.clone(), nh, nkv, hd, qw, kw, 1e-5, cs, pos, None, pool2, page)
    assert not pool2.any()


@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, hd, rd", [(4, 2, 64, 32), (16, 8, 128, 64), (3, 1, 48, 16), (8, 2, 32, 2), (2, 2, 256, 192),
                                             (5, 1, 80, 80)])
def test_rotation_of_the_first_elements_of_a_head_only(ops, nh, nkv, hd, rd, dt):
    # partial rotary: the first rd elements of each head are rotated, the others only normalised
    T, page, pages = 29, 16, 5
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=DT[dt], seed=3)
    qw, kw = 1 + 0.1 * rnd(hd, seed=1), 1 + 0.1 * rnd(hd, seed=2)
    pos = torch.randint(0, 200, (T,), dtype=torch.int32, device=DEV)
    inv = 1.0 / (5000.0 ** (torch.arange(0, rd, 2).float() / rd))
    fr = torch.outer(torch.arange(200).float(), inv)
    cs = torch.cat((fr.cos(), fr.sin()), -1).to(DEV)
    slots = torch.randperm(pages * page)[:T].to(torch.int32).to(DEV)
    pool = torch.full((pages, 2, nkv, page, hd), float("nan"), dtype=DT[dt], device=DEV)
    ref_qkv, ref_pool = qkv.clone(), pool.clone()
    ops.qk_norm_rope_kv_write(qkv, nh, nkv, hd, qw, kw, 1e-5, cs, pos, slots, pool, page, rotary_dim=rd)
    plain_ops.qk_norm_rope_kv_write(ref_qkv, nh, nkv, hd, qw, kw, 1e-5, cs, pos, slots, ref_pool, page, rotary_dim=rd)
    close(qkv, ref_qkv, DT[dt], scale=4)
    assert torch.equal(pool.isnan(), ref_pool.isnan())
    close(pool.nan_to_num(0), ref_pool.nan_to_num(0), DT[dt], scale=4)
    if rd < hd:                                       # and the table must have the width that is named
        with pytest.raises(ops.KernelError, match="rotary"):
            ops.qk_norm_rope_kv_write(qkv, nh, nkv, hd, qw, kw, 1e-5, cs, pos, slots, pool, page)
    with pytest.raises(ops.KernelError, match="interleaved"):
        ops.qk_norm_rope_kv_write(qkv, nh, nkv, hd, qw, kw, 1e-5, cs, pos, slots, pool, page, rotary_dim=rd, layout="interleaved")


def test_head_dim_is_checked(ops):
    with pytest.raises(ValueError, match="head_dim"):
        ops.check_attention_sizes(40, 4, 2)
    with pytest.raises(ValueError, match="head_dim"):
        ops.check_attention_sizes(272, 4, 2)
    with pytest.raises(ValueError):
        ops.check_attention_sizes(64, 6, 4)


# ---- attention ------------------------------------------------------------------------------
class Batch:
    """Requests with cached context and new tokens, laid out in a scattered, NaN-filled pool."""

    def __init__(self, ctx_lens, q_lens, nh, nkv, hd, page, dtype, seed=0, standout=None, window=None):
        from mini_engine_b200.engine.step_context import AttnMeta
        g = torch.Generator().manual_seed(seed)
        B, T = len(ctx_lens), sum(q_lens)
        order = sorted(range(B), key=lambda b: q_lens[b] != 1)            # single tokens first
        ctx_lens, q_lens = [ctx_lens[b] for b in order], [q_lens[b] for b in order]
        self.nh, self.nkv, self.hd, self.page = nh, nkv, hd, page
        n_pages = sum((L + page - 1) // page for L in ctx_lens) + 3
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.pool = torch.full((n_pages, 2, nkv, page, hd), float("nan"), dtype=dtype)
        width = max((L + page - 1) // page for L in ctx_lens) + 1
        bt = torch.full((B, width), -1, dtype=torch.int32)
        self.qkv = (torch.randn(T, (nh + 2 * nkv) * hd, generator=g)).to(dtype)
        cu = [0]
        for b, (L, n) in enumerate(zip(ctx_lens, q_lens)):
            k = torch.randn(L, nkv, hd, generator=g) * 0.5
            v = torch.randn(L, nkv, hd, generator=g)
            if standout is not None:                                      # one key whose score stands out
                jb, tb = standout(b, L, n)
                if jb is not None:
                    q = self.qkv[cu[-1] + tb].float().view(nh + 2 * nkv, hd)[:nh]
                    for kh in range(nkv):
                        qd = q[kh * (nh // nkv)]
                        k[jb, kh] = 12.0 * qd / qd.norm() ** 2 * math.sqrt(hd)
            for i in range((L + page - 1) // page):
                p = perm.pop()
                bt[b, i] = p
                n_in = min(page, L - i * page)
                if window is not None and (i + 1) * page <= L - n - window + 1:
                    bt[b, i] = -1                                        # behind every window: given back
                    continue
                self.pool[p, 0, :, :n_in] = k[i * page:i * page + n_in].transpose(0, 1).to(dtype)
                self.pool[p, 1, :, :n_in] = v[i * page:i * page + n_in].transpose(0, 1).to(dtype)
            cu.append(cu[-1] + n)
        D = sum(1 for n in q_lens if n == 1)
        from mini_engine_b200 import ops as o

        def tile_list(first, tq):
            t = [(b, q0) for b in range(first, B) for q0 in range(0, q_lens[b], tq)]
            return torch.tensor(t or [(0, 0)], dtype=torch.int32, device=DEV), len(t)
        self.pool, self.qkv, self.bt = self.pool.to(DEV), self.qkv.to(DEV), bt.to(DEV)
        self._ws = {}

        def workspace(name, shape, dt, zero=False):
            key = (name, tuple(shape), dt)
            if key not in self._ws:
                self._ws[key] = (torch.zeros(tuple(shape), dtype=dt, device=DEV) if zero
                                 else torch.full(tuple(shape), float("nan"), dtype=dt, device=DEV))
            return self._ws[key]
        self.meta = AttnMeta(num_reqs=B, num_tokens=T, num_decodes=D,
                             cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=DEV),
                             context_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
                             tile_lists={tq: tile_list(D, tq) for tq in o.ATTN_TILE_SIZES}, num_tiles=B - D,
                             max_context_len=max(ctx_lens), workspace=workspace,
                             error_flag=torch.zeros(4, dtype=torch.int32, device=DEV))
        self.all_tiles = {tq: tile_list(0, tq) for tq in o.ATTN_TILE_SIZES}     # single tokens as tiles too
        self.q_lens, self.ctx_lens = q_lens, ctx_lens


def run_attention(ops, bt: Batch, dtype, window, which="split"):
    T = bt.qkv.shape[0]
    out = torch.full((T, bt.nh * bt.hd), float("nan"), dtype=dtype, device=DEV)
    ref = torch.empty_like(out)
    scale = bt.hd ** -0.5
    args = (bt.nh, bt.nkv, bt.hd, bt.pool, bt.page, bt.bt, bt.meta, scale, window)
    if which == "split":                                                   # decode kernel + the dtype's prefill kernel
        ops.paged_attention(bt.qkv, out, *args)
    elif which == "chunks":                                                # everything through the CUDA-core chunk kernel
        tiles, n = bt.all_tiles[ops.ATTN_TILE_Q]
        ops.attention_chunks(bt.qkv, out, *args, tiles=tiles, num_tiles=n)
    elif which == "tensor":                                                # everything through the mma.sync kernel
        tiles, n = bt.all_tiles[64 // ops.prefill_heads_per_block(bt.nh, bt.nkv, bt.hd)]
        ops.attention_prefill(bt.qkv, out, *args, tiles=tiles, num_tiles=n)
    else:                                                                  # everything through the tcgen05 kernel
        tiles, n = bt.all_tiles[128 // ops.prefill_tcgen05_heads_per_block(bt.nh, bt.nkv, bt.hd, bt.page)]
        key_tile = 128 if which.endswith("128") or bt.page > 64 else 64
        ops.attention_prefill_tcgen05(bt.qkv, out, *args, tiles=tiles, num_tiles=n, key_tile=key_tile)
    plain_ops.paged_attention(bt.qkv, ref, *args)
    assert not out.isnan().any(), "the kernel read a slot that no request owns (NaN-filled pool)"
    assert bt.meta.error_flag.tolist() == [0, 0, 0, 0]
    return out, ref


SHAPES = [(4, 2, 16, 16), (8, 2, 32, 8), (6, 3, 48, 16), (16, 8, 128, 16), (8, 1, 64, 32), (5, 5, 80, 4), (4, 2, 256, 16)]


@pytest.mark.parametrize("nh, nkv, hd, page", SHAPES)
@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
def test_attention_mixed_batch(ops, nh, nkv, hd, page, dt):
    # portions of prompts (with and without earlier context), single tokens, lengths at tile and page edges
    ctx = [1, 300, 257, 31, 33, 64, 150, 16, 512, 17]
    ql = [1, 1, 1, 31, 17, 64, 2, 16, 1, 1]
    b = Batch(ctx, ql, nh, nkv, hd, page, DT[dt], seed=hd)
    for which in ("split", "chunks"):
        out, ref = run_attention(ops, b, DT[dt], None, which)
        close(out, ref, DT[dt])


@pytest.mark.parametrize("nh, nkv, hd, page", [(16, 8, 128, 16), (8, 1, 64, 32), (4, 4, 64, 8), (12, 4, 128, 16),
                                                  (6, 1, 64, 16), (8, 2, 128, 64), (32, 2, 64, 16)])
@pytest.mark.parametrize("window", [None, 70])
def test_attention_tensor_core_prefill(ops, nh, nkv, hd, page, window):
    # groups of 1, 2, 3 (not packed), 4, 6, 8 and 16 heads; tile, page and window edges; single tokens as tiles
    assert ops.prefill_heads_per_block(nh, nkv, hd) in (1, 2, 4, 8)
    ctx = [1, 300, 257, 31, 33, 64, 150, 16, 512, 129, 65]
    ql = [1, 1, 1, 31, 17, 64, 2, 16, 130, 129, 64]
    b = Batch(ctx, ql, nh, nkv, hd, page, torch.bfloat16, seed=hd + nh, window=window)
    kinds = ["split", "tensor"] + (["tcgen05", "tcgen05_128"] if ops.prefill_tcgen05_heads_per_block(nh, nkv, hd, page) else [])
    for which in kinds:
        out, ref = run_attention(ops, b, torch.bfloat16, window, which)
        close(out, ref, torch.bfloat16)
    assert ops.prefill_heads_per_block(8, 2, 32) == 0 and ops.prefill_heads_per_block(8, 2, 96) == 0
    assert ops.prefill_tcgen05_heads_per_block(16, 8, 128, 16) == 2 and ops.prefill_tcgen05_heads_per_block(16, 8, 128, 24) == 0


@pytest.mark.parametrize("kind", ["cuda_cores", "tensor_cores", "tensor_cores_tma"])
@pytest.mark.parametrize("nh, nkv, hd, page", [(16, 8, 128, 16), (8, 1, 64, 32), (4, 4, 64, 8), (12, 4, 128, 16),
                                                  (40, 2, 64, 16), (6, 3, 48, 16), (8, 2, 32, 8)])
@pytest.mark.parametrize("window", [None, 200])
def test_attention_decode_kernels_by_name(ops, kind, nh, nkv, hd, page, window):
    # every decode kernel on single tokens: contexts at partition (128) and page edges, groups of 1 to 20 heads
    if kind.startswith("tensor_cores") and hd not in (64, 128):
        pytest.skip("the tensor-core decode kernels take head_dim 64 and 128")
    ctx = [1, 127, 128, 129, 300, 1000, 16, 255, 256, 257, 513]
    b = Batch(ctx, [1] * len(ctx), nh, nkv, hd, page, torch.bfloat16, seed=nh + hd, window=window,
              standout=lambda r, L, n: (L // 2, 0))
    T = b.qkv.shape[0]
    out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ref = torch.empty_like(out)
    args = (nh, nkv, hd, b.pool, page, b.bt, b.meta, hd ** -0.5, window)
    ops.attention_decode(b.qkv, out, *args, kind=kind)
    plain_ops.paged_attention(b.qkv, ref, *args)
    assert not out.isnan().any() and b.meta.error_flag.tolist() == [0, 0, 0, 0]
    close(out, ref, torch.bfloat16)


@pytest.mark.parametrize("nh, nkv, hd, page", [(16, 8, 128, 16), (8, 1, 64, 32), (4, 4, 64, 8), (12, 4, 128, 16),
                                                  (40, 2, 64, 16), (16, 8, 128, 128)])
@pytest.mark.parametrize("window", [None, 200])
@pytest.mark.parametrize("norm, rope, writes", [(True, True, True), (False, True, True), (True, False, True), (True, True, False)])
@pytest.mark.parametrize("form", ["one_tile", "tile_and_half", "two_tiles", "one_tile*2", "one_tile*3", "one_tile*8"])
def test_attention_decode_that_prepares_q_and_the_newest_key_itself(ops, nh, nkv, hd, page, window, norm, rope, writes, form):
    if form == "tile_and_half" and 64 % page:
        pytest.skip("half a partition holds whole pages")
    # "one_tile*n": a block walks n tiles of 128 keys with a running softmax (partitions of 256, 384 and 1,024 keys: the
    # contexts below end before, at and after their edges; with the window the first tiles of a partition are skipped)
    form, _, tiles = form.partition("*")
    tiles = int(tiles or 1)
    # the same batch through (norm, rotation, cache write) as a pass of its own followed by plain attention, and
    # through the decode kernel that does all of it; the newest slots of its cache start as NaN
    ctx = [1, 127, 128, 129, 300, 1000, 16, 255, 256, 257, 513, 384, 385, 1024, 1025]
    b = Batch(ctx, [1] * len(ctx), nh, nkv, hd, page, torch.bfloat16, seed=nh + hd, window=window)
    B = len(ctx)
    L = b.meta.context_lens.tolist()
    pos = torch.tensor([n - 1 for n in L], dtype=torch.int32, device=DEV)
    bt = b.bt.tolist()
    slots = torch.tensor([bt[r][(L[r] - 1) // page] * page + (L[r] - 1) % page for r in range(B)], dtype=torch.int32, device=DEV)
    qw = (1 + 0.1 * rnd(hd, seed=2)) if norm else None
    kw = (1 + 0.1 * rnd(hd, seed=3)) if norm else None
    inv = 1.0 / (5000.0 ** (torch.arange(0, hd, 2).float() / hd))
    fr = torch.outer(torch.arange(1100).float(), inv)
    cs = torch.cat((fr.cos(), fr.sin()), -1).to(DEV) if rope else None
    ref_qkv, ref_pool = b.qkv.clone(), b.pool.clone()
    plain_ops.qk_norm_rope_kv_write(ref_qkv, nh, nkv, hd, qw, kw, 1e-5, cs, pos, slots, ref_pool, page)
    ref = torch.empty(B, nh * hd, dtype=torch.bfloat16, device=DEV)
    args = (nh, nkv, hd)
    plain_ops.paged_attention(ref_qkv, ref, *args, ref_pool, page, b.bt, b.meta, hd ** -0.5, window)
    pool = b.pool.clone()
    if writes:
        for r in range(B):
            s_ = int(slots[r])
            pool[s_ // page, :, :, s_ % page] = float("nan")
    else:
        pool = ref_pool.clone()                      # another layer wrote the newest key and value
    before = pool.clone()
    qkv = b.qkv.clone()
    out = torch.full((B, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.decode_fused_takes(qkv, hd, pool, page, b.meta)
    ops.attention_decode_fused(qkv, out, *args, pool, page, b.bt, b.meta, hd ** -0.5, window, qw, kw, 1e-5, cs,
                               slots if writes else None, form=form, tiles=tiles)
    assert not out.isnan().any() and b.meta.error_flag.tolist() == [0, 0, 0, 0]
    close(out, ref, torch.bfloat16)
    assert torch.equal(qkv, b.qkv)                   # the rows of the product are left alone
    if writes:
        assert torch.equal(pool.isnan(), ref_pool.isnan())
        close(pool.nan_to_num(0), ref_pool.nan_to_num(0), torch.bfloat16, scale=4)
        for r in range(B):                           # the value is copied bit for bit
            s_ = int(slots[r])
            assert torch.equal(pool[s_ // page, 1, :, s_ % page].reshape(-1), qkv[r, (nh + nkv) * hd:])
    else:
        assert torch.equal(pool.nan_to_num(7), before.nan_to_num(7))


def test_how_many_key_tiles_a_block_of_decode_attention_walks(ops):
    # the rule of ops.decode_tiles_for: one tile while single tiles make no more blocks than the device holds at once, then
    # the largest power of two (up to 32, and less than the context's tiles: two partitions at least) that still leaves that many blocks
    want = 4 * ops.sm_count()
    assert ops.decode_tiles_for(8 * 8, 9) == 1                       # 8 requests x 8 key/value heads at 1,100 tokens
    assert ops.decode_tiles_for(10 ** 6, 1) == 1                     # a context of one tile has nothing to walk
    assert ops.decode_tiles_for(8, 64) == 4 and ops.decode_tiles_for(8, 235) == 4     # one request, 8,192 / 30,000 tokens
    assert ops.decode_tiles_for(8, 40) == 2 and ops.decode_tiles_for(8, 20) == 1        # (four tiles a block would leave 80 blocks; 2,560 tokens are not long)
    for rows, key_tiles in ((512, 9), (512, 17), (512, 33), (2048, 9), (128, 9), (256, 9), (128, 16), (4096, 400)):
        t = ops.decode_tiles_for(rows, key_tiles)
        assert t in (1, 2, 4, 8, 16, 32) and (t == 1 or t < key_tiles)
        if t > 1 and not (key_tiles > 32 and t <= 4):
            assert rows * -(-key_tiles // t) >= want                 # enough blocks are left
        if t < 32 and 2 * t < key_tiles and not (key_tiles > 32 and t <= 4):
            assert rows * -(-key_tiles // (2 * t)) < want            # and twice as many tiles would leave too few


@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["split", "chunks", "tensor", "tcgen05"])
def test_attention_finds_one_far_key_among_hundreds(ops, dt, which):
    if which in ("tensor", "tcgen05") and dt != "bfloat16":
        pytest.skip("the tensor-core kernels are bfloat16 only")
    # one key far back gets a score that stands out: the output must be (nearly) its value
    ctx, ql = [700, 1000, 520, 300], [1, 1, 40, 16]
    far = {0: 3, 1: 511, 2: 256, 3: 15}                                  # page edges, partition edges, the start
    b = Batch(ctx, ql, 8, 2, 64, 16, DT[dt], seed=1, standout=lambda r, L, n: (far[r], n - 1))
    out, ref = run_attention(ops, b, DT[dt], None, which)
    close(out, ref, DT[dt])
    cu = b.meta.cu_seqlens.tolist()
    for r in range(4):                                                     # and it really dominates
        row = cu[r + 1] - 1
        j = far[r]
        v = b.pool[b.bt[r, j // 16].long(), 1, 0, j % 16].float()
        assert (ref[row, :64].float() - v).abs().max() < 0.05


@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["split", "chunks", "tensor", "tcgen05"])
@pytest.mark.parametrize("edge", [0, 1])
def test_attention_window_edge(ops, dt, which, edge):
    if which in ("tensor", "tcgen05") and dt != "bfloat16":
        pytest.skip("the tensor-core kernels are bfloat16 only")
    # the standout key sits exactly at the window's edge (edge=0: last key still seen, edge=1: first not seen)
    w = 40
    ctx, ql = [300, 130, 97], [1, 30, 1]

    def stand(r, L, n):
        p = L - 1                                                          # position of the request's last query
        return (p - w + 1 - edge, n - 1)
    b = Batch(ctx, ql, 4, 2, 64, 8, DT[dt], seed=2, standout=stand, window=w)
    out, ref = run_attention(ops, b, DT[dt], w, which)
    close(out, ref, DT[dt])
    cu = b.meta.cu_seqlens.tolist()
    for r in range(3):
        row = cu[r + 1] - 1
        j = b.ctx_lens[r] - 1 - w + 1 - edge
        page = b.bt[r, j // 8].long()
        if edge == 0:
            assert (ref[row, :64].float() - b.pool[page, 1, 0, j % 8].float()).abs().max() < 0.05
        # edge == 1: the key is outside; its page may even be given back (NaN there would show)


@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
def test_attention_does_not_depend_on_the_batch(ops, dt):
    # the same requests alone and among others (same pages, same tokens): bit-identical rows
    from mini_engine_b200.engine.step_context import AttnMeta
    ctx, ql = [300, 77, 150, 90], [1, 20, 1, 90]
    many = Batch(ctx, ql, 8, 2, 64, 16, DT[dt], seed=3)                   # batch order: 300/1, 150/1, 77/20, 90/90
    out_many, _ = run_attention(ops, many, DT[dt], None)
    cu = many.meta.cu_seqlens.tolist()
    for b in (0, 2, 3):
        n, L = many.q_lens[b], many.ctx_lens[b]
        def tl(tq):
            t = [(0, q0) for q0 in range(0, n, tq)] if n > 1 else []
            return torch.tensor(t or [(0, 0)], dtype=torch.int32, device=DEV), len(t)
        meta = AttnMeta(num_reqs=1, num_tokens=n, num_decodes=1 if n == 1 else 0,
                        cu_seqlens=torch.tensor([0, n], dtype=torch.int32, device=DEV),
                        context_lens=torch.tensor([L], dtype=torch.int32, device=DEV),
                        tile_lists={tq: tl(tq) for tq in ops.ATTN_TILE_SIZES}, num_tiles=1 if n > 1 else 0,
                        max_context_len=L, workspace=many.meta.workspace, error_flag=many.meta.error_flag)
        qkv = many.qkv[cu[b]:cu[b + 1]].clone()
        out = torch.full((n, 8 * 64), float("nan"), dtype=DT[dt], device=DEV)
        ops.paged_attention(qkv, out, 8, 2, 64, many.pool, 16, many.bt[b:b + 1].clone(), meta, 64 ** -0.5, None)
        assert torch.equal(out, out_many[cu[b]:cu[b + 1]]), f"request {b}"


# ---- sampling -------------------------------------------------------------------------------
def test_sample(ops):
    S, V = 6, 5003
    logits = rnd(S, V, seed=9, scale=2.0)
    temps = torch.tensor([0.0, 0.7, 1.0, 0.0, 1.5, 0.3], device=DEV)
    seeds = torch.tensor([1, 2, 3, 4, 5, 6], dtype=torch.int32, device=DEV)
    pos = torch.tensor([10, 11, 12, 13, 14, 2 ** 20], dtype=torch.int32, device=DEV)
    out = torch.empty(S, dtype=torch.int32, device=DEV)
    ops.sample(logits, temps, seeds, pos, out)
    got = out.tolist()
    for r in range(S):
        keys = plain_ops.sample_keys(logits[r], float(temps[r]), int(seeds[r]), int(pos[r]))
        assert keys[got[r]] >= keys.max() - 1e-4, f"row {r}"
        if float(temps[r]) == 0:
            assert got[r] == int(np.argmax(keys))
    # a vocabulary of many pieces, keys of every size: the kernel takes exact keys only for the entries whose rough
    # keys come near the best, which must never lose the winner; flat rows make thousands of near-ties
    S2, V2 = 8, 151936
    big = rnd(S2, V2, seed=11, scale=3.0)
    big[6:] = 0.25
    temps2 = torch.tensor([0.01, 0.05, 0.6, 1.0, 8.0, 100.0, 0.7, 1e-3], device=DEV)
    seeds2 = torch.arange(21, 21 + S2, dtype=torch.int32, device=DEV)
    pos2 = torch.arange(5, 5 + S2, dtype=torch.int32, device=DEV)
    out_big = torch.empty(S2, dtype=torch.int32, device=DEV)
    ops.sample(big, temps2, seeds2, pos2, out_big)
    for r, g in enumerate(out_big.tolist()):
        keys = plain_ops.sample_keys(big[r], float(temps2[r]), int(seeds2[r]), int(pos2[r]))
        assert np.isfinite(keys).all() and keys[g] >= keys.max() - 1e-4 * max(1.0, abs(keys.max()) * 1e-3), f"row {r}"
    # the draw does not depend on the row's place in the batch
    out2 = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.sample(logits[4:5], temps[4:5], seeds[4:5], pos[4:5], out2)
    assert out2.item() == got[4]
    # ties go to the lower index
    flat = torch.zeros(2, 100, device=DEV)
    ops.sample(flat, torch.zeros(2, device=DEV), seeds[:2], pos[:2], out[:2])
    assert out[:2].tolist() == [0, 0]
