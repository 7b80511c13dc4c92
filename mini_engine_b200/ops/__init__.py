"""Python side of the CUDA kernels: loads the library and checks arguments before a launch.

Every function here runs a hand-written sm_100a kernel of ``csrc/`` on the current CUDA
stream.  There is no other implementation behind them: without the library (no nvcc, no
GPU) they raise.  The reference builds its kernels with torch's JIT at import
(layers/ops.py:5-18); here the build is a plain nvcc run at the first call.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build

ATTN_TILE_Q = 16          # query tokens per block of the CUDA-core chunk kernel (csrc/attention_chunk.cu)
ATTN_TILE_SIZES = (8, 16, 32, 64, 128)   # query tokens per block that some attention kernel may ask for
DECODE_PARTITION = 128    # keys per partition of the decode kernel (csrc/attention_decode.cu)
MAX_HEAD_DIM = 256

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
_PROTOS = {
    "me_embed": [_P, _P, _I, _P, _I, _I, _I, _P, _P, _I, _P],
    "me_add_rmsnorm": [_P, _P, _I, _P, _F, _P, _I, _P, _I, _I, _I, _L, _P],
    "me_gemm_skinny": [_P, _L, _P, _P, _I, _L, _P, _I, _I, _I, _I, _P],
    "me_silu_mul": [_P, _P, _I, _I, _I, _P],
    "me_gemm_simt": [_P, _I, _L, _P, _I, _P, _I, _L, _I, _I, _I, _I, _P],
    "me_qk_norm_rope_kv_write": [_P, _I, _L, _I, _I, _I, _I, _P, _P, _F, _P, _I, _P, _P, _P, _I, _P],
    "me_attn_chunk": [_P, _I, _L, _P, _L, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    "me_attn_decode": [_P, _I, _L, _P, _L, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P, _P, _I, _P, _I, _P, _P],
    "me_attn_decode_fused": [_P, _L, _P, _L, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P, _F, _P, _P, _P, _P, _P,
                             _I, _I, _I, _P, _P],
    "me_gemm_decode": [_I, _P, _L, _P, _I, _F, _P, _P, _I, _L, _P, _P, _P, _P, _I, _I, _I, _P, ctypes.c_uint64, _P],
    "me_gemm_stream": [_I, _P, _P, _I, _F, _P, _P, _I, _L, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P],
    "me_gemm_tcgen05": [_P, _P, _P, _I, _L, _I, _I, _I, _I, _I, _I, _L, _P, _P],
    "me_gemm_tcgen05_persistent": [_P, _P, _P, _I, _L, _I, _I, _I, _I, _I, _P, _P],
    "me_gemm_tcgen05_shared": [_P, _P, _P, _I, _L, _I, _I, _I, _I, _I, _P, _P, _P, _P],
    "me_attn_prefill_tcgen05": [_P, _P, _P, _L, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "me_tma_encode_2d": [_P, _P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, _I],
    "me_attn_prefill": [_P, _L, _P, _L, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
    "me_sample": [_P, _L, _P, _P, _P, _P, _I, _I, _P, _P, _P],
    "me_test_wait_expires": [_P, _I, _P, _P],
}
_DT = {torch.float32: 0, torch.bfloat16: 1}

_lib: Optional[ctypes.CDLL] = None
launches = 0              # kernels launched through this module (counted for the benchmark)


class KernelError(RuntimeError):
    pass


def require_extension() -> ctypes.CDLL:
    """The loaded kernel library; builds it at the first call; raises if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    if not torch.cuda.is_available():
        raise KernelError("mini_engine_b200 needs a CUDA device: its kernels have no CPU path")
    path = _build.library_path()
    lib = ctypes.CDLL(path)
    lib.me_last_error.restype = ctypes.c_char_p
    for name, args in _PROTOS.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    if lib.me_attn_chunk_tile_q() != ATTN_TILE_Q or lib.me_attn_decode_partition() != DECODE_PARTITION:
        raise KernelError("the kernel library and ops/__init__.py disagree on tile sizes")
    lib.me_attn_prefill_heads_per_block.argtypes = [_I, _I, _I]
    lib.me_attn_prefill_tcgen05_heads_per_block.argtypes = [_I, _I, _I, _I]
    lib.me_sample_chunks.argtypes = [_I]
    lib.me_gemm_tcgen05_splits.argtypes = [_I, _I]
    lib.me_gemm_decode_sumsq_parts.argtypes = [_I]
    lib.me_gemm_stream_sumsq_parts.argtypes = [_I, _I]
    lib.me_gemm_stream_x_box_rows.argtypes = [_I]
    lib.me_gemm_stream_w_box_rows.argtypes = [_I]
    lib.me_attn_decode_fused_takes.argtypes = [_I, _I]
    lib.me_gemm_skinny_splits.argtypes = [_I]
    _lib = lib
    return lib


def set_programmatic_launch(on: bool) -> None:
    """Switch programmatic dependent launch (a kernel may start, and fetch weights, while its predecessor
    still runs) on or off for all later launches; it is on by default."""
    (_lib or require_extension()).me_set_pdl(1 if on else 0)


def library_file() -> str:
    require_extension()
    return _lib._name


_fns: dict = {}
_last_call = None         # (entry point, arguments) of the launch before

# Per-kernel timing for the benchmark's roofline table: while ``timeline`` is a list, every launch made through
# this module is bracketed by two CUDA events and recorded as (tag, entry point, start, end).  ``tag`` is set by
# the caller that knows what the launch is for (a Linear part sets it to its output's name).  An event between
# two launches keeps the second from starting under the first (programmatic dependent launch), so these are the
# times of kernels run one after the other, not shares of a step replayed from a graph.
timeline: Optional[list] = None
tag = ""


class _Timed:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if timeline is not None:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if timeline is not None:
            self.e1.record()
            timeline.append((tag, self.name, self.e0, self.e1))


def _call(name: str, *args) -> None:
    global launches, _last_call
    fn = _fns.get(name)
    if fn is None:
        fn = _fns[name] = getattr(_lib or require_extension(), name)
    if timeline is not None:
        with _Timed(name):
            rc = fn(*args)
    else:
        rc = fn(*args)
    if rc != 0:
        raise KernelError(_lib.me_last_error().decode())
    launches += 1
    _last_call = (fn, args)


# The same product or norm comes back step after step with the same tensors (the work buffers of a step are the
# same storage every time): a wrapper that finds its key here, with the same addresses, shapes and strides as when
# it was made, launches at once with the arguments of that time (and the stream of now) instead of checking and
# deciding everything again.  An eager step spends more host time on that than on the launches themselves.
_repeats: dict = {}
remember_launches = True  # False: every wrapper runs in full every time (a switch for comparisons)


def _repeat(key, sig) -> bool:
    global launches
    hit = _repeats.get(key) if remember_launches and timeline is None else None
    if hit is None or hit[0] != sig:
        return False
    if hit[1](*hit[2], _stream()) != 0:
        raise KernelError(_lib.me_last_error().decode())
    launches += 1
    return True


def _remember(key, sig, launches_before: int) -> None:
    """After a wrapper has run in full: keep its launch if it was exactly one, with the stream as last argument."""
    if launches == launches_before + 1 and _last_call is not None and _last_call[1][-1] == _stream():
        if len(_repeats) > 16384:
            _repeats.clear()
        _repeats[key] = (sig, _last_call[0], _last_call[1][:-1])


def forget_tensors() -> None:
    """Drop everything remembered about tensors seen so far (launch arguments, tensor maps): for a process that
    frees one engine and builds another."""
    _repeats.clear()
    _tensor_maps.clear()


_device_index: Optional[int] = None


def _stream() -> int:
    """The current stream's handle (a launch a few microseconds apart cannot afford torch's Stream object)."""
    global _device_index
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(_device_index)


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


_sm_count = 0


def sm_count() -> int:
    """Multiprocessors of the current device."""
    global _sm_count
    if not _sm_count:
        _sm_count = int((_lib or require_extension()).me_device_sm_count())
    return _sm_count


def wait_expires_selftest(err: torch.Tensor, limit: int = 4096) -> int:
    """Runs the kernel of csrc/selftest.cu: a bounded wait on a barrier that nothing completes.  It sets flag 1 of
    ``err`` (int32[4] on the device) as the tensor-map kernels do when a wait runs out; returns the polls made."""
    _need(err.dtype == torch.int32 and err.numel() >= 4 and err.is_cuda, "wait_expires_selftest: err must be int32[4] on the device")
    polls = torch.zeros(1, dtype=torch.int32, device=err.device)
    _call("me_test_wait_expires", err.data_ptr(), int(limit), polls.data_ptr(), _stream())
    return int(polls.item())


def check_attention_sizes(head_dim: int, num_heads: int, num_kv_heads: int) -> None:
    """What the attention kernels take; anything else is refused here, before any launch."""
    if head_dim % 16 or not 16 <= head_dim <= MAX_HEAD_DIM:
        raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take multiples "
                         f"of 16 from 16 to {MAX_HEAD_DIM}")
    if num_heads < 1 or num_kv_heads < 1 or num_heads % num_kv_heads:
        raise ValueError(f"{num_heads} heads with {num_kv_heads} key/value heads is not supported")


# ---- element-wise and normalisation ----------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor,
          feedback: Optional[torch.Tensor] = None) -> None:
    """Rows of ``table`` into the float32 ``out``.  An id ~j (negative) stands for ``feedback[j]`` (int32 on the
    device: the tokens the step before drew); ids outside the vocabulary set flag 0 of ``err``."""
    _need(ids.dtype == torch.int32 and ids.is_contiguous(), "embed: token ids must be contiguous int32")
    _need(feedback is None or (feedback.dtype == torch.int32 and feedback.is_contiguous()), "embed: feedback must be int32")
    _need(out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous(), "embed: bad tensors")
    T, (V, H) = ids.shape[0], table.shape
    _need(tuple(out.shape) == (T, H), "embed: output shape")
    _call("me_embed", ids.data_ptr(), table.data_ptr(), _dt(table), out.data_ptr(), T, H, V, err.data_ptr(), _ptr(feedback),
          feedback.numel() if feedback is not None else 0, _stream())


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """``residual += delta`` (float32, in place), ``out = rmsnorm(residual) * weight``; with ``rows``
    only those rows are read and ``residual`` is not written.  A 3-D ``delta`` [splits, T, H] holds the
    partial results of a split-K product; they are added in order."""
    key = ("add_rmsnorm", id(residual), id(delta), id(weight), id(out), id(rows))
    sig = (residual.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), _ptr(rows), residual.shape, residual.stride(),
           residual.dtype, None if delta is None else (delta.shape, delta.stride(), delta.dtype), weight.shape, weight.dtype,
           out.shape, out.stride(), out.dtype, None if rows is None else (rows.shape, rows.stride(), rows.dtype), eps)
    if _repeat(key, sig):
        return
    before = launches
    H = residual.shape[1]
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: residual must be float32")
    _need(weight.dtype == torch.float32 and weight.shape == (H,), "add_rmsnorm: weight must be float32 [H]")
    n = residual.shape[0] if rows is None else rows.shape[0]
    _need(out.is_contiguous() and tuple(out.shape) == (n, H), "add_rmsnorm: output shape")
    splits, stride = 1, 0
    if delta is not None:
        if delta.dim() == 3:                      # partial results of a split-K product: [splits, T, H]
            splits, stride = delta.shape[0], delta.stride(0)
            _need(delta.is_contiguous() and tuple(delta.shape[1:]) == tuple(residual.shape), "add_rmsnorm: delta shape")
        else:
            _need(delta.is_contiguous() and delta.shape == residual.shape, "add_rmsnorm: delta shape")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.is_contiguous(), "add_rmsnorm: rows must be int32")
    _call("me_add_rmsnorm", residual.data_ptr(), _ptr(delta), _dt(delta) if delta is not None else 0,
          weight.data_ptr(), float(eps), out.data_ptr(), _dt(out), _ptr(rows), n, H, splits, stride, _stream())
    _remember(key, sig, before)


def silu_mul(x: torch.Tensor, out: torch.Tensor) -> None:
    T, I2 = x.shape
    _need(I2 % 2 == 0 and tuple(out.shape) == (T, I2 // 2) and x.dtype == out.dtype, "silu_mul: shapes")
    _need(x.is_contiguous() and out.is_contiguous(), "silu_mul: contiguous tensors")
    _call("me_silu_mul", x.data_ptr(), out.data_ptr(), _dt(x), T, I2 // 2, _stream())


# ---- matrix products ----------------------------------------------------------------------
library_calls = 0         # cuBLAS products issued through torch (not counted as this package's kernels)


SKINNY_MAX_ROWS = 16      # rows up to which bfloat16 products run csrc/gemm_skinny.cu


def skinny_splits(M: int, K: int, x: torch.Tensor, weight: torch.Tensor) -> int:
    """How many float32 partial results the small-batch kernel would leave for this product
    (0: the kernel does not take it; 1: it writes the result itself)."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 0 < M <= SKINNY_MAX_ROWS
            and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0):
        return 0
    return (_lib or require_extension()).me_gemm_skinny_splits(K)


def linear_partials(x: torch.Tensor, weight: torch.Tensor, workspace, name: str,
                    err: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``x @ weight.T`` as float32 partial results [splits, M, N] of a split-K product, for a consumer that
    adds them (``add_rmsnorm``); None when the product is not one that is split: the small-batch kernel splits long
    rows of few requests, the tcgen05 kernel products of a few hundred rows whose tiles would leave most SMs idle.
    ``err``: the int32[4] error word of the step (the tcgen05 kernel reports a wait that ran out there); without it
    the tcgen05 kernel is not used."""
    M, K = x.shape
    N = weight.shape[0]
    splits = skinny_splits(M, K, x, weight)
    if splits >= 2:
        part = workspace(name, (splits, M, N), torch.float32)
        _call("me_gemm_skinny", x.data_ptr(), x.stride(0), weight.data_ptr(), 0, 0, 0, part.data_ptr(), M, N, K, 0, _stream())
        return part
    if err is not None and use_tcgen05_gemm and tcgen05_takes(x, weight) and weight.is_contiguous():
        bn, parts = tcgen05_split_plan(M, N, K)
        if parts >= 2:
            part = workspace(name, (parts, M, N), torch.float32)
            linear_tcgen05(x, weight, part, "none", err, tile_n=bn, splits=parts)
            return part
    return None


DECODE_MAX_K = 3072       # largest K of csrc/gemm_decode.cu (one block covers all of K); beyond: csrc/gemm_stream.cu
# Which of the two kernels a decode product runs: "auto" (gemm_decode up to DECODE_MAX_K, gemm_stream beyond),
# "stream" (gemm_stream for every K) or "decode" (gemm_decode only; larger K is then not taken).  A switch for comparisons.
decode_kernel = "auto"


def _decode_uses_stream(K: int) -> bool:
    return decode_kernel == "stream" or (decode_kernel == "auto" and K > DECODE_MAX_K)


# Which products over a K beyond DECODE_MAX_K run csrc/gemm_stream.cu: "all", or "residual" (only those that add into
# the residual stream; the others go to the library).  A switch for comparisons.
stream_products = "all"
# Weights from this many elements on (32 MB of bfloat16: the LM head) go through csrc/gemm_stream.cu in ``linear`` too
# when the batch has up to 16 rows: a product that long is all stream, and that kernel streams fastest.
STREAM_MIN_WEIGHT_ELEMENTS = 1 << 24


def _decode_operands_ok(M: int, K: int, weight: torch.Tensor) -> bool:
    return (weight.is_cuda and weight.dtype == torch.bfloat16 and 0 < M <= SKINNY_MAX_ROWS and K % 8 == 0
            and weight.data_ptr() % 16 == 0)


def decode_linear_takes(M: int, K: int, weight: torch.Tensor, adds_to_residual: bool = True) -> bool:
    """Whether a decode product with norm / residual folded in (csrc/gemm_decode.cu, csrc/gemm_stream.cu: up to 16
    rows) takes the shape; ``adds_to_residual``: the product is one whose result is added to the residual stream."""
    if not _decode_operands_ok(M, K, weight):
        return False
    if _decode_uses_stream(K):
        return decode_kernel == "stream" or stream_products == "all" or adds_to_residual
    return K <= DECODE_MAX_K


_stream_ws: dict = {}


def _stream_work_buffers(device) -> tuple[torch.Tensor, torch.Tensor]:
    """What csrc/gemm_stream.cu needs beside its operands: room for the sums a block leaves to the block that finishes its
    group of rows, and a flag a block (zero between launches).  One pair a device: launches in one stream never overlap."""
    ws = _stream_ws.get(device)
    if ws is None:
        lib = _lib or require_extension()
        ws = _stream_ws[device] = (torch.empty(lib.me_gemm_stream_partial_floats(), dtype=torch.float32, device=device),
                                   torch.zeros(lib.me_gemm_stream_flag_ints(), dtype=torch.int32, device=device))
    return ws


_shared_ws: dict = {}


def _tcgen05_shared_buffers(device) -> tuple[torch.Tensor, torch.Tensor]:
    """The same for the work-sharing form of csrc/gemm_tcgen05.cu: a 128 x 256 tile of float32 sums a block, four flags a block."""
    ws = _shared_ws.get(device)
    if ws is None:
        lib = _lib or require_extension()
        ws = _shared_ws[device] = (torch.empty(lib.me_gemm_tcgen05_shared_partial_floats(), dtype=torch.float32, device=device),
                                   torch.zeros(lib.me_gemm_tcgen05_shared_flag_ints(), dtype=torch.int32, device=device))
    return ws


def reset_stream_work_buffers() -> None:
    """Clear the flags of the work buffers of csrc/gemm_stream.cu and of the work-sharing tcgen05 product.  Every launch
    leaves them zero, except one whose bounded wait ran out (flag 1 of the error word): the caller that reports that
    error calls this, so that a later launch does not take a stale flag for a neighbour's finished sums."""
    for _, flags in list(_stream_ws.values()) + list(_shared_ws.values()):
        flags.zero_()


def decode_linear_sumsq_parts(N: int, K: int = 0, stream: Optional[bool] = None) -> int:
    """Parts in which the residual epilogue of ``decode_linear`` writes sums of squares, for N columns over K
    (``stream``: by which of the two kernels; None: the one that ``decode_kernel`` picks for K)."""
    lib = _lib or require_extension()
    stream = _decode_uses_stream(K) if stream is None else stream
    return lib.me_gemm_stream_sumsq_parts(N, K) if stream else lib.me_gemm_decode_sumsq_parts(N)


def decode_linear(weight: torch.Tensor, x: torch.Tensor, *, out: Optional[torch.Tensor] = None, epilogue: str = "none",
                  row_scale=None, residual_out: Optional[torch.Tensor] = None, sumsq_out: Optional[torch.Tensor] = None,
                  next_norm=None, fetch_ahead: Optional[torch.Tensor] = None, err: Optional[torch.Tensor] = None,
                  kernel: Optional[str] = None) -> None:
    """One decode product with its neighbours folded in (csrc/gemm_decode.cu, csrc/gemm_stream.cu; ``kernel``:
    "stream" asks for the latter whatever ``decode_kernel`` says).

    ``x``: bfloat16 [M, K].  ``row_scale`` = (sums of squares float32 [parts, M], eps): x is a residual times a
    norm's weight, and the float32 results of row m are multiplied by rsqrt(sum / K + eps), which completes that
    RMSNorm.  Output: ``out`` (epilogue "none" or "silu_mul") or ``residual_out`` (float32 [M, N], epilogue
    "residual": residual_out += x W^T; ``sumsq_out`` [decode_linear_sumsq_parts(N), M] gets the new residual's sums
    of squares per strip of columns, and with ``next_norm`` = (weight float32 [N], xw bfloat16 [M, N]) xw gets the new
    residual times that weight).  ``fetch_ahead``: a tensor that a later kernel reads (the next product's weight);
    this kernel asks it into L2."""
    epi = {"none": 0, "silu_mul": 1, "residual": 2}[epilogue]
    M, K = x.shape
    _need(x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0, "decode_linear: x")
    stream = kernel == "stream" or _decode_uses_stream(K)
    _need((stream or K <= DECODE_MAX_K) and _decode_operands_ok(M, K, weight) and weight.shape[1] == K
          and weight.is_contiguous(), "decode_linear: shape not taken")
    sumsq, eps = row_scale if row_scale is not None else (None, 0.0)
    if sumsq is not None:
        _need(sumsq.dtype == torch.float32 and sumsq.is_contiguous() and sumsq.dim() == 2 and sumsq.shape[1] == M,
              "decode_linear: sums of squares")
    N = weight.shape[0] // 2 if epi == 1 else weight.shape[0]
    nw, xw = next_norm if next_norm is not None else (None, None)
    if epi == 2:
        _need(residual_out.dtype == torch.float32 and residual_out.is_contiguous() and tuple(residual_out.shape) == (M, N)
              and sumsq_out.dtype == torch.float32 and sumsq_out.is_contiguous()
              and tuple(sumsq_out.shape) == (decode_linear_sumsq_parts(N, K, stream), M), "decode_linear: residual output")
        if nw is not None:
            _need(nw.dtype == torch.float32 and tuple(nw.shape) == (N,) and nw.is_contiguous() and xw.dtype == torch.bfloat16
                  and tuple(xw.shape) == (M, N) and xw.is_contiguous(), "decode_linear: pre-weighted output")
        yp, ydt, ldy = 0, 0, 0
    else:
        _need(next_norm is None, "decode_linear: the pre-weighted output belongs to the residual epilogue")
        _need(tuple(out.shape) == (M, N) and out.stride(1) == 1, "decode_linear: output shape")
        yp, ydt, ldy = out.data_ptr(), _dt(out), out.stride(0)
    if stream:
        _need(err is not None, "decode_linear: the streaming kernel needs the step's error word (err=)")
        lib = _lib or require_extension()
        partials, flags = _stream_work_buffers(x.device)
        _call("me_gemm_stream", epi, matrix_tensor_map(x, lib.me_gemm_stream_x_box_rows(M)).ptr, _ptr(sumsq),
              sumsq.shape[0] if sumsq is not None else 0, float(eps), matrix_tensor_map(weight, lib.me_gemm_stream_w_box_rows(epi)).ptr, yp, ydt, ldy,
              _ptr(residual_out), _ptr(sumsq_out), _ptr(nw), _ptr(xw), M, N, K, partials.data_ptr(), flags.data_ptr(),
              err.data_ptr(), _stream())
        return
    _call("me_gemm_decode", epi, x.data_ptr(), x.stride(0), _ptr(sumsq), sumsq.shape[0] if sumsq is not None else 0, float(eps),
          weight.data_ptr(), yp, ydt, ldy, _ptr(residual_out), _ptr(sumsq_out), _ptr(nw), _ptr(xw), M, N, K,
          _ptr(fetch_ahead), fetch_ahead.numel() * fetch_ahead.element_size() if fetch_ahead is not None else 0, _stream())


TCGEN05_MIN_ROWS = 128    # rows from which bfloat16 products run csrc/gemm_tcgen05.cu whatever the weight (fewer: cuBLAS) ...
# ... and from 48 rows on where the weight is small (up to 8 M elements: every product of a layer at the 0.6B sizes).  There a
# decode step of 64 requests takes 2.39 ms against 2.44 with the library's products and a SiLU kernel, one of 96 requests 3.36
# against 3.50 (32 requests: level); at the 8B and 32B sizes, where such a product streams 30 to 260 MB of weights over a
# half-empty tile of rows, the library is 5 to 12% ahead and keeps them.
TCGEN05_SMALL_MIN_ROWS = 48
TCGEN05_SMALL_MAX_WEIGHT_ELEMENTS = 8 << 20
use_tcgen05_gemm = True   # False: such products go to cuBLAS instead (a switch for comparisons)


def tcgen05_min_rows(weight_elements: int) -> int:
    """Rows from which a product with a weight of that many elements runs the tcgen05 kernels."""
    return min(TCGEN05_MIN_ROWS, TCGEN05_SMALL_MIN_ROWS) if weight_elements <= TCGEN05_SMALL_MAX_WEIGHT_ELEMENTS else TCGEN05_MIN_ROWS


def matrix_tensor_map(t: torch.Tensor, box_rows: int) -> "TensorMap":
    """The tensor map of a row-major bfloat16 matrix [rows, cols] (row pitch ``t.stride(0)``) with boxes of
    ``box_rows`` x 64 columns and the 128-byte swizzle; cached by address and shape."""
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows)
    tm = _tensor_maps.get(key)
    if tm is None:
        if len(_tensor_maps) > 8192:
            _tensor_maps.clear()
            _repeats.clear()          # remembered launches hold the addresses of the maps just dropped
        tm = TensorMap()
        lib = _lib or require_extension()
        if lib.me_tma_encode_2d(tm.ptr, t.data_ptr(), t.shape[0], t.shape[1], t.stride(0) * 2, box_rows, 64, 128) != 0:
            raise KernelError(lib.me_last_error().decode())
        _tensor_maps[key] = tm
    return tm


def tcgen05_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    M, K = x.shape
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M >= tcgen05_min_rows(weight.numel())
            and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


tcgen05_persistent = "auto"     # the persistent form of the tcgen05 product: "auto", True or False (for comparisons)


def tcgen05_persistent_pays(M: int, N: int, K: int, epi: int) -> bool:
    """Whether a product of M rows and N output columns runs the persistent form of the tcgen05 kernel (one block an
    SM walking 128 x 256 tiles with two accumulators): from two tiles an SM on (a little earlier where K is short and a
    tile's fixed part weighs more: q|k|v of 2,048 rows at the 0.6B sizes).  There the loads of the next tile and
    the epilogue of the last one run beside a tile's products, which is worth a fifth to a third of gate|up at every
    size measured and of q|k|v at 2,048 rows; with fewer tiles (o_proj, down_proj up to a few thousand rows) the form
    with two blocks an SM is level or ahead."""
    out_cols = 128 if epi else 256
    tiles = ((M + 127) // 128) * ((N + out_cols - 1) // out_cols)
    return tiles >= 2 * sm_count() or (K <= 1024 and 10 * tiles >= 17 * sm_count())


tcgen05_share = "auto"          # the work-sharing form of the tcgen05 product: "auto" or False (for comparisons)


def tcgen05_share_pays(M: int, N: int, K: int, epi: int) -> bool:
    """Whether a product of M rows and N output columns runs the work-sharing form of the tcgen05 kernel (the last
    rounds' stages cut into one equal range an SM, partial sums added by the tile's owner).  It pays where whole tiles
    leave SMs idle: a last round that is less than half full (1.1 or 2.2 tiles of 128 x 256 an SM: q|k|v of 1,024 rows at
    the 8B sizes 52 against 66 us, o_proj of 1,024 rows at the 32B sizes 79 against 124), or fewer tiles than SMs with a
    long K and up to 512 rows (q|k|v of 256 rows at the 32B sizes 55 against 75 us, down_proj of 512 rows at the 8B sizes
    74 against 90).  It does not pay with the SiLU epilogue (many tiles anyway), nor where the blocks that share a tile of
    W, now at different places along K, push each other's part of it out of L2: down_proj of 1,024 rows at the 8B sizes
    (eight tiles to a tile of W, 128 tiles for 148 SMs) took 124 against 90 us and read 670 MB from DRAM for operands of
    126 MB; hence the bound on the rows there, and on the operands' bytes where there are more tiles than SMs (wins were
    measured up to 117 MB: q|k|v of 512 and 1,024 rows at the 32B sizes 61 against 97 and 117 against 134 us)."""
    if epi:
        return False
    sms = sm_count()
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    if tiles >= sms:
        # (K: handing a tile's sums over costs 3 to 5 us, a tile of K = 1,024 takes 5: at the 0.6B sizes it never paid)
        rounds = -(-tiles // sms)
        return K >= 4096 and tiles <= 0.75 * rounds * sms and (M + N) * K * 2 <= 128 << 20
    return 5 * tiles >= sms and K >= 5120 and M <= 512


def tcgen05_one_round_width(M: int, N: int) -> int:
    """The tile width (256 or 128) at which a product of M rows and N columns has about one tile an SM, or 0."""
    sms, m_tiles = sm_count(), (M + 127) // 128
    if 0.85 * sms <= m_tiles * ((N + 255) // 256) <= sms:
        return 256
    if 0.8 * sms <= m_tiles * ((N + 127) // 128) < 2 * sms:
        return 128
    return 0


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str, err: torch.Tensor,
                   tile_n: Optional[int] = None, splits: int = 1, persistent: Optional[bool] = None,
                   share: Optional[bool] = None) -> None:
    """The tcgen05 product of csrc/gemm_tcgen05.cu: TMA -> swizzled shared memory -> tcgen05.mma -> tensor memory.

    With ``splits`` > 1 ``out`` is float32 [tcgen05_splits(K, splits), M, N]: partial results over parts of K.
    ``share``: the form that cuts the stages of all tiles into one equal range an SM (``tile_n`` 128 or 256)."""
    M, K = x.shape
    epi = {"none": 0, "silu_mul": 1}[epilogue]
    N = weight.shape[0] // 2 if epi else weight.shape[0]
    if share is None and tile_n is None and persistent is None and splits == 1 and tcgen05_share == "auto" and tcgen05_takes(x, weight):
        share = tcgen05_share_pays(M, N, K, epi)
    if share:
        bn = tile_n or 256
        _need(tcgen05_takes(x, weight) and splits == 1 and bn in (128, 256), "linear_tcgen05: operands not taken by the work-sharing form")
        partials, flags = _tcgen05_shared_buffers(x.device)
        _call("me_gemm_tcgen05_shared", matrix_tensor_map(x, 128).ptr, matrix_tensor_map(weight, bn // 2 if epi else bn).ptr,
              out.data_ptr(), _dt(out), out.stride(0), M, N, K, epi, bn, partials.data_ptr(), flags.data_ptr(), err.data_ptr(), _stream())
        return
    if tile_n is None:
        # The widest accumulator that still leaves enough tiles: about two an SM where a tile is short (K up to 3,072),
        # one for every other SM where it is long (measured at the 8B and 32B sizes: with 512 rows the 256-wide tile is a
        # third faster than the 64-wide one that two tiles an SM would ask for).  The SiLU epilogue (half as many output
        # columns per tile) does best at 128 while both the rows and K are few, and again where the output is so large
        # (a quarter of a GB and more) that the wide tiles' order through it stops fitting L2.
        m_tiles = (M + 127) // 128
        if persistent is None and tcgen05_persistent == "auto" and splits == 1 and tcgen05_persistent_pays(M, N, K, epi):
            tile_n, persistent = 256, True
        elif persistent is None and tcgen05_persistent == "auto" and splits == 1 and not epi and K <= 3072 and (
                tcgen05_one_round_width(M, N)):
            # about one tile an SM and a short K (o_proj and down_proj of 2,048 and 4,096 rows at the 0.6B sizes): a block that
            # has the SM to itself, with the persistent form's deeper ring, beats two blocks an SM on narrower tiles (10.0 and
            # 13.2 us against 11.4 and 15.3 at 2,048 rows, 14.6 and 19.2 against 15.1 and 21.0 at 4,096)
            tile_n, persistent = tcgen05_one_round_width(M, N), True
        elif epi:
            tile_n = 256 if (M >= 4096 or K >= 4096) and m_tiles * ((N + 127) // 128) <= 10000 else 128
        else:
            need = 200 if K < 4096 else 64
            tile_n = next((bn for bn in (256, 128) if m_tiles * ((N + bn - 1) // bn) >= need), 64)
    bn = tile_n
    _need(tcgen05_takes(x, weight) or M < tcgen05_min_rows(weight.numel()), "linear_tcgen05: operands not taken")
    box_w = bn // 2 if epi else bn
    if splits > 1:
        _need(out.dim() == 3 and out.shape[0] == tcgen05_splits(K, splits) and out.dtype == torch.float32 and out.is_contiguous(),
              "linear_tcgen05: partial results must be float32 [splits, M, N]")
        ldc, split_stride = out.stride(1), out.stride(0)
    else:
        ldc, split_stride = out.stride(0), 0
    if persistent is None:
        persistent = tcgen05_persistent
    if persistent == "auto":
        persistent = False
    if persistent and splits == 1 and bn >= 128:
        _call("me_gemm_tcgen05_persistent", matrix_tensor_map(x, 128).ptr, matrix_tensor_map(weight, box_w).ptr, out.data_ptr(),
              _dt(out), ldc, M, N, K, epi, bn, err.data_ptr(), _stream())
        return
    _call("me_gemm_tcgen05", matrix_tensor_map(x, 128).ptr, matrix_tensor_map(weight, box_w).ptr, out.data_ptr(), _dt(out),
          ldc, M, N, K, epi, bn, splits, split_stride, err.data_ptr(), _stream())


def tcgen05_splits(K: int, splits: int) -> int:
    """Partial results that ``linear_tcgen05`` writes when asked to split K ``splits`` ways (whole blocks of 64)."""
    return (_lib or require_extension()).me_gemm_tcgen05_splits(K, splits)


TCGEN05_SPLIT_MAX_ROWS = 1024      # rows up to which a product with few tiles is split along K


def tcgen05_split_plan(M: int, N: int, K: int) -> tuple[int, int]:
    """(tile width, parts of K) for a product of ``M`` rows whose consumer adds float32 partial results, or (0, 1).

    A product of a few hundred rows by a thousand columns has a handful of tiles for 148 SMs; shared out along K
    four ways it ran 25 to 40% faster (o_proj and down_proj of the 0.6B shape at 512 and 1,024 rows), at 2,048 rows
    no faster once the partial results are added."""
    if not (tcgen05_min_rows(N * K) <= M <= TCGEN05_SPLIT_MAX_ROWS):
        return 0, 1
    m_tiles = (M + 127) // 128
    bn = 64 if m_tiles * ((N + 127) // 128) * 4 < 128 else 128
    tiles = m_tiles * ((N + bn - 1) // bn)
    want = max(1, min(4, 256 // max(tiles, 1), K // 512))
    parts = tcgen05_splits(K, want)
    return (bn, parts) if parts >= 2 and tcgen05_splits(K, parts) == parts else (0, 1)


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: str = "none",
           workspace=None, err: Optional[torch.Tensor] = None) -> None:
    """``out = x @ weight.T`` with float32 accumulation; ``epilogue="silu_mul"`` takes a weight of
    rows gate | up and writes ``silu(x Wg^T) * (x Wu^T)``.

    float32 operands (and any mix of dtypes) run the CUDA-core kernel of csrc/gemm_simt.cu: plain
    FMA, no reduced-precision matrix mode.  bfloat16 x bfloat16 products of up to 16 rows run csrc/gemm_stream.cu
    where the weight has 32 MB and more (the vocabulary product of a decode step) and csrc/gemm_skinny.cu else
    (the layers' own products in decode do not come here: ``decode_linear``); 128 rows and more, and 48 rows and more
    where the weight is small (``tcgen05_min_rows``), run the tcgen05 kernels of csrc/gemm_tcgen05.cu; the rows between,
    and shapes those refuse (K no multiple of 8), go to cuBLAS, as all the
    reference's products do through ``F.linear`` (layers/linear.py:26,45), with SiLU-and-multiply as a kernel of ours
    behind it.

    ``err``: the int32[4] error word of the step; the tcgen05 kernel sets flag 1 there when one of its bounded
    waits runs out.  Without it products of 128 rows and more go to cuBLAS."""
    global library_calls
    key = ("linear", id(x), id(weight), id(out), epilogue)
    sig = (x.data_ptr(), weight.data_ptr(), out.data_ptr(), _ptr(err), x.shape, x.stride(), x.dtype, weight.shape,
           weight.stride(), weight.dtype, out.shape, out.stride(), out.dtype, use_tcgen05_gemm)
    if _repeat(key, sig):
        return
    before = launches
    M, K = x.shape
    _need(weight.dim() == 2 and weight.shape[1] == K and weight.is_contiguous(), "linear: weight shape")
    _need(x.stride(1) == 1 and out.stride(1) == 1, "linear: rows must be contiguous")
    epi = {"none": 0, "silu_mul": 1}[epilogue]
    N = weight.shape[0] // 2 if epi else weight.shape[0]
    _need(tuple(out.shape) == (M, N), f"linear: output is {tuple(out.shape)}, expected {(M, N)}")
    if M == 0:
        return
    if (err is not None and epi == 0 and weight.numel() >= STREAM_MIN_WEIGHT_ELEMENTS and skinny_splits(M, K, x, weight) > 0
            and out.dtype in (torch.bfloat16, torch.float32)):
        decode_linear(weight, x, out=out, err=err, kernel="stream")
        _remember(key, sig, before)
        return
    if skinny_splits(M, K, x, weight) == 1 and (epi == 0 or out.dtype == torch.bfloat16):
        _call("me_gemm_skinny", x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), _dt(out), out.stride(0),
              0, M, N, K, epi, _stream())
        _remember(key, sig, before)
        return
    if err is not None and use_tcgen05_gemm and tcgen05_takes(x, weight) and (epi == 0 or out.dtype == torch.bfloat16):
        linear_tcgen05(x, weight, out, epilogue, err)
        _remember(key, sig, before)
        return
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.is_cuda:
        if epi == 0 and out.dtype == torch.bfloat16:
            with _Timed("library_mm"):
                torch.mm(x, weight.t(), out=out)
            library_calls += 1
            return
        if epi == 0 and out.dtype == torch.float32:
            with _Timed("library_mm"):
                torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
            library_calls += 1
            return
        if epi == 1 and out.dtype == torch.bfloat16 and workspace is not None:
            tmp = workspace("linear_gate_up", (M, 2 * N), torch.bfloat16)
            with _Timed("library_mm"):
                torch.mm(x, weight.t(), out=tmp)
            library_calls += 1
            silu_mul(tmp, out)
            return
    _call("me_gemm_simt", x.data_ptr(), _dt(x), x.stride(0), weight.data_ptr(), _dt(weight),
          out.data_ptr(), _dt(out), out.stride(0), M, N, K, epi, _stream())


# ---- attention ------------------------------------------------------------------------------
ROTARY_LAYOUTS = ("half_split",)     # what the kernels rotate: element i with element i + rotary_dim / 2, i < rotary_dim / 2


def check_rotary(cos_sin: Optional[torch.Tensor], head_dim: int, rotary_dim: Optional[int], layout: str) -> int:
    """The rotary contract between a position encoding and the kernels: a float32 table [positions, rotary_dim]
    (cosines of the rotary_dim / 2 frequencies, then their sines), ``rotary_dim`` even and at most ``head_dim``
    (elements from rotary_dim on are left unrotated), and a layout the kernels know by name.  Returns rotary_dim."""
    if layout not in ROTARY_LAYOUTS:
        raise KernelError(f"rotary layout {layout!r} is not supported by the kernels (they take: {', '.join(ROTARY_LAYOUTS)}); "
                          "another pairing of elements needs another kernel branch")
    if cos_sin is None:
        return head_dim
    rd = head_dim if rotary_dim is None else int(rotary_dim)
    _need(rd % 2 == 0 and 2 <= rd <= head_dim, f"rotary_dim {rd} must be even and at most head_dim {head_dim}")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.dim() == 2 and cos_sin.shape[1] == rd,
          f"the rotary table must be float32 [positions, rotary_dim = {rd}]")
    return rd


def qk_norm_rope_kv_write(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                          q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                          cos_sin: Optional[torch.Tensor], positions: torch.Tensor,
                          slot_mapping: Optional[torch.Tensor], pool: torch.Tensor, page_size: int,
                          rotary_dim: Optional[int] = None, layout: str = "half_split") -> None:
    """In place on the packed rows q|k|v: RMSNorm of every q and k head, rotary embedding of the first
    ``rotary_dim`` elements of each (default: all of them), and the write of k and v to ``pool``
    [pages, 2, kv_heads, page_size, head_dim] at ``slot_mapping``."""
    T = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim, "qk_norm_rope: qkv shape")
    _need(pool.dtype == qkv.dtype and pool.is_contiguous()
          and tuple(pool.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "qk_norm_rope: pool shape")
    for w in (q_weight, k_weight):
        if w is not None:
            _need(w.dtype == torch.float32 and w.shape == (head_dim,), "qk_norm_rope: norm weights are float32 [head_dim]")
    rd = check_rotary(cos_sin, head_dim, rotary_dim, layout)
    _need(positions.dtype == torch.int32 and positions.shape[0] == T, "qk_norm_rope: positions")
    if slot_mapping is not None:
        _need(slot_mapping.dtype == torch.int32 and slot_mapping.shape[0] == T, "qk_norm_rope: slot mapping")
    _call("me_qk_norm_rope_kv_write", qkv.data_ptr(), _dt(qkv), qkv.stride(0), T, num_heads, num_kv_heads,
          head_dim, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos_sin), rd, positions.data_ptr(),
          _ptr(slot_mapping), pool.data_ptr(), page_size, _stream())


def attention_chunks(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta,
                     scale, window, tiles=None, num_tiles=None) -> None:
    """The CUDA-core chunk kernel over query tiles of 16 tokens (requests that bring several tokens)."""
    if tiles is None:
        tiles, num_tiles = meta.tile_lists[ATTN_TILE_Q]
    _call("me_attn_chunk", qkv.data_ptr(), _dt(qkv), qkv.stride(0), out.data_ptr(), out.stride(0),
          pool.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), meta.cu_seqlens.data_ptr(),
          meta.context_lens.data_ptr(), tiles.data_ptr(), num_tiles, num_heads, num_kv_heads, head_dim,
          page_size, float(scale), int(window or 0), _stream())


def prefill_heads_per_block(num_heads: int, num_kv_heads: int, head_dim: int) -> int:
    """How many heads of a group share a block of the tensor-core prefill kernel; 0 if it refuses the shape."""
    return (_lib or require_extension()).me_attn_prefill_heads_per_block(num_heads, num_kv_heads, head_dim)


def attention_prefill(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta,
                      scale, window, tiles=None, num_tiles=None) -> None:
    """The tensor-core prefill kernel (bfloat16, head_dim 64 or 128) over tiles of 64 / heads-per-block tokens."""
    gp = prefill_heads_per_block(num_heads, num_kv_heads, head_dim)
    _need(gp > 0 and qkv.dtype == torch.bfloat16, "attention_prefill: shape or dtype not taken by the tensor-core kernel")
    if tiles is None:
        tiles, num_tiles = meta.tile_lists[64 // gp]
    _call("me_attn_prefill", qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), pool.data_ptr(),
          block_tables.data_ptr(), block_tables.stride(0), meta.cu_seqlens.data_ptr(), meta.context_lens.data_ptr(),
          tiles.data_ptr(), num_tiles, num_heads, num_kv_heads, head_dim, page_size, float(scale),
          int(window or 0), _stream())


DECODE_KINDS = {"auto": 0, "cuda_cores": 1, "tensor_cores": 3, "tensor_cores_tma": 4}

_tensor_maps: dict = {}


class TensorMap:
    """A CUtensorMap (128 bytes, 64-byte aligned) kept alive on the host for kernels that take it by value."""

    def __init__(self):
        self._raw = ctypes.create_string_buffer(128 + 64)
        self.ptr = (ctypes.addressof(self._raw) + 63) & ~63


def kv_tensor_map(pool: torch.Tensor, page_size: int) -> Optional[TensorMap]:
    """The tensor map of one cache slot [pages, 2, kv_heads, page_size, head_dim] (bfloat16) as the 2-D tensor
    [pages * 2 * kv_heads * page_size, head_dim] with boxes of one page x 64 columns, 128-byte swizzle;
    None where the tensor-map kernels do not apply."""
    hd = pool.shape[-1]
    if pool.dtype != torch.bfloat16 or hd not in (64, 128) or page_size < 8 or DECODE_PARTITION % page_size:
        return None
    key = (pool.data_ptr(), tuple(pool.shape))
    tm = _tensor_maps.get(key)
    if tm is None:
        tm = TensorMap()
        rows = pool.shape[0] * 2 * pool.shape[2] * page_size
        lib = _lib or require_extension()
        if lib.me_tma_encode_2d(tm.ptr, pool.data_ptr(), rows, hd, hd * 2, page_size, 64, 128) != 0:
            raise KernelError(lib.me_last_error().decode())
        _tensor_maps[key] = tm
    return tm


def prefill_tcgen05_heads_per_block(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> int:
    """How many heads of a group share a block of the tcgen05 prefill kernel; 0 if it refuses the shape."""
    return (_lib or require_extension()).me_attn_prefill_tcgen05_heads_per_block(num_heads, num_kv_heads, head_dim, page_size)


def attention_prefill_tcgen05(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta,
                              scale, window, tiles=None, num_tiles=None, key_tile: int = 0) -> None:
    """The tcgen05 / tensor-memory prefill kernel (bfloat16, head_dim 64 or 128, page sizes dividing 128) over
    tiles of 128 / heads-per-block tokens; Q, K and V arrive by tensor-map loads."""
    gp = prefill_tcgen05_heads_per_block(num_heads, num_kv_heads, head_dim, page_size)
    _need(gp > 0 and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and qkv.data_ptr() % 16 == 0,
          "attention_prefill_tcgen05: shape or dtype not taken by the kernel")
    tq = 128 // gp
    if tiles is None:
        tiles, num_tiles = meta.tile_lists[tq]
    _call("me_attn_prefill_tcgen05", matrix_tensor_map(qkv, tq).ptr, kv_tensor_map(pool, page_size).ptr, out.data_ptr(),
          out.stride(0), block_tables.data_ptr(), block_tables.stride(0), meta.cu_seqlens.data_ptr(),
          meta.context_lens.data_ptr(), tiles.data_ptr(), num_tiles, num_heads, num_kv_heads, head_dim, page_size,
          float(scale), int(window or 0), key_tile, meta.error_flag.data_ptr(), _stream())


use_tcgen05_attention = True   # False: portions of prompts use the mma.sync kernel instead (a switch for comparisons)


def attention_decode(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta,
                     scale, window, kind: str = "auto") -> None:
    """The split-K decode kernel and its merge over requests [0, meta.num_decodes).

    ``kind`` picks the partition kernel: "auto" (for bfloat16 with head_dim 64 or 128 the tensor cores, fed by
    tensor-map loads where the page size divides 128, else by cp.async; otherwise the CUDA cores), or one
    of them by name (tests run each)."""
    D = meta.num_decodes
    parts = max(1, (meta.max_context_len + DECODE_PARTITION - 1) // DECODE_PARTITION)
    room = max(parts, (getattr(meta, "scratch_context_len", 0) + DECODE_PARTITION - 1) // DECODE_PARTITION)
    tmp_out = meta.workspace("decode_tmp_out", (D * num_heads * room * head_dim,), torch.float32)
    tmp_ml = meta.workspace("decode_tmp_ml", (2, D * num_heads * room), torch.float32)
    tm = kv_tensor_map(pool, page_size) if kind in ("auto", "tensor_cores_tma") else None
    _call("me_attn_decode", qkv.data_ptr(), _dt(qkv), qkv.stride(0), out.data_ptr(), out.stride(0),
          pool.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), meta.cu_seqlens.data_ptr(),
          meta.context_lens.data_ptr(), D, num_heads, num_kv_heads, head_dim, page_size, float(scale),
          int(window or 0), tmp_out.data_ptr(), tmp_ml[0].data_ptr(), tmp_ml[1].data_ptr(), parts,
          _ptr(meta.error_flag), DECODE_KINDS[kind], tm.ptr if tm is not None else 0, _stream())
    global launches
    launches += 1          # partition kernel + merge kernel


def decode_fused_takes(qkv: torch.Tensor, head_dim: int, pool: torch.Tensor, page_size: int, meta,
                       rotary_dim: Optional[int] = None) -> bool:
    """Whether ``attention_decode_fused`` takes the step: bfloat16, head size 64 or 128, pages of 8 to 128 tokens
    that divide 128, a tensor map over the cache, and a rotation over the whole head (or none)."""
    lib = _lib or require_extension()
    return (qkv.is_cuda and (rotary_dim is None or rotary_dim == head_dim) and qkv.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and meta.error_flag is not None
            and bool(lib.me_attn_decode_fused_takes(head_dim, page_size)) and (qkv.stride(0) * 2) % 16 == 0
            and kv_tensor_map(pool, page_size) is not None)


# The form of the decode partition kernel: "one_tile" (K and V pass through the same shared-memory tile, five blocks
# an SM), "two_tiles" (a tile each, three blocks an SM) or "tile_and_half" (half a tile for V beside K's, four blocks).
DECODE_FORMS = {"one_tile": 0, "two_tiles": 2, "tile_and_half": 3}
# "auto": by the number of partitions with keys.  Up to what three blocks an SM hold at once, two tiles (all loads in
# flight together); beyond, one tile (more blocks an SM).  In a step of the 0.6B shape at 1,024 tokens of context:
# batch 4, 0.770 ms against 0.815 with one tile; batch 8, 0.885 with one tile against 0.898 with two and 0.938 with a
# tile and a half; batch 16, 1.199 against 1.221 and 1.252; batch 64, 2.50 against 2.89 and 3.08.
decode_form = "auto"


decode_tiles = "auto"     # tiles of 128 keys that a block of the "one_tile" form walks: "auto" or a number (for comparisons)


def decode_tiles_for(rows: int, key_tiles: int) -> int:
    """How many tiles of 128 keys a block of the fused decode kernel's "one_tile" form walks, for ``rows`` = requests x
    key/value heads (x strips of 16 query heads) and contexts of ``key_tiles`` tiles: the largest power of two (up to 32)
    that still leaves two partitions a request and as many blocks as the device holds at once (four of the tiled
    kernel share an SM).  Measured on batches of 16 to 256 at contexts of 1,100 to 4,100 with 2 and 8 query heads a
    group: the best count was this one in every case (one partition for the whole context was 2 to 4% behind two)."""
    want = 4 * sm_count()
    tiles = 1
    while tiles < 32 and 2 * tiles < key_tiles and rows * -(-key_tiles // (2 * tiles)) >= want:
        tiles *= 2
    if tiles < 4 and key_tiles > 32:
        # Few requests with long contexts: single tiles would make dozens of partitions a head, whose partial results and
        # merge (more than 16 partitions take the merge kernel several trips to memory) cost more than the blocks that
        # four tiles a block leave idle.  Measured at 1 to 8 requests of 8,192 tokens and 1 of 30,000: 18 to 48% faster.
        tiles = 4 if rows * -(-key_tiles // 4) >= 100 else 2
    return tiles


def decode_forms_for(page_size: int) -> list[str]:
    """The forms of the fused decode kernel that take pages of ``page_size`` tokens (for a caller that times them)."""
    return [f for f in DECODE_FORMS if f != "tile_and_half" or (DECODE_PARTITION // 2) % page_size == 0]


def attention_decode_fused(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta, scale, window,
                           q_weight, k_weight, eps, cos_sin, slot_mapping, form: Optional[str] = None,
                           tiles: Optional[int] = None) -> None:
    """Decode attention over requests [0, meta.num_decodes) straight from the q|k|v product's rows: the kernel
    applies the q/k norm and the rotary embedding to q and to the newest key itself and writes that key and the
    newest value into the cache (``slot_mapping``; None if another layer wrote them), so the step needs no
    ``qk_norm_rope_kv_write`` for these rows.  The token's position is its request's context length minus one.
    Other arguments as for that function and ``attention_decode``.  ``form``: one of ``DECODE_FORMS`` (default
    ``decode_form``).  ``tiles``: how many tiles of 128 keys a block of the "one_tile" form walks (default
    ``decode_tiles``; "auto": by how many blocks there would be)."""
    form = form or decode_form
    typical = getattr(meta, "typical_context_len", 0) or meta.max_context_len
    rows = meta.num_decodes * num_kv_heads * ((num_heads // num_kv_heads + 15) // 16)
    key_tiles = (typical + DECODE_PARTITION - 1) // DECODE_PARTITION
    blocks = rows * key_tiles
    tiles = decode_tiles if tiles is None else tiles
    if form == "auto":
        resident = 3 * sm_count()                   # blocks of the two-tile form that the device holds at once
        form = "two_tiles" if blocks <= resident else "one_tile"
        if tiles == "auto" and decode_tiles_for(rows, key_tiles) > 1:
            form = "one_tile"                       # (the form whose blocks can walk several tiles)
    if form != "one_tile":
        tiles = 1
    elif tiles == "auto":
        tiles = decode_tiles_for(rows, key_tiles)
    D = meta.num_decodes
    part_keys = DECODE_PARTITION * tiles
    parts = max(1, (meta.max_context_len + part_keys - 1) // part_keys)
    room = max(parts, (getattr(meta, "scratch_context_len", 0) + part_keys - 1) // part_keys)
    tmp_out = meta.workspace("decode_tmp_out", (D * num_heads * room * head_dim,), torch.float32)
    tmp_ml = meta.workspace("decode_tmp_ml", (2, D * num_heads * room), torch.float32)
    tm = kv_tensor_map(pool, page_size)
    _need(tm is not None and tuple(pool.shape[1:]) == (2, num_kv_heads, page_size, head_dim) and pool.is_contiguous(),
          "attention_decode_fused: cache slot")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and tuple(w.shape) == (head_dim,)), "attention_decode_fused: norm weights")
    _need(check_rotary(cos_sin, head_dim, None, "half_split") == head_dim, "attention_decode_fused: the rotation covers the whole head")
    _need(slot_mapping is None or slot_mapping.dtype == torch.int32, "attention_decode_fused: slots are int32")
    _call("me_attn_decode_fused", qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), pool.data_ptr(), tm.ptr,
          block_tables.data_ptr(), block_tables.stride(0), meta.cu_seqlens.data_ptr(), meta.context_lens.data_ptr(), D,
          num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0), _ptr(q_weight), _ptr(k_weight),
          float(eps), _ptr(cos_sin), _ptr(slot_mapping), tmp_out.data_ptr(), tmp_ml[0].data_ptr(),
          tmp_ml[1].data_ptr(), parts, DECODE_FORMS[form], int(tiles), meta.error_flag.data_ptr(), _stream())
    global launches
    launches += 1          # partition kernel + merge kernel


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                    pool: torch.Tensor, page_size: int, block_tables: torch.Tensor, meta, scale: float,
                    window: Optional[int], decodes: bool = True) -> None:
    """Attention of one step over the paged cache: requests that bring one token go to the decode
    kernel (unless ``decodes`` is False: the caller has run them), portions of prompts to the chunk kernel;
    both write their rows of ``out`` (the split of layers/attention.py:64-76)."""
    check_attention_sizes(head_dim, num_heads, num_kv_heads)
    _need(qkv.stride(1) == 1 and out.stride(1) == 1 and out.shape[1] == num_heads * head_dim, "paged_attention: shapes")
    _need(pool.dtype == qkv.dtype == out.dtype and pool.is_contiguous(), "paged_attention: dtypes")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "paged_attention: block tables")
    if decodes and meta.num_decodes > 0:
        attention_decode(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta, scale, window)
    if meta.num_tiles > 0:
        fn = attention_chunks
        if qkv.dtype == torch.bfloat16:
            if (use_tcgen05_attention and meta.error_flag is not None and qkv.is_contiguous()
                    and prefill_tcgen05_heads_per_block(num_heads, num_kv_heads, head_dim, page_size) > 0):
                fn = attention_prefill_tcgen05
            elif prefill_heads_per_block(num_heads, num_kv_heads, head_dim) > 0:
                fn = attention_prefill
        fn(qkv, out, num_heads, num_kv_heads, head_dim, pool, page_size, block_tables, meta, scale, window)


# ---- sampling -------------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperatures: torch.Tensor, seeds: torch.Tensor, positions: torch.Tensor,
           out: torch.Tensor, workspace=None) -> None:
    """Greedy (temperature 0) or exponential-race draw per row; two passes over pieces of the vocabulary."""
    global launches
    S, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: logits must be float32 rows")
    _need(temperatures.dtype == torch.float32 and seeds.dtype == torch.int32 and positions.dtype == torch.int32
          and out.dtype == torch.int32, "sample: dtypes")
    _need(temperatures.shape[0] == S and seeds.shape[0] == S and positions.shape[0] == S and out.shape[0] == S, "sample: sizes")
    chunks = (_lib or require_extension()).me_sample_chunks(V)
    if workspace is None:
        part = torch.empty(2, S * chunks, dtype=torch.float32, device=logits.device)
    else:
        part = workspace("sample_partials", (2, S * chunks), torch.float32)
    _call("me_sample", logits.data_ptr(), logits.stride(0), temperatures.data_ptr(), seeds.data_ptr(),
          positions.data_ptr(), out.data_ptr(), S, V, part[0].data_ptr(), part[1].data_ptr(), _stream())
    launches += 1
