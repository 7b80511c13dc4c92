// Products of a decode step (up to 16 rows) with the neighbouring element-wise work folded in, so that a
// layer needs no separate normalisation kernels.  RMSNorm (layers/layernorm.py:11-16 in the reference) is
// y = x * rsqrt(mean(x^2) + eps) * w: the factor rsqrt(...) is one number per row, so it commutes with the
// product that follows, (y W^T)[m][n] = rsqrt(...)[m] * ((x * w) W^T)[m][n].  That splits the norm in two
// halves that need no pass of their own:
//
//   epilogue RESID: residual += X W^T (the add of layers/layernorm.py:19-23, which the reference does inside
//                   the next norm); the new residual times the NEXT norm's weight is written in bfloat16
//                   beside it, and the strip's partial sums of squares of the new residual.
//   row scale:      a product whose X is such a pre-weighted residual multiplies its float32 results by the
//                   row's rsqrt(mean square + eps), from the partial sums added in strip order.
//   epilogue SILU:  rows gate | up, writes silu(gate) * up (layers/activation.py:4-7).
//
// As in gemm_skinny.cu the weight rows fill the M side of mma.sync m16n8k16 and a block owns a strip of
// 16 weight rows (8 where 16 would leave most SMs without a block); but here the block covers ALL of K with
// one warp per 256 elements (up to 12 warps), so every output element is finished inside one block and can
// be added to the residual by exactly one thread.  Weights are requested (cp.async) before
// griddepcontrol.wait, activations and the residual's old values after.
#include "common.cuh"
#include "mma_prims.cuh"

namespace {
using namespace mma_prims;

constexpr int DL_KW = 256, DL_PIECES = DL_KW / 8, DL_MAX_WARPS = 12;

__device__ __forceinline__ bf16* dl_ptr(bf16* base, int row, int piece) {
  return base + row * DL_KW + ((piece ^ (row & 7)) << 3);
}

// X is bfloat16 [M][ldx].  With ``sumsq_in`` ([sumsq_parts][M], the sums of squares of the rows that X was made
// from, over ``K`` columns) the results are multiplied by rsqrt(sum / K + eps) of their row.
// EPI 0: Y[m][n] (bfloat16 or float32).  EPI 1: SiLU(gate) * up, bfloat16.
// EPI 2: residual_out[m][n] += v, sumsq_out, and with ``next_w`` also xw_out[m][n] = residual_out[m][n] * next_w[n].
template <int EPI, typename TO, int R /* weight rows of a strip: 16, or 8 with the upper half of the tile idle */>
__global__ void __launch_bounds__(DL_MAX_WARPS * 32)
gemm_decode_kernel(const bf16* __restrict__ X, int64_t ldx, const float* __restrict__ sumsq_in, int sumsq_parts, float eps,
                   const bf16* __restrict__ W, TO* __restrict__ Y, int64_t ldy, float* __restrict__ res_out,
                   float* __restrict__ sumsq_out, const float* __restrict__ next_w, bf16* __restrict__ xw_out, int M,
                   int N, int K, const unsigned char* __restrict__ ahead, unsigned long long ahead_bytes) {
  extern __shared__ __align__(128) unsigned char dl_smem[];
  // The weights of the product that runs after this one are asked into L2 now: a decode step is a chain of
  // short dependent kernels, and without this the memory system idles while each waits for the one before.
  if (ahead != nullptr && threadIdx.x < 32) {
    const unsigned long long per = ((ahead_bytes + gridDim.x - 1) / gridDim.x + 15) & ~15ull;
    const unsigned long long lo = blockIdx.x * per, hi = lo + per < ahead_bytes ? lo + per : ahead_bytes;
    constexpr unsigned long long PIECE = 16384;
    for (unsigned long long o = lo + threadIdx.x * PIECE; o < hi; o += 32 * PIECE) {
      const unsigned n = (unsigned)((hi - o < PIECE ? hi - o : PIECE) & ~15ull);
      if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ahead + o), "r"(n) : "memory");
    }
  }
  __shared__ float row_scale[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  // the warps' partial products [nwarps][16][17] lie behind the operand tiles: sized by the launch, so that a
  // product over a short K keeps three blocks on an SM
  float (*red)[16][17] = reinterpret_cast<float (*)[16][17]>(dl_smem + (size_t)nwarps * 2 * 16 * DL_KW * sizeof(bf16));
  bf16* ws = reinterpret_cast<bf16*>(dl_smem) + warp * 2 * 16 * DL_KW;
  bf16* xs = ws + 16 * DL_KW;
  const int strip = blockIdx.x;
  const int k0 = warp * DL_KW;
  auto w_row = [&](int r) -> int64_t {
    if (EPI == 1) return r < 8 ? (int64_t)strip * 8 + r : (int64_t)N + strip * 8 + (r - 8);
    return (int64_t)strip * R + r;
  };
  const int n_rows = EPI == 1 ? 2 * N : N;
  // piece index of this lane is the same for all rows it copies: c = lane + 32 i -> row i, piece lane
  const int k = k0 + lane * 8;
#pragma unroll
  for (int row = 0; row < R; ++row) {
    const int64_t wr = w_row(row);
    const bool okw = k < K && wr < n_rows && (EPI != 1 || strip * 8 + (row & 7) < N);
    cp_async16(dl_ptr(ws, row, lane), okw ? W + wr * K + k : W, okw);
  }
  cp_async_commit();
  // rows of X beyond M are zero: written here, so that after the wait only real rows are asked for
#pragma unroll
  for (int row = 0; row < 16; ++row)
    if (row >= M || k >= K) *reinterpret_cast<uint4*>(dl_ptr(xs, row, lane)) = make_uint4(0, 0, 0, 0);
  constexpr int EPI_ITERS = 16 * R / 32;     // a block of one warp walks the strip's 16 x R results in so many rounds
  float old[EPI_ITERS], nw[EPI_ITERS];       // EPI 2: the residual's values this thread will add to; the next norm's weights
  if (EPI == 2) {
#pragma unroll
    for (int i = 0; i < EPI_ITERS; ++i) {
      const int idx = tid + i * (int)blockDim.x, m = idx / R, n = strip * R + idx % R;
      nw[i] = (idx < 16 * R && m < M && n < N && next_w != nullptr) ? next_w[n] : 0.f;
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  // After the wait, in the order of their latency's weight: the sums of squares and the residual's old values
  // (plain loads, needed in registers), then the rows of X (asynchronous copies).  Warp w computes the factors
  // of rows w, w + nwarps, ...; all sums of squares that a lane adds are requested before the first is used
  // (one L2 latency, not one per strip) and added in strip order; the factors are read after the block-wide
  // barrier in front of the epilogue.
  constexpr int SQ_J = 6;                    // 32 * 6 strips at most (checked by the host)
  float v[4][SQ_J];                          // (a block of fewer than 4 warps repeats this for rows beyond 4 * nwarps, below)
#pragma unroll
  for (int mi = 0; mi < 4; ++mi) {
    const int m = warp + mi * nwarps;
#pragma unroll
    for (int j = 0; j < SQ_J; ++j) {
      const int p = lane + 32 * j;
      v[mi][j] = (sumsq_in != nullptr && m < M && p < sumsq_parts) ? sumsq_in[(int64_t)p * M + m] : 0.f;
    }
  }
  if (EPI == 2) {
#pragma unroll
    for (int i = 0; i < EPI_ITERS; ++i) {
      const int idx = tid + i * (int)blockDim.x, m = idx / R, n = strip * R + idx % R;
      old[i] = (idx < 16 * R && m < M && n < N) ? res_out[(int64_t)m * N + n] : 0.f;
    }
  }
#pragma unroll
  for (int row = 0; row < 16; ++row)
    if (row < M && k < K) cp_async16(dl_ptr(xs, row, lane), X + (int64_t)row * ldx + k, true);
  cp_async_commit();
  for (int m0 = warp; m0 < 16; m0 += 4 * nwarps) {
    if (m0 != warp) {
#pragma unroll
      for (int mi = 0; mi < 4; ++mi) {
        const int m = m0 + mi * nwarps;
#pragma unroll
        for (int j = 0; j < SQ_J; ++j) {
          const int p = lane + 32 * j;
          v[mi][j] = (sumsq_in != nullptr && m < M && p < sumsq_parts) ? sumsq_in[(int64_t)p * M + m] : 0.f;
        }
      }
    }
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
      const int m = m0 + mi * nwarps;
      if (m >= 16) break;
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < SQ_J; ++j) s += v[mi][j];
      s = warp_sum(s);
      if (lane == 0) row_scale[m] = sumsq_in != nullptr ? (m < M ? 1.0f / sqrtf(s / (float)K + eps) : 0.f) : 1.0f;
    }
  }
  cp_async_wait<0>();
  __syncwarp();
  float c[2][4] = {};
  const int mi = lane >> 3;
  if (k0 < K) {
#pragma unroll
    for (int kk = 0; kk < DL_KW / 16; ++kk) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, dl_ptr(ws, (mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1)));
      ldmatrix_x4(b, dl_ptr(xs, (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
      mma_bf16(c[0], a, b[0], b[1]);
      mma_bf16(c[1], a, b[2], b[3]);
    }
  }
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    red[warp][g][nt * 8 + 2 * t4] = c[nt][0];
    red[warp][g][nt * 8 + 2 * t4 + 1] = c[nt][1];
    if (R == 16) {
      red[warp][g + 8][nt * 8 + 2 * t4] = c[nt][2];
      red[warp][g + 8][nt * 8 + 2 * t4 + 1] = c[nt][3];
    }
  }
  __syncthreads();
  auto total = [&](int r, int m) {
    float v = red[0][r][m];
    for (int w = 1; w < nwarps; ++w) v += red[w][r][m];   // warps in index order
    return v;
  };
  if (EPI == 1) {
    for (int idx = tid; idx < 16 * 8; idx += blockDim.x) {
      const int m = idx >> 3, r = idx & 7;
      const int n = strip * 8 + r;
      if (m >= M || n >= N) continue;
      const float gate = total(r, m) * row_scale[m], up = total(r + 8, m) * row_scale[m];
      Y[(int64_t)m * ldy + n] = from_f<TO>(gate / (1.0f + expf(-gate)) * up);
    }
  } else if (EPI == 2) {
    // R consecutive threads hold the R columns of one row: add into the residual, then the row's sum of squares
#pragma unroll
    for (int i = 0; i < EPI_ITERS; ++i) {            // whole warps: the R lanes of a row stay together
      const int idx = tid + i * (int)blockDim.x;
      if (idx - lane >= 16 * R) break;
      const int m = idx / R, r = idx % R;
      const int n = strip * R + r;
      float sq = 0.f;
      if (m < M && n < N) {
        const float v = old[i] + total(r, m) * row_scale[m];
        res_out[(int64_t)m * N + n] = v;
        sq = v * v;
        if (xw_out != nullptr) xw_out[(int64_t)m * N + n] = __float2bfloat16(v * nw[i]);
      }
#pragma unroll
      for (int o = R / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (r == 0 && m < M) sumsq_out[(int64_t)strip * M + m] = sq;
    }
  } else {
    for (int idx = tid; idx < 16 * R; idx += blockDim.x) {
      const int m = idx / R, r = idx % R;
      const int n = strip * R + r;
      if (m >= M || n >= N) continue;
      Y[(int64_t)m * ldy + n] = from_f<TO>(total(r, m) * row_scale[m]);
    }
  }
}

template <int EPI, typename TO, int R>
int launch_dl(int strips, int warps, cudaStream_t stream, const void* X, int64_t ldx, const float* sumsq_in, int sumsq_parts,
              float eps, const void* W, void* Y, int64_t ldy, float* res_out, float* sumsq_out, const float* next_w,
              void* xw_out, int M, int N, int K, const void* ahead, unsigned long long ahead_bytes) {
  const size_t smem = (size_t)warps * (2 * 16 * DL_KW * sizeof(bf16) + 16 * 17 * sizeof(float));
  static size_t attr = 0;
  if (smem > attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_decode_kernel<EPI, TO, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_gemm_decode: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr = smem;
  }
  me_launch(gemm_decode_kernel<EPI, TO, R>, dim3(strips), dim3(warps * 32), smem, stream, (const bf16*)X, ldx, sumsq_in,
            sumsq_parts, eps, (const bf16*)W, (TO*)Y, ldy, res_out, sumsq_out, next_w, (bf16*)xw_out, M, N, K,
            (const unsigned char*)ahead, ahead_bytes);
  return 0;
}
}  // namespace

// Largest K the kernel covers inside one block.
ME_API int me_gemm_decode_max_k() { return DL_MAX_WARPS * DL_KW; }
// Weight rows of a strip for N output columns: 16, or 8 where strips of 16 would occupy fewer than about two
// thirds of the SMs (a block streams its weight rows alone; more blocks pull more bandwidth).
static int strip_rows(int N) { return (N + 15) / 16 < 96 ? 8 : 16; }
// Parts of the sums of squares that the residual epilogue writes for N output columns.
ME_API int me_gemm_decode_sumsq_parts(int N) { const int r = strip_rows(N); return (N + r - 1) / r; }

// X bfloat16 [M][ldx].  sumsq_in (or null) [sumsq_parts][M] with eps: the results of row m are multiplied by
// rsqrt(sum_p sumsq_in[p][m] / K + eps).
// epi 0: Y (y_dtype) [M][ldy]; epi 1: SiLU-and-multiply (weight rows gate | up, N = columns of Y);
// epi 2: res_out [M][N] += X W^T, sumsq_out [me_gemm_decode_sumsq_parts(N)][M] and, with next_w [N], xw_out
// bfloat16 [M][N] = res_out * next_w.
// ahead (or null), ahead_bytes: memory that a later kernel will read (the next product's weights), asked into
// L2 by this one; 16-byte aligned.
ME_API int me_gemm_decode(int epi, const void* X, int64_t ldx, const float* sumsq_in, int sumsq_parts, float eps,
                          const void* W, void* Y, int y_dtype, int64_t ldy, float* res_out, float* sumsq_out,
                          const float* next_w, void* xw_out, int M, int N, int K, const void* ahead,
                          unsigned long long ahead_bytes, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && M <= 16, "me_gemm_decode: M=%d is not in 1..16", M);
  ME_REQUIRE(K % 8 == 0 && K > 0 && K <= DL_MAX_WARPS * DL_KW, "me_gemm_decode: K=%d must be a multiple of 8 up to %d", K,
             DL_MAX_WARPS * DL_KW);
  ME_REQUIRE(X != nullptr && (ldx * 2) % 16 == 0, "me_gemm_decode: X is missing or its rows are not 16-byte aligned");
  ME_REQUIRE(sumsq_in == nullptr || (sumsq_parts > 0 && sumsq_parts <= 192), "me_gemm_decode: sums of squares in %d parts (1..192)",
             sumsq_parts);
  ME_REQUIRE(epi == 0 || epi == 1 || (epi == 2 && res_out != nullptr && sumsq_out != nullptr), "me_gemm_decode: epilogue %d", epi);
  ME_REQUIRE((next_w == nullptr) == (xw_out == nullptr) && (next_w == nullptr || epi == 2),
             "me_gemm_decode: the pre-weighted copy needs the residual epilogue, a weight and an output");
  ME_REQUIRE(ahead == nullptr || ((uintptr_t)ahead & 15) == 0, "me_gemm_decode: memory to fetch ahead must be 16-byte aligned");
  const int warps = (K + DL_KW - 1) / DL_KW;
  const int rows = epi == 1 ? 16 : strip_rows(N);
  const int strips = epi == 1 ? (N + 7) / 8 : (N + rows - 1) / rows;
  int rc = 1;
#define ME_DL(EPI_, TO_, R_)                                                                                        \
  rc = launch_dl<EPI_, TO_, R_>(strips, warps, stream, X, ldx, sumsq_in, sumsq_parts, eps, W, Y, ldy, res_out, sumsq_out, \
                                next_w, xw_out, M, N, K, ahead, ahead_bytes)
  if (epi == 2) {
    if (rows == 8) ME_DL(2, float, 8); else ME_DL(2, float, 16);
  } else if (epi == 1) {
    ME_REQUIRE(y_dtype == ME_BF16, "me_gemm_decode: the SiLU epilogue writes bfloat16");
    ME_DL(1, bf16, 16);
  } else if (y_dtype == ME_BF16) {
    if (rows == 8) ME_DL(0, bf16, 8); else ME_DL(0, bf16, 16);
  } else {
    if (rows == 8) ME_DL(0, float, 8); else ME_DL(0, float, 16);
  }
#undef ME_DL
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_gemm_decode");
  return 0;
}
