// Products of a decode step (up to 16 rows) with the neighbouring element-wise work folded in, so that a
// layer needs no separate normalisation kernels:
//
//   prologue NORM:  X = rmsnorm(residual) * weight is formed on the fly from the float32 residual stream
//                   (layers/layernorm.py:11-16 in the reference); the row's mean square comes from per-strip
//                   partial sums that the product before left behind, added in strip order.
//   epilogue RESID: residual += X W^T (the add of layers/layernorm.py:19-23, which the reference does inside
//                   the next norm), and the strip's partial sums of squares of the new residual are written
//                   for the next product's prologue.
//   epilogue SILU:  rows gate | up, writes silu(gate) * up (layers/activation.py:4-7).
//
// As in gemm_skinny.cu the weight rows fill the M side of mma.sync m16n8k16 and a block owns a strip of
// 16 weight rows; but here the block covers ALL of K with one warp per 256 elements (up to 12 warps), so
// every output element is finished inside one block and can be added to the residual by exactly one
// thread.  Weights are requested (cp.async) before griddepcontrol.wait, activations after.
#include "common.cuh"
#include "mma_prims.cuh"

namespace {
using namespace mma_prims;

constexpr int DL_KW = 256, DL_PIECES = DL_KW / 8, DL_MAX_WARPS = 12;

__device__ __forceinline__ bf16* dl_ptr(bf16* base, int row, int piece) {
  return base + row * DL_KW + ((piece ^ (row & 7)) << 3);
}

// PRO 0: X is bfloat16 [M][ldx].  PRO 1: X = residual * inv_rms * norm_w, residual float32 [M][K].
// EPI 0: Y[m][n] (bfloat16 or float32).  EPI 1: SiLU(gate) * up, bfloat16.  EPI 2: residual_out[m][n] += v, sumsq_out.
template <int PRO, int EPI, typename TO>
__global__ void __launch_bounds__(DL_MAX_WARPS * 32)
gemm_decode_kernel(const bf16* __restrict__ X, int64_t ldx, const float* __restrict__ res_in, const float* __restrict__ norm_w,
                   const float* __restrict__ sumsq_in, int sumsq_parts, float eps, const bf16* __restrict__ W,
                   TO* __restrict__ Y, int64_t ldy, float* __restrict__ res_out, float* __restrict__ sumsq_out, int M,
                   int N, int K) {
  extern __shared__ __align__(128) unsigned char dl_smem[];
  __shared__ float red[DL_MAX_WARPS][16][17];
  __shared__ float inv_rms[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  bf16* ws = reinterpret_cast<bf16*>(dl_smem) + warp * 2 * 16 * DL_KW;
  bf16* xs = ws + 16 * DL_KW;
  const int strip = blockIdx.x;
  const int k0 = warp * DL_KW;
  auto w_row = [&](int r) -> int64_t {
    if (EPI == 1) return r < 8 ? (int64_t)strip * 8 + r : (int64_t)N + strip * 8 + (r - 8);
    return (int64_t)strip * 16 + r;
  };
  const int n_rows = EPI == 1 ? 2 * N : N;
  // piece index of this lane is the same for all rows it copies: c = lane + 32 i -> row i, piece lane
  const int k = k0 + lane * 8;
#pragma unroll
  for (int row = 0; row < 16; ++row) {
    const int64_t wr = w_row(row);
    const bool okw = k < K && wr < n_rows && (EPI != 1 || strip * 8 + (row & 7) < N);
    cp_async16(dl_ptr(ws, row, lane), okw ? W + wr * K + k : W, okw);
  }
  cp_async_commit();
  pdl_wait();
  pdl_launch_dependents();
  if (PRO == 1) {
    // every warp needs every row's 1/rms: warp w computes rows w, w + nwarps, ...
    for (int m = warp; m < 16; m += nwarps) {
      float s = 0.f;
      if (m < M)
        for (int p = lane; p < sumsq_parts; p += 32) s += sumsq_in[(int64_t)p * M + m];
      // lanes hold strided partial sums; add them in a fixed order
      s = warp_sum(s);
      if (lane == 0) inv_rms[m] = m < M ? 1.0f / sqrtf(s / (float)K + eps) : 0.f;
    }
    __syncthreads();
    float wv[8];
    if (k < K) {
      const float4 a = *reinterpret_cast<const float4*>(norm_w + k), b = *reinterpret_cast<const float4*>(norm_w + k + 4);
      wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
    }
#pragma unroll 4
    for (int row = 0; row < 16; ++row) {
      uint4 pk = make_uint4(0, 0, 0, 0);
      if (row < M && k < K) {
        const float* rp = res_in + (int64_t)row * K + k;
        const float4 a = *reinterpret_cast<const float4*>(rp), b = *reinterpret_cast<const float4*>(rp + 4);
        const float inv = inv_rms[row];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
        h[0] = __floats2bfloat162_rn((a.x * inv) * wv[0], (a.y * inv) * wv[1]);
        h[1] = __floats2bfloat162_rn((a.z * inv) * wv[2], (a.w * inv) * wv[3]);
        h[2] = __floats2bfloat162_rn((b.x * inv) * wv[4], (b.y * inv) * wv[5]);
        h[3] = __floats2bfloat162_rn((b.z * inv) * wv[6], (b.w * inv) * wv[7]);
      }
      *reinterpret_cast<uint4*>(dl_ptr(xs, row, lane)) = pk;
    }
    __syncwarp();
  } else {
#pragma unroll
    for (int row = 0; row < 16; ++row) {
      const bool okx = k < K && row < M;
      cp_async16(dl_ptr(xs, row, lane), okx ? X + (int64_t)row * ldx + k : X, okx);
    }
    cp_async_commit();
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
    red[warp][g + 8][nt * 8 + 2 * t4] = c[nt][2];
    red[warp][g + 8][nt * 8 + 2 * t4 + 1] = c[nt][3];
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
      const float gate = total(r, m), up = total(r + 8, m);
      Y[(int64_t)m * ldy + n] = from_f<TO>(gate / (1.0f + expf(-gate)) * up);
    }
  } else if (EPI == 2) {
    // 16 consecutive threads hold the 16 columns of one row: add into the residual, then the row's sum of squares
    for (int idx = tid; idx < 256; idx += blockDim.x) {     // whole warps: 16 lanes per row stay together
      const int m = idx >> 4, r = idx & 15;
      const int n = strip * 16 + r;
      float sq = 0.f;
      if (m < M && n < N) {
        float* p = res_out + (int64_t)m * N + n;
        const float v = *p + total(r, m);
        *p = v;
        sq = v * v;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (r == 0 && m < M) sumsq_out[(int64_t)strip * M + m] = sq;
    }
  } else {
    for (int idx = tid; idx < 16 * 16; idx += blockDim.x) {
      const int m = idx >> 4, r = idx & 15;
      const int n = strip * 16 + r;
      if (m >= M || n >= N) continue;
      Y[(int64_t)m * ldy + n] = from_f<TO>(total(r, m));
    }
  }
}

template <int PRO, int EPI, typename TO>
int launch_dl(int strips, int warps, cudaStream_t stream, const void* X, int64_t ldx, const float* res_in, const float* norm_w,
              const float* sumsq_in, int sumsq_parts, float eps, const void* W, void* Y, int64_t ldy, float* res_out,
              float* sumsq_out, int M, int N, int K) {
  const size_t smem = (size_t)warps * 2 * 16 * DL_KW * sizeof(bf16);
  static size_t attr = 0;
  if (smem > attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_decode_kernel<PRO, EPI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_gemm_decode: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr = smem;
  }
  me_launch(gemm_decode_kernel<PRO, EPI, TO>, dim3(strips), dim3(warps * 32), smem, stream, (const bf16*)X, ldx, res_in, norm_w,
            sumsq_in, sumsq_parts, eps, (const bf16*)W, (TO*)Y, ldy, res_out, sumsq_out, M, N, K);
  return 0;
}
}  // namespace

// Largest K the kernel covers inside one block.
ME_API int me_gemm_decode_max_k() { return DL_MAX_WARPS * DL_KW; }
// Parts of the sums of squares that the residual epilogue writes for N output columns.
ME_API int me_gemm_decode_sumsq_parts(int N) { return (N + 15) / 16; }

// pro 0: X bfloat16 [M][ldx]; pro 1: X = rmsnorm(res_in [M][K]) * norm_w with sums of squares sumsq_in [parts][M].
// epi 0: Y (y_dtype) [M][ldy]; epi 1: SiLU-and-multiply (weight rows gate | up, N = columns of Y);
// epi 2: res_out [M][N] += X W^T and sumsq_out [me_gemm_decode_sumsq_parts(N)][M].
ME_API int me_gemm_decode(int pro, int epi, const void* X, int64_t ldx, const float* res_in, const float* norm_w,
                          const float* sumsq_in, int sumsq_parts, float eps, const void* W, void* Y, int y_dtype,
                          int64_t ldy, float* res_out, float* sumsq_out, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && M <= 16, "me_gemm_decode: M=%d is not in 1..16", M);
  ME_REQUIRE(K % 8 == 0 && K > 0 && K <= DL_MAX_WARPS * DL_KW, "me_gemm_decode: K=%d must be a multiple of 8 up to %d", K,
             DL_MAX_WARPS * DL_KW);
  ME_REQUIRE((pro == 0 && X != nullptr && (ldx * 2) % 16 == 0) ||
                 (pro == 1 && res_in != nullptr && norm_w != nullptr && sumsq_in != nullptr && sumsq_parts > 0),
             "me_gemm_decode: operands of prologue %d are missing or misaligned", pro);
  ME_REQUIRE(epi == 0 || epi == 1 || (epi == 2 && res_out != nullptr && sumsq_out != nullptr), "me_gemm_decode: epilogue %d", epi);
  const int warps = (K + DL_KW - 1) / DL_KW;
  const int strips = epi == 1 ? (N + 7) / 8 : (N + 15) / 16;
  int rc = 1;
#define ME_DL(PRO_, EPI_, TO_)                                                                                      \
  rc = launch_dl<PRO_, EPI_, TO_>(strips, warps, stream, X, ldx, res_in, norm_w, sumsq_in, sumsq_parts, eps, W, Y, ldy, res_out, \
                                  sumsq_out, M, N, K)
  if (epi == 2) {
    if (pro == 0) ME_DL(0, 2, float); else ME_DL(1, 2, float);
  } else if (epi == 1) {
    ME_REQUIRE(y_dtype == ME_BF16, "me_gemm_decode: the SiLU epilogue writes bfloat16");
    if (pro == 0) ME_DL(0, 1, bf16); else ME_DL(1, 1, bf16);
  } else if (y_dtype == ME_BF16) {
    if (pro == 0) ME_DL(0, 0, bf16); else ME_DL(1, 0, bf16);
  } else {
    if (pro == 0) ME_DL(0, 0, float); else ME_DL(1, 0, float);
  }
#undef ME_DL
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_gemm_decode");
  return 0;
}
