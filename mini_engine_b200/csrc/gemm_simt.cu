// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores, float32 accumulate, any sizes and any mix of
// float32 / bfloat16 operands.  This is the true 32-bit product of the float32 engine (plain
// FMA, no reduced-precision matrix mode) and the fallback of the bfloat16 engine for shapes
// or dtype mixes its tensor-core kernels refuse.  Each output element is summed over k in
// ascending order whatever M is, so a row's result does not depend on the rest of the batch.
//
// EPI 0: C = A W^T.  EPI 1: W has 2N rows (gate | up); C = silu(A Wg^T) * (A Wu^T)
// (layers/activation.py:4-7 folded into the product of layers/linear.py:45).
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, int64_t lda, const TW* __restrict__ W,
                 TO* __restrict__ C, int64_t ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[EPI == 1 ? BK : 1][BN + 4];
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4] = {}, acu[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + 256 * i, r = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      const int m = m0 + r, n = n0 + r;
      As[kk][r] = (m < M && k < K) ? to_f<TA>(A[(int64_t)m * lda + k]) : 0.f;
      Ws[kk][r] = (n < N && k < K) ? to_f<TW>(W[(int64_t)n * K + k]) : 0.f;
      if (EPI == 1) Us[kk][r] = (n < N && k < K) ? to_f<TW>(W[((int64_t)N + n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
      if (EPI == 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) u[j] = Us[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (EPI == 1) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (EPI == 1) v = v / (1.0f + expf(-v)) * acu[i][j];
      C[(int64_t)m * ldc + n] = from_f<TO>(v);
    }
  }
}

template <typename TA, typename TW, typename TO>
static int launch_simt(const void* A, int64_t lda, const void* W, void* C, int64_t ldc, int M, int N,
                       int K, int epi, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (epi == 0)
    me_launch(gemm_simt_kernel<TA, TW, TO, 0>, grid, dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, (TO*)C, ldc, M, N, K);
  else
    me_launch(gemm_simt_kernel<TA, TW, TO, 1>, grid, dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, (TO*)C, ldc, M, N, K);
  return 0;
}

// N is the number of output columns (for epi 1 the weight has 2N rows).
ME_API int me_gemm_simt(const void* A, int a_dtype, int64_t lda, const void* W, int w_dtype, void* C,
                        int c_dtype, int64_t ldc, int M, int N, int K, int epi, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && N > 0 && K > 0, "me_gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  ME_REQUIRE(epi == 0 || epi == 1, "me_gemm_simt: unknown epilogue %d", epi);
  ME_REQUIRE((M + BM - 1) / BM <= 65535, "me_gemm_simt: M=%d is too large", M);
  ME_DISPATCH_DTYPE(a_dtype, TA, ME_DISPATCH_DTYPE(w_dtype, TW, ME_DISPATCH_DTYPE(c_dtype, TO,
      (launch_simt<TA, TW, TO>(A, lda, W, C, ldc, M, N, K, epi, stream)))));
  ME_LAUNCH_CHECK("me_gemm_simt");
  return 0;
}
