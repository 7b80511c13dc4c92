// Y[M,N] = X[M,K] W[N,K]^T for a handful of rows (M <= 16): the products of a decode step, which
// are a stream of weights.  The weight rows fill the M side of mma.sync m16n8k16 (a strip of 16
// rows per block), the batch sits on the N side.  The four warps of a block split K between them
// (256 elements each, all of a warp's weights requested at once by cp.async, so a block has 32 KB
// in flight), their partial sums are added in warp order in shared memory; K beyond 1024 goes to
// further blocks (grid.y) whose float32 partial results [split][M][N] are summed, in order, by the
// kernel that consumes them (the residual add in front of the next RMSNorm).
//
// EPI 1: rows gate | up (layers/linear.py:29-45 packs them so); a strip holds 8 gate rows and
// their 8 up rows and writes silu(gate) * up (layers/activation.py:4-7).
#include "common.cuh"
#include "mma_prims.cuh"

namespace {
using namespace mma_prims;

constexpr int SK_THREADS = 128, SK_KW = 256, SK_PIECES = SK_KW / 8;   // per warp: 16 rows x 256 k

__device__ __forceinline__ bf16* sk_ptr(bf16* base, int row, int piece) {
  return base + row * SK_KW + ((piece ^ (row & 7)) << 3);
}

// XR: rows of the X tile, 16, or 8 for up to 8 rows of X (the upper n8 tile then reads one chunk of zeros): a
// block needs 48 KB instead of 64 KB, four share an SM instead of three, and a product with thousands of strips
// (the vocabulary) has a third more weights in flight.
template <int EPI, typename TO, int XR>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const bf16* __restrict__ X, int64_t ldx, const bf16* __restrict__ W, TO* __restrict__ Y,
                   int64_t ldy, float* __restrict__ partial, int M, int N, int K) {
  extern __shared__ __align__(128) unsigned char sk_smem[];
  __shared__ float red[4][16][17];
  __shared__ __align__(16) bf16 zero_chunk[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  if (tid < 8) zero_chunk[tid] = __float2bfloat16_rn(0.f);
  bf16* ws = reinterpret_cast<bf16*>(sk_smem) + warp * (16 + XR) * SK_KW;  // this warp's W tile [16][256]
  bf16* xs = ws + 16 * SK_KW;                                              // this warp's X tile [XR][256]
  const int strip = blockIdx.x;
  const int k0 = (blockIdx.y * 4 + warp) * SK_KW;
  // rows of W in this strip
  auto w_row = [&](int r) -> int64_t {
    if (EPI == 1) return r < 8 ? (int64_t)strip * 8 + r : (int64_t)N + strip * 8 + (r - 8);
    return (int64_t)strip * 16 + r;
  };
  const int n_rows = EPI == 1 ? 2 * N : N;
  // The weights do not depend on the kernel before this one: they are on their way before it has finished.
  for (int c = lane; c < 16 * SK_PIECES; c += 32) {
    const int row = c / SK_PIECES, piece = c % SK_PIECES;
    const int k = k0 + piece * 8;
    const int64_t wr = w_row(row);
    const bool okw = k < K && wr < n_rows && (EPI == 0 || strip * 8 + (row & 7) < N);
    cp_async16(sk_ptr(ws, row, piece), okw ? W + wr * K + k : W, okw);
  }
  pdl_wait();
  pdl_launch_dependents();
  for (int c = lane; c < XR * SK_PIECES; c += 32) {
    const int row = c / SK_PIECES, piece = c % SK_PIECES;
    const int k = k0 + piece * 8;
    const bool okx = k < K && row < M;
    cp_async16(sk_ptr(xs, row, piece), okx ? X + (int64_t)row * ldx + k : X, okx);
  }
  cp_async_commit();
  cp_async_wait<0>();
  if (XR == 8) __syncthreads();                      // (the chunk of zeros is another warp's write)
  __syncwarp();
  float c[2][4] = {};
  const int mi = lane >> 3;
  if (k0 < K) {
#pragma unroll
    for (int kk = 0; kk < SK_KW / 16; ++kk) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, sk_ptr(ws, (mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1)));
      ldmatrix_x4(b, (XR == 8 && (mi >> 1)) ? zero_chunk : sk_ptr(xs, (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
      mma_bf16(c[0], a, b[0], b[1]);
      mma_bf16(c[1], a, b[2], b[3]);
    }
  }
  // c[nt][0..1]: weight row g, batch rows nt*8 + 2*t4, +1;  c[nt][2..3]: weight row g + 8
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    red[warp][g][nt * 8 + 2 * t4] = c[nt][0];
    red[warp][g][nt * 8 + 2 * t4 + 1] = c[nt][1];
    red[warp][g + 8][nt * 8 + 2 * t4] = c[nt][2];
    red[warp][g + 8][nt * 8 + 2 * t4 + 1] = c[nt][3];
  }
  __syncthreads();
  const bool split = gridDim.y > 1;
  if (EPI == 0) {
    for (int idx = tid; idx < 16 * 16; idx += SK_THREADS) {
      const int m = idx >> 4, r = idx & 15;                       // consecutive threads: consecutive columns
      const int n = strip * 16 + r;
      if (m >= M || n >= N) continue;
      const float v = ((red[0][r][m] + red[1][r][m]) + red[2][r][m]) + red[3][r][m];
      if (split) partial[((int64_t)blockIdx.y * M + m) * N + n] = v;
      else Y[(int64_t)m * ldy + n] = from_f<TO>(v);
    }
  } else {
    for (int idx = tid; idx < 16 * 8; idx += SK_THREADS) {
      const int m = idx >> 3, r = idx & 7;
      const int n = strip * 8 + r;
      if (m >= M || n >= N) continue;
      const float gate = ((red[0][r][m] + red[1][r][m]) + red[2][r][m]) + red[3][r][m];
      const float up = ((red[0][r + 8][m] + red[1][r + 8][m]) + red[2][r + 8][m]) + red[3][r + 8][m];
      Y[(int64_t)m * ldy + n] = from_f<TO>(gate / (1.0f + expf(-gate)) * up);
    }
  }
}

template <int EPI, typename TO, int XR>
int launch_skinny(const void* X, int64_t ldx, const void* W, void* Y, int64_t ldy, float* partial, int M, int N,
                  int K, int strips, int splits, cudaStream_t stream) {
  const size_t smem = (size_t)4 * (16 + XR) * SK_KW * sizeof(bf16);    // 64 KB, or 48 KB with 8 rows of X
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<EPI, TO, XR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_gemm_skinny: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  me_launch(gemm_skinny_kernel<EPI, TO, XR>, dim3(strips, splits), dim3(SK_THREADS), smem, stream,
      (const bf16*)X, ldx, (const bf16*)W, (TO*)Y, ldy, partial, M, N, K);
  return 0;
}
}  // namespace

// How many float32 partial results [split][M][N] the product leaves for its consumer (1: none, Y is final).
ME_API int me_gemm_skinny_splits(int K) { return (K + 4 * SK_KW - 1) / (4 * SK_KW); }

// N counts output columns (epi 1: the weight has 2N rows).  With me_gemm_skinny_splits(K) > 1 the caller
// passes ``partial`` (float32 [splits][M][N]) and Y is not written; epi 1 needs K <= 1024.
ME_API int me_gemm_skinny(const void* X, int64_t ldx, const void* W, void* Y, int y_dtype, int64_t ldy,
                          float* partial, int M, int N, int K, int epi, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && M <= 16, "me_gemm_skinny: M=%d is not in 1..16", M);
  ME_REQUIRE(K % 8 == 0 && (ldx * 2) % 16 == 0, "me_gemm_skinny: K=%d and the row stride must be multiples of 8 elements", K);
  ME_REQUIRE(epi == 0 || epi == 1, "me_gemm_skinny: unknown epilogue %d", epi);
  const int splits = me_gemm_skinny_splits(K);
  ME_REQUIRE(splits == 1 || (epi == 0 && partial != nullptr), "me_gemm_skinny: K=%d needs a buffer for partial results", K);
  ME_REQUIRE(splits <= 65535, "me_gemm_skinny: K too large");
  const int strips = epi == 1 ? (N + 7) / 8 : (N + 15) / 16;
  int rc;
  if (epi == 1) {
    ME_REQUIRE(y_dtype == ME_BF16, "me_gemm_skinny: the SiLU epilogue writes bfloat16");
    rc = M <= 8 ? launch_skinny<1, bf16, 8>(X, ldx, W, Y, ldy, partial, M, N, K, strips, splits, stream)
                : launch_skinny<1, bf16, 16>(X, ldx, W, Y, ldy, partial, M, N, K, strips, splits, stream);
  } else if (y_dtype == ME_BF16) {
    rc = M <= 8 ? launch_skinny<0, bf16, 8>(X, ldx, W, Y, ldy, partial, M, N, K, strips, splits, stream)
                : launch_skinny<0, bf16, 16>(X, ldx, W, Y, ldy, partial, M, N, K, strips, splits, stream);
  } else {
    rc = M <= 8 ? launch_skinny<0, float, 8>(X, ldx, W, Y, ldy, partial, M, N, K, strips, splits, stream)
                : launch_skinny<0, float, 16>(X, ldx, W, Y, ldy, partial, M, N, K, strips, splits, stream);
  }
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_gemm_skinny");
  return 0;
}
