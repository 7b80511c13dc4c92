// Products of a decode step (up to 16 rows) over ANY K, with the neighbouring element-wise work folded in:
// the kernel of gemm_decode.cu for layers whose rows are too long for one block to hold (K beyond 3,072: the
// 8B and 32B layer sizes), where a product is a long stream of weights and what counts is bytes in flight.
//
// As there, the weight rows fill the M side of mma.sync m16n8k16, the batch sits on the N side, and the epilogues
// are the same three (see gemm_decode.cu): plain results; SiLU(gate) * up for a weight of rows gate | up
// (layers/activation.py:4-7 in the reference); residual += X W^T with the new residual's sums of squares and its
// product with the next norm's weight (the add of layers/layernorm.py:19-23 and half of the norm behind it);
// and, on the input side, results scaled by the row's rsqrt(mean square + eps) when X is such a pre-weighted
// residual (the other half of the norm in front: layers/layernorm.py:11-16).
//
// What differs is how the work is laid out.  The product is cut into stages of 32 weight rows by 512 elements of
// K (a group of 32 rows is walked along all of K, then the next group), and the stages are shared out evenly:
// block b of one block an SM takes stages [b T / blocks, (b + 1) T / blocks), so every SM streams the same
// number of bytes whatever N and K are.  A fifth warp is the producer: it brings a stage's weights [32][512] and
// activations [8 or 16][512] in by tensor-map loads (boxes of 64 columns, 128-byte swizzle, zero fill beyond N, M
// and K; a lane a box) into a ring of five or four stages: 128 or 96 KB of weights in flight an SM.  The four
// consumer warps are two halves of the rows by two halves of the stage's K; they keep their sums in registers
// along a group and at its end add them in a fixed order in shared memory and run the epilogue, while the
// producer is already stages ahead.  A group that spans several blocks belongs to the block that holds its
// beginning: that block reaches the group last of all it does, while the blocks behind it walk their piece of
// the group first of all they do, leave their sums in a work buffer and set a flag; so when the owner asks for
// the flags (all blocks are resident: one an SM) they are long set.  It adds its own sums, then theirs in block
// order, clears the flags and runs the epilogue: every output element is finished by one block, with no atomics
// and a fixed order of summation.
// Every wait is bounded; a wait that gives up sets flag 1 of ``err``.
#include "common.cuh"
#include "mma_prims.cuh"
#include "tma.cuh"

namespace {
using namespace mma_prims;

constexpr int GS_BK = 512, GS_KW = 256, GS_ROWS = 32, GS_WARPS = 4, GS_THREADS = (GS_WARPS + 1) * 32;
constexpr int GS_W_BYTES = GS_ROWS * GS_BK * 2;                  // a stage's weights: 8 sub-tiles of [32 rows][64]
constexpr int GS_PARTIAL = GS_ROWS * 16;                         // floats a block leaves for the owner of a group
constexpr unsigned GS_FLAG_POLLS = 1u << 22;
template <int XR> constexpr int gs_stage_bytes() { return GS_W_BYTES + XR * GS_BK * 2; }
template <int XR> constexpr int gs_stages() { return XR == 8 ? 5 : 4; }

__host__ __device__ __forceinline__ long long gs_first_stage(long long total, int nb, int b) { return total * b / nb; }
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(GS_WARPS * 32) : "memory"); }

// EPI 0: Y[m][n] (bfloat16 or float32).  EPI 1: SiLU(gate) * up, bfloat16 (a group is 16 gate rows and their 16 up
// rows).  EPI 2: residual_out[m][n] += v; sumsq_out[block][m] = the block's share of the new residual's sums of
// squares; with ``next_w`` also xw_out[m][n] = residual_out[m][n] * next_w[n].
// XR: rows of the X tile and of map_x's boxes (8 for up to 8 rows of X: the upper n8 tile then reads one chunk of zeros).
// partials: float32 [gridDim.x][GS_PARTIAL]; flags: int32 [gridDim.x], zero before the first launch and left zero.
template <int EPI, typename TO, int XR>
__global__ void __launch_bounds__(GS_THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const float* __restrict__ sumsq_in, int sumsq_parts, float eps, TO* __restrict__ Y, int64_t ldy,
                   float* __restrict__ res_out, float* __restrict__ sumsq_out, const float* __restrict__ next_w,
                   bf16* __restrict__ xw_out, int M, int N, int K, int groups, float* __restrict__ partials,
                   int* __restrict__ flags, int* __restrict__ err) {
  constexpr int STAGES = gs_stages<XR>(), STAGE_BYTES = gs_stage_bytes<XR>();
  constexpr int COLS = EPI == 1 ? 16 : 32;           // output columns of a group
  extern __shared__ unsigned char gs_smem_raw[];
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
  __shared__ float red[GS_WARPS][16][17];
  __shared__ float row_scale[16];
  __shared__ float sq_acc[16];                       // EPI 2: this block's sums of squares of the new residual, per row
  __shared__ __align__(16) bf16 zero_chunk[8];
  unsigned char* smem = gs_smem_raw + ((1024u - (tma::smem_addr(gs_smem_raw) & 1023u)) & 1023u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const int n_its = (K + GS_BK - 1) / GS_BK, nb = gridDim.x;
  const long long T = (long long)groups * n_its;
  const long long t_lo = gs_first_stage(T, nb, blockIdx.x), t_hi = gs_first_stage(T, nb, blockIdx.x + 1);
  const int total = (int)(t_hi - t_lo);              // stages of this block
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tma::mbar_init(&full_bar[s], 1);
      tma::mbar_init(&empty_bar[s], GS_WARPS);
    }
    tma::mbar_fence_init();
    tma::prefetch_map(&map_w);
    tma::prefetch_map(&map_x);
  }
  if (tid < 8) zero_chunk[tid] = __float2bfloat16_rn(0.f);
  if (tid < 16) sq_acc[tid] = 0.f;
  __syncthreads();
  bool ok = true;

  if (warp == GS_WARPS) {
    // ---- producer: lanes 0..15 bring in the weights' 16 boxes of a stage, lanes 16..23 the activations' 8
    auto issue_w = [&](int item) {
      const long long t = t_lo + item;
      const int s = item % STAGES, grp = (int)(t / n_its), k0 = (int)(t % n_its) * GS_BK;
      unsigned char* dst = smem + s * STAGE_BYTES;
      if (lane == 0) tma::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
      __syncwarp();
      if (lane < 16) {                               // sub-tile lane / 2 (64 columns), rows 16 (lane & 1) .. + 15
        const int sub = lane >> 1, half = lane & 1;
        const int row = EPI == 1 ? (half ? N + grp * 16 : grp * 16) : grp * 32 + half * 16;
        tma::load_2d(dst + sub * 4096 + half * 2048, &map_w, k0 + sub * 64, row, &full_bar[s]);
      }
    };
    auto issue_x = [&](int item) {
      const long long t = t_lo + item;
      const int s = item % STAGES, k0 = (int)(t % n_its) * GS_BK;
      if (lane >= 16 && lane < 24)
        tma::load_2d(smem + s * STAGE_BYTES + GS_W_BYTES + (lane - 16) * (XR * 128), &map_x, k0 + (lane - 16) * 64, 0, &full_bar[s]);
    };
    // The weights are no output of the kernel before this one: the ring's first stages are asked for before it has
    // finished; the activations after.
    const int ahead = total < STAGES ? total : STAGES;
    for (int item = 0; item < ahead; ++item) issue_w(item);
    pdl_wait();
    pdl_launch_dependents();
    for (int item = 0; item < ahead; ++item) issue_x(item);
    for (int item = ahead; item < total && ok; ++item) {
      ok = tma::mbar_wait(&empty_bar[item % STAGES], ((item / STAGES) & 1) ^ 1);
      if (!ok) break;
      issue_w(item);
      issue_x(item);
    }
  } else {
    pdl_wait();
    pdl_launch_dependents();
    // the rows' factors rsqrt(mean square + eps), from the partial sums in part order (warp w: rows w, w + 4, ...)
    for (int m = warp; m < 16; m += GS_WARPS) {
      float s = 0.f;
      if (sumsq_in != nullptr && m < M)
        for (int p = lane; p < sumsq_parts; p += 32) s += sumsq_in[(int64_t)p * M + m];
      s = warp_sum(s);
      if (lane == 0) row_scale[m] = sumsq_in != nullptr ? (m < M ? 1.0f / sqrtf(s / (float)K + eps) : 0.f) : 1.0f;
    }
    consumers_sync();
    float c[2][4] = {};
    const int mi = lane >> 3, rg = warp & 1, kh = warp >> 1;     // this warp: rows 16 rg .. + 15, K half kh of the stage
    // sums of this block's warps for one group, K halves in order: rows 16 rg + r, column m of the batch
    auto put_sums = [&]() {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        red[warp][g][nt * 8 + 2 * t4] = c[nt][0];
        red[warp][g][nt * 8 + 2 * t4 + 1] = c[nt][1];
        red[warp][g + 8][nt * 8 + 2 * t4] = c[nt][2];
        red[warp][g + 8][nt * 8 + 2 * t4 + 1] = c[nt][3];
        c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
      }
    };
    auto sum_of = [&](int row, int m) { return red[row >> 4][row & 15][m] + red[2 + (row >> 4)][row & 15][m]; };
    for (int item = 0; item < total; ++item) {
      const long long t = t_lo + item;
      const int s = item % STAGES, it = (int)(t % n_its);
      if (ok) ok = tma::mbar_wait(&full_bar[s], (item / STAGES) & 1);
      if (ok && it * GS_BK + kh * GS_KW < K) {
        bf16* ws = reinterpret_cast<bf16*>(smem + s * STAGE_BYTES) + kh * 4 * (GS_ROWS * 64);      // this K half's four sub-tiles
        bf16* xs = reinterpret_cast<bf16*>(smem + s * STAGE_BYTES + GS_W_BYTES) + kh * 4 * (XR * 64);
#pragma unroll
        for (int kk = 0; kk < GS_KW / 16; ++kk) {
          uint32_t a[4], b[4];
          const int pa = kk * 2 + (mi >> 1), pb = kk * 2 + (mi & 1);      // 16-byte pieces within the 256 elements
          ldmatrix_x4(a, tma::swz128(ws + (pa >> 3) * (GS_ROWS * 64), rg * 16 + (mi & 1) * 8 + (lane & 7), pa & 7));
          ldmatrix_x4(b, (XR == 8 && (mi >> 1)) ? zero_chunk : tma::swz128(xs + (pb >> 3) * (XR * 64), (mi >> 1) * 8 + (lane & 7), pb & 7));
          mma_bf16(c[0], a, b[0], b[1]);
          mma_bf16(c[1], a, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tma::smem_addr(&empty_bar[s])) : "memory");
      const bool group_ends = it == n_its - 1, block_ends = item == total - 1;
      if (!group_ends && !block_ends) continue;
      put_sums();
      consumers_sync();
      const int grp = (int)(t / n_its);
      const long long t0 = (long long)grp * n_its;   // the group's first stage
      if (t0 < t_lo) {
        // ---- the group began in an earlier block (this block walked its end, or a piece of its middle): leave the sums
        // for that block, which gets to the group last of all it does
        float* mine = partials + (int64_t)blockIdx.x * GS_PARTIAL;
        for (int idx = tid; idx < GS_PARTIAL; idx += GS_WARPS * 32) mine[idx] = sum_of(idx >> 4, idx & 15);
        __threadfence();
        consumers_sync();
        if (tid == 0) asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(flags + blockIdx.x), "r"(1) : "memory");
        continue;
      }
      // ---- the group began in this block: its sums, then those of the blocks that walked the rest of it, in block order
      int b_last = blockIdx.x;
      if (!group_ends) {
        const long long t_end = t0 + n_its - 1;
        b_last = (int)(t_end * nb / T);
        while (b_last > 0 && gs_first_stage(T, nb, b_last) > t_end) --b_last;
        while (gs_first_stage(T, nb, b_last + 1) <= t_end) ++b_last;
      }
      float v4[GS_PARTIAL / (GS_WARPS * 32)];
#pragma unroll
      for (int i = 0; i < GS_PARTIAL / (GS_WARPS * 32); ++i) {
        const int idx = tid + i * GS_WARPS * 32;
        v4[i] = sum_of(idx >> 4, idx & 15);
      }
      for (int b = blockIdx.x + 1; b <= b_last; ++b) {
        if (ok) {
          unsigned polls = 0;
          int seen = 0;
          do {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(seen) : "l"(flags + b) : "memory");
          } while (seen == 0 && ++polls < GS_FLAG_POLLS);
          ok = seen != 0;
        }
        const float* theirs = partials + (int64_t)b * GS_PARTIAL;
#pragma unroll
        for (int i = 0; i < GS_PARTIAL / (GS_WARPS * 32); ++i) v4[i] += __ldcg(theirs + tid + i * GS_WARPS * 32);
      }
      if (b_last > (int)blockIdx.x) {
        consumers_sync();                            // every thread has seen the flags and read the sums
        for (int b = blockIdx.x + 1 + tid; b <= b_last; b += GS_WARPS * 32) flags[b] = 0;      // left clean for the next launch
      }
#pragma unroll
      for (int i = 0; i < GS_PARTIAL / (GS_WARPS * 32); ++i) {
        const int m = (tid + i * GS_WARPS * 32) & 15;        // (16 consecutive threads: a weight row)
        v4[i] *= row_scale[m];
      }
      if (EPI == 1) {
        // rows 0..15 are gate, 16..31 their up rows: thread (row, m) of the first half needs the up value of row + 16,
        // which thread tid of round i + 2 holds: through shared memory
        consumers_sync();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = tid + i * GS_WARPS * 32;
          red[idx >> 8][(idx >> 4) & 15][idx & 15] = v4[i];
        }
        consumers_sync();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int idx = tid + i * GS_WARPS * 32, m = idx >> 4, r = idx & 15;      // 16 consecutive threads: consecutive columns
          const int n = grp * 16 + r;
          if (m < M && n < N) {
            const float gate = red[0][r][m], up = red[1][r][m];
            Y[(int64_t)m * ldy + n] = from_f<TO>(gate / (1.0f + expf(-gate)) * up);
          }
        }
      } else {
        // results (row n, batch m) sit 16 threads a weight row; through shared memory to 32 threads a batch row
        consumers_sync();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = tid + i * GS_WARPS * 32;
          red[idx >> 8][(idx >> 4) & 15][idx & 15] = v4[i];        // [row / 16][row % 16][m]
        }
        consumers_sync();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int m = warp + i * GS_WARPS, r = lane;             // a warp a batch row: 32 consecutive columns
          const int n = grp * 32 + r;
          const bool live = m < M && n < N;
          float v = live ? red[r >> 4][r & 15][m] : 0.f;
          if (EPI == 2) {
            float sq = 0.f;
            if (live) {
              v += res_out[(int64_t)m * N + n];
              res_out[(int64_t)m * N + n] = v;
              sq = v * v;
              if (xw_out != nullptr) xw_out[(int64_t)m * N + n] = __float2bfloat16(v * next_w[n]);
            }
            sq = warp_sum(sq);
            if (lane == 0 && m < M) sq_acc[m] += sq;               // one thread a row, groups in order
          } else if (live) {
            Y[(int64_t)m * ldy + n] = from_f<TO>(v);
          }
        }
      }
      consumers_sync();                              // the sums are read: the next group may overwrite them
    }
    if (EPI == 2 && tid < M) sumsq_out[(int64_t)blockIdx.x * M + tid] = sq_acc[tid];
  }
  if (!ok && lane == 0) atomicOr(err + 1, 1);
}

int gs_blocks(int groups, int n_its) {
  const long long T = (long long)groups * n_its;
  return (int)(T < me_sm_count() ? T : me_sm_count());
}

template <int EPI, typename TO, int XR>
int launch_gs(cudaStream_t stream, const void* map_w, const void* map_x, const float* sumsq_in, int sumsq_parts, float eps, void* Y,
              int64_t ldy, float* res_out, float* sumsq_out, const float* next_w, void* xw_out, int M, int N, int K,
              float* partials, int* flags, int* err) {
  const size_t smem = (size_t)gs_stages<XR>() * gs_stage_bytes<XR>() + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<EPI, TO, XR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_gemm_stream: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  const int groups = EPI == 1 ? (N + 15) / 16 : (N + 31) / 32, n_its = (K + GS_BK - 1) / GS_BK;
  me_launch(gemm_stream_kernel<EPI, TO, XR>, dim3(gs_blocks(groups, n_its)), dim3(GS_THREADS), smem, stream,
            *reinterpret_cast<const CUtensorMap*>(map_w), *reinterpret_cast<const CUtensorMap*>(map_x), sumsq_in, sumsq_parts, eps,
            (TO*)Y, ldy, res_out, sumsq_out, next_w, (bf16*)xw_out, M, N, K, groups, partials, flags, err);
  return 0;
}
}  // namespace

// Parts of the sums of squares that the residual epilogue writes for N output columns over K: one a block.
ME_API int me_gemm_stream_sumsq_parts(int N, int K) { return gs_blocks((N + 31) / 32, (K + GS_BK - 1) / GS_BK); }
// Rows of the boxes that the caller's tensor maps must have: of W (always 16), of X for M rows.
ME_API int me_gemm_stream_w_box_rows() { return 16; }
ME_API int me_gemm_stream_x_box_rows(int M) { return M <= 8 ? 8 : 16; }
// Floats and ints of the work buffers (``partials``, ``flags``) that a launch may use.
ME_API int me_gemm_stream_partial_floats() { return me_sm_count() * GS_PARTIAL; }
ME_API int me_gemm_stream_flag_ints() { return me_sm_count(); }

// Arguments as for me_gemm_decode (gemm_decode.cu), for any K that is a multiple of 8, with the operands given as
// tensor maps (me_tma_encode_2d, 64 columns a box, 128-byte swizzle): map_w over W [rows][K] with boxes of 16 rows,
// map_x over X [M][K] with boxes of me_gemm_stream_x_box_rows(M) rows.  sumsq_out is
// [me_gemm_stream_sumsq_parts(N, K)][M].  partials / flags: work buffers of me_gemm_stream_partial_floats() floats and
// me_gemm_stream_flag_ints() ints; the flags are zero before the first launch and every launch leaves them zero (launches
// that share them must not overlap on the device).  err: int32[4]; flag 1 is set when a wait ran out.
ME_API int me_gemm_stream(int epi, const void* map_x, const float* sumsq_in, int sumsq_parts, float eps, const void* map_w,
                          void* Y, int y_dtype, int64_t ldy, float* res_out, float* sumsq_out, const float* next_w,
                          void* xw_out, int M, int N, int K, float* partials, int* flags, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && M <= 16, "me_gemm_stream: M=%d is not in 1..16", M);
  ME_REQUIRE(K % 8 == 0 && K > 0, "me_gemm_stream: K=%d must be a positive multiple of 8", K);
  ME_REQUIRE(map_x != nullptr && map_w != nullptr && err != nullptr && partials != nullptr && flags != nullptr,
             "me_gemm_stream: tensor maps, work buffers and the error word are required");
  ME_REQUIRE(sumsq_in == nullptr || sumsq_parts > 0, "me_gemm_stream: sums of squares in %d parts", sumsq_parts);
  ME_REQUIRE(epi == 0 || epi == 1 || (epi == 2 && res_out != nullptr && sumsq_out != nullptr), "me_gemm_stream: epilogue %d", epi);
  ME_REQUIRE((next_w == nullptr) == (xw_out == nullptr) && (next_w == nullptr || epi == 2),
             "me_gemm_stream: the pre-weighted copy needs the residual epilogue, a weight and an output");
  int rc = 1;
#define ME_GS(EPI_, TO_)                                                                                                      \
  rc = M <= 8 ? launch_gs<EPI_, TO_, 8>(stream, map_w, map_x, sumsq_in, sumsq_parts, eps, Y, ldy, res_out, sumsq_out, next_w,  \
                                        xw_out, M, N, K, partials, flags, err)                                                 \
              : launch_gs<EPI_, TO_, 16>(stream, map_w, map_x, sumsq_in, sumsq_parts, eps, Y, ldy, res_out, sumsq_out, next_w, \
                                         xw_out, M, N, K, partials, flags, err)
  if (epi == 2) {
    ME_GS(2, float);
  } else if (epi == 1) {
    ME_REQUIRE(y_dtype == ME_BF16, "me_gemm_stream: the SiLU epilogue writes bfloat16");
    ME_GS(1, bf16);
  } else if (y_dtype == ME_BF16) {
    ME_GS(0, bf16);
  } else {
    ME_GS(0, float);
  }
#undef ME_GS
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_gemm_stream");
  return 0;
}
