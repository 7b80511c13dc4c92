// Products of a decode step (up to 16 rows) over ANY K, with the neighbouring element-wise work folded in:
// the kernel of gemm_decode.cu for layers whose rows are too long for one block to hold (K beyond 3,072: the
// 8B and 32B layer sizes) and for the vocabulary product at every size, where a product is a long stream of weights and what
// counts is bytes in flight.
//
// As there, the weight rows fill the M side of mma.sync m16n8k16, the batch sits on the N side, and the epilogues
// are the same three (see gemm_decode.cu): plain results; SiLU(gate) * up for a weight of rows gate | up
// (layers/activation.py:4-7 in the reference); residual += X W^T with the new residual's sums of squares and its
// product with the next norm's weight (the add of layers/layernorm.py:19-23 and half of the norm behind it);
// and, on the input side, results scaled by the row's rsqrt(mean square + eps) when X is such a pre-weighted
// residual (the other half of the norm in front: layers/layernorm.py:11-16).
//
// What differs is how the work is laid out.  The product is cut into stages of 128 weight rows by 128 elements of
// K (a group of 128 rows is walked along all of K, then the next group), and the stages are shared out evenly:
// block b of one block an SM takes stages [b T / blocks, (b + 1) T / blocks), so every SM streams the same
// number of bytes whatever N and K are.  One warp is the producer: it brings a stage's weights [128][128] and
// activations [8 or 16][128] in by tensor-map loads (64 columns a box, 128-byte swizzle, zero fill beyond N, M and K)
// into a ring of six or five stages: 192 or 160 KB of weights in flight an SM.  The boxes are as tall as the stage
// (two for the weights, two for the activations): what limits a stream of small boxes is the number of boxes an SM
// can ask for, not their bytes.  Each of the eight consumer warps owns 16 of the group's rows over all of K and keeps
// their sums in registers along the group; at its end the sums go through shared memory to the epilogue, while
// the producer is already stages ahead.  A group that spans several blocks belongs to the block that holds its
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

constexpr int GS_BK = 128, GS_ROWS = 128, GS_WARPS = GS_ROWS / 16, GS_CONSUMERS = GS_WARPS * 32, GS_THREADS = GS_CONSUMERS + 32;
constexpr int GS_SUB_BYTES = GS_ROWS * 128;                      // a sub-tile of the weights: [128 rows][64 columns]
constexpr int GS_W_BYTES = (GS_BK / 64) * GS_SUB_BYTES;          // a stage's weights
constexpr int GS_PARTIAL = GS_ROWS * 16;                         // floats a block leaves for the owner of a group
constexpr int GS_PER = GS_PARTIAL / GS_CONSUMERS;                // sums of a group that a consumer thread finishes
constexpr unsigned GS_FLAG_POLLS = 1u << 22;
template <int XR> constexpr int gs_stage_bytes() { return GS_W_BYTES + XR * GS_BK * 2; }
template <int XR> constexpr int gs_stages() { return XR == 8 ? 6 : 5; }

__host__ __device__ __forceinline__ long long gs_first_stage(long long total, int nb, int b) { return total * b / nb; }
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(GS_CONSUMERS) : "memory"); }

// EPI 0: Y[m][n] (bfloat16 or float32).  EPI 1: SiLU(gate) * up, bfloat16 (a group is 64 gate rows and their 64 up
// rows).  EPI 2: residual_out[m][n] += v; sumsq_out[block][m] = the block's share of the new residual's sums of
// squares; with ``next_w`` also xw_out[m][n] = residual_out[m][n] * next_w[n].
// XR: rows of the X tile and of map_x's boxes (8 for up to 8 rows of X: the upper n8 tile then reads one chunk of zeros).
// map_w has boxes of 128 rows (EPI 1: 64).
// partials: float32 [gridDim.x][GS_PARTIAL]; flags: int32 [gridDim.x], zero before the first launch and left zero.
template <int EPI, typename TO, int XR>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const float* __restrict__ sumsq_in, int sumsq_parts, float eps, TO* __restrict__ Y, int64_t ldy,
                   float* __restrict__ res_out, float* __restrict__ sumsq_out, const float* __restrict__ next_w,
                   bf16* __restrict__ xw_out, int M, int N, int K, int groups, float* __restrict__ partials,
                   int* __restrict__ flags, int* __restrict__ err) {
  constexpr int STAGES = gs_stages<XR>(), STAGE_BYTES = gs_stage_bytes<XR>();
  constexpr int COLS = EPI == 1 ? GS_ROWS / 2 : GS_ROWS;         // output columns of a group
  extern __shared__ unsigned char gs_smem_raw[];
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES];
  __shared__ float red[GS_ROWS][17];                 // a group's sums: [weight row][batch row]
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
    // ---- producer: a lane a box
    auto issue_w = [&](int item) {
      const long long t = t_lo + item;
      const int s = item % STAGES, grp = (int)(t / n_its), k0 = (int)(t % n_its) * GS_BK;
      unsigned char* dst = smem + s * STAGE_BYTES;
      if (lane == 0) tma::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
      __syncwarp();
      if (EPI == 1) {
        if (lane < 2 * (GS_BK / 64)) {               // sub-tile lane / 2 (64 columns): 64 gate rows, then their up rows
          const int sub = lane >> 1, half = lane & 1;
          tma::load_2d(dst + sub * GS_SUB_BYTES + half * (GS_SUB_BYTES / 2), &map_w, k0 + sub * 64,
                       half ? N + grp * COLS : grp * COLS, &full_bar[s]);
        }
      } else if (lane < GS_BK / 64) {                // sub-tile lane (64 columns), all rows in one box
        tma::load_2d(dst + lane * GS_SUB_BYTES, &map_w, k0 + lane * 64, grp * GS_ROWS, &full_bar[s]);
      }
    };
    auto issue_x = [&](int item) {
      const long long t = t_lo + item;
      const int s = item % STAGES, k0 = (int)(t % n_its) * GS_BK;
      if (lane >= 16 && lane < 16 + GS_BK / 64)
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
    // the rows' factors rsqrt(mean square + eps), from the partial sums in part order (warp w: rows w, w + GS_WARPS)
    for (int m = warp; m < 16; m += GS_WARPS) {
      float s = 0.f;
      if (sumsq_in != nullptr && m < M)
        for (int p = lane; p < sumsq_parts; p += 32) s += sumsq_in[(int64_t)p * M + m];
      s = warp_sum(s);
      if (lane == 0) row_scale[m] = sumsq_in != nullptr ? (m < M ? 1.0f / sqrtf(s / (float)K + eps) : 0.f) : 1.0f;
    }
    consumers_sync();
    float c[2][4] = {};
    const int mi = lane >> 3;                        // this warp: rows 16 warp .. + 15 of the group
    // this warp's sums for one group: rows 16 warp + r, column m of the batch
    auto put_sums = [&]() {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        red[warp * 16 + g][nt * 8 + 2 * t4] = c[nt][0];
        red[warp * 16 + g][nt * 8 + 2 * t4 + 1] = c[nt][1];
        red[warp * 16 + g + 8][nt * 8 + 2 * t4] = c[nt][2];
        red[warp * 16 + g + 8][nt * 8 + 2 * t4 + 1] = c[nt][3];
        c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
      }
    };
    for (int item = 0; item < total; ++item) {
      const long long t = t_lo + item;
      const int s = item % STAGES, it = (int)(t % n_its);
      if (ok) ok = tma::mbar_wait(&full_bar[s], (item / STAGES) & 1);
      if (ok) {
        bf16* ws = reinterpret_cast<bf16*>(smem + s * STAGE_BYTES);
        bf16* xs = reinterpret_cast<bf16*>(smem + s * STAGE_BYTES + GS_W_BYTES);
#pragma unroll
        for (int kk = 0; kk < GS_BK / 16; ++kk) {
          uint32_t a[4], b[4];
          const int pa = kk * 2 + (mi >> 1), pb = kk * 2 + (mi & 1);      // 16-byte pieces within the stage's K
          ldmatrix_x4(a, tma::swz128(ws + (pa >> 3) * (GS_ROWS * 64), warp * 16 + (mi & 1) * 8 + (lane & 7), pa & 7));
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
        for (int idx = tid; idx < GS_PARTIAL; idx += GS_CONSUMERS) mine[idx] = red[idx >> 4][idx & 15];
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
      float v[GS_PER];                               // thread tid: sums tid + i * GS_CONSUMERS = (row, m) of [128][16]
#pragma unroll
      for (int i = 0; i < GS_PER; ++i) {
        const int idx = tid + i * GS_CONSUMERS;
        v[i] = red[idx >> 4][idx & 15];
      }
      float old[EPI == 2 ? 16 / GS_WARPS : 1][GS_ROWS / 32];      // EPI 2: the residual's values, asked for before the waits
      if (EPI == 2) {
#pragma unroll
        for (int i = 0; i < 16 / GS_WARPS; ++i)
#pragma unroll
          for (int j = 0; j < GS_ROWS / 32; ++j) {
            const int m = warp + i * GS_WARPS, n = grp * GS_ROWS + lane + 32 * j;
            old[i][j] = m < M && n < N ? res_out[(int64_t)m * N + n] : 0.f;
          }
      }
      if (b_last > (int)blockIdx.x) {
        // a thread a block: wait for its flag and leave it clean for the next launch (the blocks of that launch set
        // theirs only after this grid has ended)
        for (int b = blockIdx.x + 1 + tid; b <= b_last; b += GS_CONSUMERS) {
          unsigned polls = 0;
          int seen = 0;
          do {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(seen) : "l"(flags + b) : "memory");
          } while (seen == 0 && ++polls < GS_FLAG_POLLS);
          if (seen == 0) atomicOr(err + 1, 1);
          flags[b] = 0;
        }
        consumers_sync();                            // all flags are seen: the sums behind them may be read
        // four blocks' sums asked for at a time (one trip to L2, not four), added in block order
        for (int b0 = blockIdx.x + 1; b0 <= b_last; b0 += 4) {
          float theirs[4][GS_PER];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const bool there = b0 + u <= b_last;
            const float* src = partials + (int64_t)(there ? b0 + u : b0) * GS_PARTIAL;
#pragma unroll
            for (int i = 0; i < GS_PER; ++i) theirs[u][i] = there ? __ldcg(src + tid + i * GS_CONSUMERS) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int i = 0; i < GS_PER; ++i) v[i] += theirs[u][i];
        }
      }
      // back into shared memory (a thread rewrites the places it read), scaled by the batch row's norm factor
#pragma unroll
      for (int i = 0; i < GS_PER; ++i) {
        const int idx = tid + i * GS_CONSUMERS;
        red[idx >> 4][idx & 15] = v[i] * row_scale[idx & 15];
      }
      consumers_sync();
      if (EPI == 1) {
        // rows 0..63 are gate, 64..127 their up rows; 64 consecutive threads: a batch row's consecutive columns
#pragma unroll
        for (int i = 0; i < COLS * 16 / GS_CONSUMERS; ++i) {
          const int idx = tid + i * GS_CONSUMERS, m = idx / COLS, r = idx % COLS;
          const int n = grp * COLS + r;
          if (m < M && n < N) {
            const float gate = red[r][m], up = red[COLS + r][m];
            Y[(int64_t)m * ldy + n] = from_f<TO>(gate / (1.0f + expf(-gate)) * up);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16 / GS_WARPS; ++i) {
          const int m = warp + i * GS_WARPS;         // a warp a batch row: 128 consecutive columns, 32 at a time
          float sq = 0.f;
#pragma unroll
          for (int j = 0; j < GS_ROWS / 32; ++j) {
            const int r = lane + 32 * j, n = grp * GS_ROWS + r;
            if (m < M && n < N) {
              float val = red[r][m];
              if (EPI == 2) {
                val += old[i][j];
                res_out[(int64_t)m * N + n] = val;
                sq += val * val;
                if (xw_out != nullptr) xw_out[(int64_t)m * N + n] = __float2bfloat16(val * next_w[n]);
              } else {
                Y[(int64_t)m * ldy + n] = from_f<TO>(val);
              }
            }
          }
          if (EPI == 2) {
            sq = warp_sum(sq);
            if (lane == 0 && m < M) sq_acc[m] += sq;               // one thread a row, groups in order
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
  const int groups = EPI == 1 ? (2 * N + GS_ROWS - 1) / GS_ROWS : (N + GS_ROWS - 1) / GS_ROWS, n_its = (K + GS_BK - 1) / GS_BK;
  me_launch(gemm_stream_kernel<EPI, TO, XR>, dim3(gs_blocks(groups, n_its)), dim3(GS_THREADS), smem, stream,
            *reinterpret_cast<const CUtensorMap*>(map_w), *reinterpret_cast<const CUtensorMap*>(map_x), sumsq_in, sumsq_parts, eps,
            (TO*)Y, ldy, res_out, sumsq_out, next_w, (bf16*)xw_out, M, N, K, groups, partials, flags, err);
  return 0;
}
}  // namespace

// Parts of the sums of squares that the residual epilogue writes for N output columns over K: one a block.
ME_API int me_gemm_stream_sumsq_parts(int N, int K) { return gs_blocks((N + GS_ROWS - 1) / GS_ROWS, (K + GS_BK - 1) / GS_BK); }
// Rows of the boxes that the caller's tensor maps must have: of W for an epilogue, of X for M rows.
ME_API int me_gemm_stream_w_box_rows(int epi) { return epi == 1 ? GS_ROWS / 2 : GS_ROWS; }
ME_API int me_gemm_stream_x_box_rows(int M) { return M <= 8 ? 8 : 16; }
// Floats and ints of the work buffers (``partials``, ``flags``) that a launch may use.
ME_API int me_gemm_stream_partial_floats() { return me_sm_count() * GS_PARTIAL; }
ME_API int me_gemm_stream_flag_ints() { return me_sm_count(); }

// Arguments as for me_gemm_decode (gemm_decode.cu), for any K that is a multiple of 8, with the operands given as
// tensor maps (me_tma_encode_2d, 64 columns a box, 128-byte swizzle): map_w over W [rows][K] with boxes of
// me_gemm_stream_w_box_rows(epi) rows,
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
