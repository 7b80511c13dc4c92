// C[M,N] = A[M,K] W[N,K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05), for many rows
// (portions of prompts).  The reference leaves these products to cuBLAS through F.linear
// (layers/linear.py:26,45); this kernel is the engine's own, with SiLU-and-multiply
// (layers/activation.py:4-7) in its epilogue and float32 results for the output head.
//
// One block computes a 128 x BN tile.  Warp 0: one thread streams A and W tiles of 64 K-elements
// through a ring of shared-memory stages by TMA (128-byte swizzle, zero fill at the edges).
// Warp 1: allocates BN columns of tensor memory; one thread issues tcgen05.mma (M 128, N BN, K 16,
// four per stage) and hands stages back through tcgen05.commit.  Warps 2..5: when the accumulator is
// complete, each thread reads its row from tensor memory (tcgen05.ld), applies the epilogue and writes
// it.  Every wait is bounded; a wait that gives up sets flag 1 of ``err`` and the block still frees its
// tensor memory and exits.
//
// EPI 1: W has rows gate | up; a stage's W tile holds BN/2 gate rows and the matching BN/2 up rows, so
// the accumulator's first half is gate and its second half up, and the block writes BN/2 columns of
// silu(gate) * up.
#include "tcgen05.cuh"

namespace {

constexpr int TG_BM = 128, TG_BK = 64, TG_THREADS = 192;
constexpr int TG_A_BYTES = TG_BM * TG_BK * 2;

// Stages sized so that two blocks fit on an SM (about 96 KB each): one block's epilogue overlaps the other's main loop.
// A grid of no more blocks than SMs has the SM to itself and takes twice the stages: what bounds these products
// is the bytes a block has on their way from L2.
template <int BN> constexpr int tg_stages(bool deep) { return (BN <= 64 ? 4 : (BN <= 128 ? 3 : 2)) * (deep ? 2 : 1); }

// 32 consecutive results of one row: 16-byte stores where the row's place allows, else one by one.
__device__ __forceinline__ void store_row32(bf16* dst, const float (&v)[32], int n_left, bool vec) {
  if (vec && n_left >= 32) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 pk;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[q * 8 + 2 * j], v[q * 8 + 2 * j + 1]);
      *reinterpret_cast<uint4*>(dst + q * 8) = pk;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < n_left) dst[j] = __float2bfloat16_rn(v[j]);
  }
}
__device__ __forceinline__ void store_row32(float* dst, const float (&v)[32], int n_left, bool vec) {
  if (vec && n_left >= 32) {
#pragma unroll
    for (int q = 0; q < 8; ++q)
      *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < n_left) dst[j] = v[j];
  }
}

// gridDim.z blocks share a tile: block z takes ``kb_per_split`` blocks of 64 along K from z * kb_per_split on and writes
// its partial result ``split_stride`` elements after the one before (float32 results that the next kernel adds).
template <int BN, int EPI, typename TO, bool DEEP>
__global__ void __launch_bounds__(TG_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    TO* __restrict__ C, int64_t ldc, int M, int N, int K, int kb_per_split, int64_t split_stride,
                    int* __restrict__ err) {
  constexpr int STAGES = tg_stages<BN>(DEEP);
  constexpr int B_BYTES = BN * TG_BK * 2, STAGE_BYTES = TG_A_BYTES + B_BYTES;
  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
  extern __shared__ unsigned char tg_smem_raw[];
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], done_bar;
  __shared__ uint32_t tmem_slot;
  unsigned char* smem = tg_smem_raw + ((1024u - (tma::smem_addr(tg_smem_raw) & 1023u)) & 1023u);
  const int warp = tc5::uniform_warp_index(), lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TG_BM, n0 = blockIdx.x * OUT_COLS;
  const int kb0 = blockIdx.z * kb_per_split;
  const int num_kb = min(kb_per_split, (K + TG_BK - 1) / TG_BK - kb0);
  C += blockIdx.z * split_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tma::mbar_init(&full_bar[s], 1);
      tma::mbar_init(&empty_bar[s], 1);
    }
    tma::mbar_init(&done_bar, 1);
    tma::mbar_fence_init();
    tma::prefetch_map(&map_a);
    tma::prefetch_map(&map_w);
  }
  if (warp == 1) tc5::tmem_alloc(&tmem_slot, BN < 32 ? 32 : BN);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      // The weights are no output of the kernel before this one; the activations are.
      bool waited = false;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        ok = tma::mbar_wait(&empty_bar[s], ((kb / STAGES) & 1) ^ 1);
        if (!ok) break;
        unsigned char* a_dst = smem + s * STAGE_BYTES;
        unsigned char* b_dst = a_dst + TG_A_BYTES;
        tma::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        if (EPI == 1) {
          tma::load_2d(b_dst, &map_w, (kb0 + kb) * TG_BK, n0, &full_bar[s]);
          tma::load_2d(b_dst + B_BYTES / 2, &map_w, (kb0 + kb) * TG_BK, N + n0, &full_bar[s]);
        } else {
          tma::load_2d(b_dst, &map_w, (kb0 + kb) * TG_BK, n0, &full_bar[s]);
        }
        if (!waited && (kb == STAGES - 1 || kb == num_kb - 1)) {
          // first ring of weights requested: now wait for the predecessor and send the held-back A tiles
          pdl_wait();
          waited = true;
          for (int k2 = 0; k2 <= kb; ++k2)
            tma::load_2d(smem + (k2 % STAGES) * STAGE_BYTES, &map_a, (kb0 + k2) * TG_BK, m0, &full_bar[k2 % STAGES]);
        } else if (waited) {
          tma::load_2d(a_dst, &map_a, (kb0 + kb) * TG_BK, m0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // all lanes run the loop, an elected one issues
    constexpr uint32_t idesc = tc5::instr_desc_bf16(TG_BM, BN);
    const tc5::DescWords a_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(smem));
    const tc5::DescWords b_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(smem + TG_A_BYTES));
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % STAGES;
      ok = tc5::mbar_wait_warp(&full_bar[s], (kb / STAGES) & 1);
      if (!ok) break;
      tc5::fence_after_sync();
      const uint32_t stage = (uint32_t)(s * STAGE_BYTES) >> 4;
#pragma unroll
      for (int k = 0; k < TG_BK / 16; ++k)         // 32 bytes further along K per step: +2 in units of 16 bytes
        tc5::mma_f16_elect(tmem, a_desc, stage + 2 * k, b_desc, stage + 2 * k, idesc, kb > 0 || k > 0);
      tc5::commit_elect(&empty_bar[s]);            // the stage is free once these MMAs have read it
    }
    tc5::commit_elect(&done_bar);                  // the accumulator is complete
  } else {
    // Epilogue: warp w reads lanes 32 (w % 4) .. +31 of tensor memory; a lane is a row of the tile.
    ok = tma::mbar_wait(&done_bar, 0);
    tc5::fence_after_sync();
    const int lane_base = (warp & 3) * 32;
    const int m = m0 + lane_base + lane;
    const bool vec = (ldc * sizeof(TO)) % 16 == 0 && (n0 * sizeof(TO)) % 16 == 0 && ((uintptr_t)C & 15) == 0;
    if (ok) {
      if (EPI == 1) {
#pragma unroll 1
        for (int c = 0; c < OUT_COLS; c += 32) {
          float g[32], u[32];
          tc5::ld_32cols(tmem + ((uint32_t)lane_base << 16) + c, g);
          tc5::ld_32cols(tmem + ((uint32_t)lane_base << 16) + OUT_COLS + c, u);
          tc5::wait_ld();
          if (m < M && n0 + c < N) {
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * u[j];
            store_row32(C + (int64_t)m * ldc + n0 + c, g, N - n0 - c, vec);
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < OUT_COLS; c += 32) {
          float v[32];
          tc5::ld_32cols(tmem + ((uint32_t)lane_base << 16) + c, v);
          tc5::wait_ld();
          if (m < M && n0 + c < N) store_row32(C + (int64_t)m * ldc + n0 + c, v, N - n0 - c, vec);
        }
      }
    }
  }
  if (!ok) atomicOr(err + 1, 1);
  pdl_launch_dependents();
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tmem, BN < 32 ? 32 : BN);
}

template <int BN, int EPI, typename TO, bool DEEP>
int launch_tg(const void* map_a, const void* map_w, void* C, int64_t ldc, int M, int N, int K, int splits, int64_t split_stride,
              int* err, cudaStream_t stream) {
  constexpr int STAGES = tg_stages<BN>(DEEP);
  const size_t smem = (size_t)STAGES * (TG_A_BYTES + BN * TG_BK * 2) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI, TO, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_gemm_tcgen05: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
  const int num_kb = (K + TG_BK - 1) / TG_BK, kb_per_split = (num_kb + splits - 1) / splits;
  dim3 grid((N + OUT_COLS - 1) / OUT_COLS, (M + TG_BM - 1) / TG_BM, (num_kb + kb_per_split - 1) / kb_per_split);
  me_launch(gemm_tcgen05_kernel<BN, EPI, TO, DEEP>, grid, dim3(TG_THREADS), smem, stream, *reinterpret_cast<const CUtensorMap*>(map_a),
            *reinterpret_cast<const CUtensorMap*>(map_w), (TO*)C, ldc, M, N, K, kb_per_split, split_stride, err);
  return 0;
}

// ---- the persistent form: one block an SM walks tiles --------------------------------------------------------
// For products with many tiles (several an SM).  A block keeps its ring of stages and its tensor memory over all the
// tiles it computes (tile blockIdx.x, blockIdx.x + gridDim.x, ...; rows fastest, so that the blocks running at one
// time share few W tiles): the loads of the next tile are on their way while this tile's last products run, and with
// two accumulators the epilogue of a tile runs beside the products of the next.  The ring has the SM's whole shared
// memory (four stages of 128 x 64 and 256 x 64, or six with a 128-wide tile).
template <int BN> constexpr int tp_stages() { return BN <= 128 ? 6 : 4; }

template <int BN, int EPI, typename TO>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                               TO* __restrict__ C, int64_t ldc, int M, int N, int K, int* __restrict__ err) {
  constexpr int STAGES = tp_stages<BN>();
  constexpr int B_BYTES = BN * TG_BK * 2, STAGE_BYTES = TG_A_BYTES + B_BYTES;
  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
  constexpr uint32_t TMEM_COLS = 2 * BN;             // two accumulators
  extern __shared__ unsigned char tg_smem_raw[];
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  unsigned char* smem = tg_smem_raw + ((1024u - (tma::smem_addr(tg_smem_raw) & 1023u)) & 1023u);
  const int warp = tc5::uniform_warp_index(), lane = threadIdx.x & 31;
  const int m_tiles = (M + TG_BM - 1) / TG_BM, n_tiles = (N + OUT_COLS - 1) / OUT_COLS, num_kb = (K + TG_BK - 1) / TG_BK;
  const int tiles = m_tiles * n_tiles;
  const int my_tiles = blockIdx.x < tiles ? (tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const long long total = (long long)my_tiles * num_kb;      // stages of this block
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tma::mbar_init(&full_bar[s], 1);
      tma::mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tma::mbar_init(&acc_full[i], 1);
      tma::mbar_init(&acc_empty[i], 4);
    }
    tma::mbar_fence_init();
    tma::prefetch_map(&map_a);
    tma::prefetch_map(&map_w);
  }
  if (warp == 1) tc5::tmem_alloc(&tmem_slot, TMEM_COLS);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      auto place = [&](long long item, int& m0, int& n0, int& k0) {
        const int tile = blockIdx.x + (int)(item / num_kb) * gridDim.x;
        m0 = (tile % m_tiles) * TG_BM;
        n0 = (tile / m_tiles) * OUT_COLS;
        k0 = (int)(item % num_kb) * TG_BK;
      };
      auto issue_w = [&](long long item) {
        int m0, n0, k0;
        place(item, m0, n0, k0);
        const int s = (int)(item % STAGES);
        unsigned char* b_dst = smem + s * STAGE_BYTES + TG_A_BYTES;
        tma::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        if (EPI == 1) {
          tma::load_2d(b_dst, &map_w, k0, n0, &full_bar[s]);
          tma::load_2d(b_dst + B_BYTES / 2, &map_w, k0, N + n0, &full_bar[s]);
        } else {
          tma::load_2d(b_dst, &map_w, k0, n0, &full_bar[s]);
        }
      };
      auto issue_a = [&](long long item) {
        int m0, n0, k0;
        place(item, m0, n0, k0);
        const int s = (int)(item % STAGES);
        tma::load_2d(smem + s * STAGE_BYTES, &map_a, k0, m0, &full_bar[s]);
      };
      // The weights are no output of the kernel before this one; the activations are.
      const long long ahead = total < STAGES ? total : STAGES;
      for (long long item = 0; item < ahead; ++item) issue_w(item);
      pdl_wait();
      for (long long item = 0; item < ahead; ++item) issue_a(item);
      for (long long item = ahead; item < total && ok; ++item) {
        ok = tma::mbar_wait(&empty_bar[item % STAGES], (uint32_t)(((item / STAGES) & 1) ^ 1));
        if (!ok) break;
        issue_w(item);
        issue_a(item);
      }
    }
  } else if (warp == 1) {
    // all lanes run the loop, an elected one issues
    constexpr uint32_t idesc = tc5::instr_desc_bf16(TG_BM, BN);
    const tc5::DescWords a_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(smem));
    const tc5::DescWords b_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(smem + TG_A_BYTES));
    uint32_t s = 0, phase = 0;                       // the ring's stage and the parity of its round
    for (int i = 0; i < my_tiles; ++i) {
      const int buf = i & 1;
      if (i >= 2 && ok) ok = tc5::mbar_wait_warp(&acc_empty[buf], (uint32_t)(((i >> 1) - 1) & 1));      // read out by the epilogue
      tc5::fence_after_sync();
      for (int kb = 0; kb < num_kb; ++kb) {
        if (ok) ok = tc5::mbar_wait_warp(&full_bar[s], phase);
        tc5::fence_after_sync();
        if (ok) {
          const uint32_t stage = (s * (uint32_t)STAGE_BYTES) >> 4;
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k)       // 32 bytes further along K per step: +2 in units of 16 bytes
            tc5::mma_f16_elect(tmem + buf * BN, a_desc, stage + 2 * k, b_desc, stage + 2 * k, idesc, kb > 0 || k > 0);
        }
        tc5::commit_elect(&empty_bar[s]);            // the stage is free once these MMAs have read it
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
      tc5::commit_elect(&acc_full[buf]);             // the tile's sums are complete
    }
  } else {
    // Epilogue: warp w reads lanes 32 (w % 4) .. +31 of tensor memory; a lane is a row of the tile.
    const int lane_base = (warp & 3) * 32;
    for (int i = 0; i < my_tiles; ++i) {
      const int tile = blockIdx.x + i * gridDim.x, buf = i & 1;
      const int m0 = (tile % m_tiles) * TG_BM, n0 = (tile / m_tiles) * OUT_COLS;
      const int m = m0 + lane_base + lane;
      if (ok) ok = tma::mbar_wait(&acc_full[buf], (uint32_t)((i >> 1) & 1));
      tc5::fence_after_sync();
      const uint32_t acc = tmem + ((uint32_t)lane_base << 16) + buf * BN;
      const bool vec = (ldc * sizeof(TO)) % 16 == 0 && (n0 * sizeof(TO)) % 16 == 0 && ((uintptr_t)C & 15) == 0;
      if (ok) {
        if (EPI == 1) {
#pragma unroll 1
          for (int c = 0; c < OUT_COLS; c += 32) {
            float g[32], u[32];
            tc5::ld_32cols(acc + c, g);
            tc5::ld_32cols(acc + OUT_COLS + c, u);
            tc5::wait_ld();
            if (m < M && n0 + c < N) {
#pragma unroll
              for (int j = 0; j < 32; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * u[j];
              store_row32(C + (int64_t)m * ldc + n0 + c, g, N - n0 - c, vec);
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < OUT_COLS; c += 32) {
            float v[32];
            tc5::ld_32cols(acc + c, v);
            tc5::wait_ld();
            if (m < M && n0 + c < N) store_row32(C + (int64_t)m * ldc + n0 + c, v, N - n0 - c, vec);
          }
        }
      }
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tma::smem_addr(&acc_empty[buf])) : "memory");
    }
  }
  if (!ok) atomicOr(err + 1, 1);
  pdl_launch_dependents();
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tmem, TMEM_COLS);
}

template <int BN, int EPI, typename TO>
int launch_tp(const void* map_a, const void* map_w, void* C, int64_t ldc, int M, int N, int K, int* err, cudaStream_t stream) {
  const size_t smem = (size_t)tp_stages<BN>() * (TG_A_BYTES + BN * TG_BK * 2) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<BN, EPI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_gemm_tcgen05: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
  const long long tiles = (long long)((N + OUT_COLS - 1) / OUT_COLS) * ((M + TG_BM - 1) / TG_BM);
  ME_REQUIRE(tiles < (1ll << 30), "me_gemm_tcgen05: too many tiles");
  const int blocks = (int)(tiles < me_sm_count() ? tiles : me_sm_count());
  me_launch(gemm_tcgen05_persistent_kernel<BN, EPI, TO>, dim3(blocks), dim3(TG_THREADS), smem, stream,
            *reinterpret_cast<const CUtensorMap*>(map_a), *reinterpret_cast<const CUtensorMap*>(map_w), (TO*)C, ldc, M, N, K, err);
  return 0;
}

}  // namespace

// How many partial results a product over K asked to be split ``splits`` ways writes (whole blocks of 64 along K each).
ME_API int me_gemm_tcgen05_splits(int K, int splits) {
  if (splits < 1) return 0;
  const int num_kb = (K + TG_BK - 1) / TG_BK, per = (num_kb + splits - 1) / splits;
  return (num_kb + per - 1) / per;
}

// Rows of W that one block's TMA box covers for a given tile width and epilogue (the caller encodes the map so).
ME_API int me_gemm_tcgen05_w_box_rows(int bn, int epi) { return epi == 1 ? bn / 2 : bn; }

// The persistent form of me_gemm_tcgen05 (same operands, no split along K): bn 128 or 256.
ME_API int me_gemm_tcgen05_persistent(const void* map_a, const void* map_w, void* C, int c_dtype, int64_t ldc, int M, int N,
                                      int K, int epi, int bn, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0, "me_gemm_tcgen05_persistent: bad sizes M=%d N=%d K=%d (K must be a multiple of 8)", M, N, K);
  ME_REQUIRE(map_a != nullptr && map_w != nullptr && err != nullptr, "me_gemm_tcgen05_persistent: tensor maps and the error word are required");
  ME_REQUIRE(epi == 0 || (epi == 1 && c_dtype == ME_BF16), "me_gemm_tcgen05_persistent: epilogue %d", epi);
  ME_REQUIRE(bn == 128 || bn == 256, "me_gemm_tcgen05_persistent: tile width %d is not 128 or 256", bn);
  int rc = 1;
#define ME_TP_CASE(BN_)                                                                                  \
  if (bn == BN_) {                                                                                       \
    if (epi == 1) rc = launch_tp<BN_, 1, bf16>(map_a, map_w, C, ldc, M, N, K, err, stream);              \
    else if (c_dtype == ME_BF16) rc = launch_tp<BN_, 0, bf16>(map_a, map_w, C, ldc, M, N, K, err, stream); \
    else rc = launch_tp<BN_, 0, float>(map_a, map_w, C, ldc, M, N, K, err, stream);                      \
  }
  ME_TP_CASE(128) ME_TP_CASE(256)
#undef ME_TP_CASE
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_gemm_tcgen05_persistent");
  return 0;
}

// map_a: X as [M][K], boxes 128 x 64, 128-byte swizzle; map_w: W as [rows][K], boxes
// me_gemm_tcgen05_w_box_rows(bn, epi) x 64.  N counts output columns (epi 1: W has 2N rows).
// bn is the accumulator's width: 64, 128 or 256.  ``splits`` > 1: the K range is shared out over that many blocks a tile, whose
// float32 partial results lie ``split_stride`` elements apart (me_gemm_tcgen05_splits says how many there will be).
ME_API int me_gemm_tcgen05(const void* map_a, const void* map_w, void* C, int c_dtype, int64_t ldc, int M, int N,
                           int K, int epi, int bn, int splits, int64_t split_stride, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0, "me_gemm_tcgen05: bad sizes M=%d N=%d K=%d (K must be a multiple of 8)", M, N, K);
  ME_REQUIRE(map_a != nullptr && map_w != nullptr && err != nullptr, "me_gemm_tcgen05: tensor maps and the error word are required");
  ME_REQUIRE(epi == 0 || (epi == 1 && c_dtype == ME_BF16), "me_gemm_tcgen05: epilogue %d", epi);
  ME_REQUIRE((M + TG_BM - 1) / TG_BM <= 65535, "me_gemm_tcgen05: M=%d is too large", M);
  ME_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || (epi == 0 && c_dtype == ME_F32)),
             "me_gemm_tcgen05: %d splits (they need float32 results and no epilogue)", splits);
  ME_REQUIRE(bn == 64 || bn == 128 || bn == 256, "me_gemm_tcgen05: tile width %d is not 64, 128 or 256", bn);
  const int out_cols = epi == 1 ? bn / 2 : bn;
  const bool deep = (int64_t)((N + out_cols - 1) / out_cols) * ((M + TG_BM - 1) / TG_BM) * me_gemm_tcgen05_splits(K, splits) <= me_sm_count();
  int rc = 1;
#define ME_TG_CASE(BN_)                                                                                              \
  if (bn == BN_) {                                                                                                   \
    if (epi == 1) rc = launch_tg<BN_, 1, bf16, false>(map_a, map_w, C, ldc, M, N, K, 1, 0, err, stream);             \
    else if (c_dtype == ME_BF16) rc = deep ? launch_tg<BN_, 0, bf16, true>(map_a, map_w, C, ldc, M, N, K, 1, 0, err, stream)   \
                                           : launch_tg<BN_, 0, bf16, false>(map_a, map_w, C, ldc, M, N, K, 1, 0, err, stream); \
    else rc = deep ? launch_tg<BN_, 0, float, true>(map_a, map_w, C, ldc, M, N, K, splits, split_stride, err, stream)          \
                   : launch_tg<BN_, 0, float, false>(map_a, map_w, C, ldc, M, N, K, splits, split_stride, err, stream);        \
  }
  ME_TG_CASE(64) ME_TG_CASE(128) ME_TG_CASE(256)
#undef ME_TG_CASE
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_gemm_tcgen05");
  return 0;
}
