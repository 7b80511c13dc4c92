// C[M,N] = A[M,K] W[N,K]^T in bfloat16 on the 5th-generation tensor cores (tcgen05), for many rows
// (portions of prompts).  The reference leaves these products to cuBLAS through F.linear
// (layers/linear.py:26,45); this kernel is the engine's own, with SiLU-and-multiply
// (layers/activation.py:4-7) in its epilogue and float32 results for the output head.
//
// One block computes a 128 x BN tile.  Warp 0: one thread streams A and W tiles of 64 K-elements
// through a ring of shared-memory stages by TMA (128-byte swizzle, zero fill at the edges).
// Warp 1: allocates BN columns of tensor memory; all its lanes run the loop and an elected lane issues
// tcgen05.mma (M 128, N BN, K 16, four per stage) and hands stages back through tcgen05.commit.
// Warps 2..5: when the accumulator is complete, each thread reads its row from tensor memory
// (tcgen05.ld) and applies the epilogue; the rows leave through shared memory in whole lines
// (write_rows).  Every wait is bounded; a wait that gives up sets flag 1 of ``err`` and the block still
// frees its tensor memory and exits.
//
// Three forms: a tile a block (gemm_tcgen05_kernel, with K shared out over gridDim.z blocks where the
// caller adds float32 partial results), blocks that walk whole tiles (gemm_tcgen05_persistent_kernel), and
// blocks that share the last rounds' stages out evenly (gemm_tcgen05_shared_kernel).
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

// 32 consecutive results of one row, one by one (rows of C that are not 16-byte aligned).
__device__ __forceinline__ void store_row32(bf16* dst, const float (&v)[32], int n_left) {
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j < n_left) dst[j] = __float2bfloat16_rn(v[j]);
}
__device__ __forceinline__ void store_row32(float* dst, const float (&v)[32], int n_left) {
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j < n_left) dst[j] = v[j];
}

// The epilogue of one warp: its 32 rows of a tile (a lane a row) go out OUT_COLS columns wide.  ``load(col, v)`` asks for 32
// accumulator columns of the lane's row from ``col`` on (tcgen05.ld, not waited for), ``fix(col, v)`` is applied to them once
// they are there (the work-sharing form adds the other blocks' sums).  A thread holds a row, so stores straight from the
// registers would touch 32 different lines each (270 clocks a store instruction, 9,800 a 128 x 256 tile: as long as the
// tile's products at K = 1,024); the results go through ``stage`` (4 KB of shared memory of the warp's own, 128-byte
// aligned) in groups of 128 bytes a row, swizzled by 16-byte pieces, and leave with whole lines: a store instruction
// writes four rows' 128 bytes.  Without 16-byte alignment of the rows of C (``vec`` false) they leave one by one.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

template <int EPI, typename TO, int OUT_COLS, typename Load, typename Fix>
__device__ __forceinline__ void write_rows(Load&& load, Fix&& fix, unsigned char* stage, TO* __restrict__ C, int64_t ldc, int M, int N,
                                           int m0, int n0, int lane_base, int lane, bool vec) {
  const int m = m0 + lane_base + lane;
  // 32 results of the lane's row from output column ``c`` on
  auto results = [&](int c, float (&g)[32]) {
    if (EPI == 1) {
      float u[32];
      load(c, g);
      load(OUT_COLS + c, u);
      tc5::wait_ld();
      fix(c, g);
      fix(OUT_COLS + c, u);
#pragma unroll
      for (int j = 0; j < 32; ++j) g[j] = silu_mul(g[j], u[j]);
    } else {
      load(c, g);
      tc5::wait_ld();
      fix(c, g);
    }
  };
  if (!vec) {
#pragma unroll 1
    for (int c = 0; c < OUT_COLS; c += 32) {
      float g[32];
      results(c, g);
      if (m < M && n0 + c < N) store_row32(C + (int64_t)m * ldc + n0 + c, g, N - n0 - c);
    }
    return;
  }
  constexpr int GROUP = 128 / (int)sizeof(TO), PER = 16 / (int)sizeof(TO);       // columns a 128-byte group, a 16-byte piece
  const int rows_left = M - (m0 + lane_base);
#pragma unroll 1
  for (int c = 0; c < OUT_COLS; c += GROUP) {
    uint4 pk[8];
#pragma unroll
    for (int h = 0; h < GROUP / 32; ++h) {
      if (c + 32 * h < OUT_COLS) {                           // (a tile of 32 output columns is half a group of bfloat16)
        float g[32];
        results(c + 32 * h, g);
        if (sizeof(TO) == 2) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk[h * 4 + q]);
#pragma unroll
            for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(g[q * 8 + 2 * j], g[q * 8 + 2 * j + 1]);
          }
        } else {
#pragma unroll
          for (int q = 0; q < 8; ++q) pk[q] = make_uint4(__float_as_uint(g[q * 4]), __float_as_uint(g[q * 4 + 1]), __float_as_uint(g[q * 4 + 2]),
                                                         __float_as_uint(g[q * 4 + 3]));
        }
      }
    }
    const int cols_left = min(N - n0, OUT_COLS) - c;         // columns of this group that are the tile's and the product's
    if (rows_left > 0 && cols_left > 0) {                    // (the same in all lanes)
#pragma unroll
      for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(stage + lane * 128 + ((q ^ (lane & 7)) << 4)) = pk[q];
      __syncwarp();
      const int piece = lane & 7;
      TO* dst0 = C + (int64_t)(m0 + lane_base) * ldc + n0 + c + piece * PER;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = i * 4 + (lane >> 3);
        if (row < rows_left && piece * PER < cols_left) {
          const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 128 + ((piece ^ (row & 7)) << 4));
          TO* dst = dst0 + (int64_t)row * ldc;
          if (piece * PER + PER <= cols_left) {
            *reinterpret_cast<uint4*>(dst) = v;
          } else {
            const TO* e = reinterpret_cast<const TO*>(&v);
#pragma unroll
            for (int j = 0; j < PER; ++j)
              if (j < cols_left - piece * PER) dst[j] = e[j];
          }
        }
      }
      __syncwarp();
    }
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
    const bool vec = (ldc * sizeof(TO)) % 16 == 0 && (n0 * sizeof(TO)) % 16 == 0 && ((uintptr_t)C & 15) == 0;
    if (ok) {
      // every product is over and every load has been read: the ring's first 16 KB are the four warps' staging rows
      auto load = [&](int col, float (&v)[32]) { tc5::ld_32cols(tmem + ((uint32_t)lane_base << 16) + col, v); };
      auto fix = [](int, float (&)[32]) {};
      write_rows<EPI, TO, OUT_COLS>(load, fix, smem + (warp & 3) * 4096, C, ldc, M, N, m0, n0, lane_base, lane, vec);
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
      // A place in this block's sequence of stages, moved on without a division (one thread feeds the whole SM).
      struct Walk { int tile, kb, m0, n0, s; uint32_t phase; };
      auto start = [&](Walk& w) {
        w.tile = blockIdx.x;
        w.kb = 0;
        w.m0 = (w.tile % m_tiles) * TG_BM;
        w.n0 = (w.tile / m_tiles) * OUT_COLS;
        w.s = 0;
        w.phase = 0;
      };
      auto step = [&](Walk& w) {
        if (++w.kb == num_kb) {
          w.kb = 0;
          w.tile += gridDim.x;
          w.m0 = (w.tile % m_tiles) * TG_BM;
          w.n0 = (w.tile / m_tiles) * OUT_COLS;
        }
        if (++w.s == STAGES) {
          w.s = 0;
          w.phase ^= 1;
        }
      };
      auto issue_w = [&](const Walk& w) {
        unsigned char* b_dst = smem + w.s * STAGE_BYTES + TG_A_BYTES;
        tma::mbar_expect_tx(&full_bar[w.s], STAGE_BYTES);
        if (EPI == 1) {
          tma::load_2d(b_dst, &map_w, w.kb * TG_BK, w.n0, &full_bar[w.s]);
          tma::load_2d(b_dst + B_BYTES / 2, &map_w, w.kb * TG_BK, N + w.n0, &full_bar[w.s]);
        } else {
          tma::load_2d(b_dst, &map_w, w.kb * TG_BK, w.n0, &full_bar[w.s]);
        }
      };
      auto issue_a = [&](const Walk& w) { tma::load_2d(smem + w.s * STAGE_BYTES, &map_a, w.kb * TG_BK, w.m0, &full_bar[w.s]); };
      // The weights are no output of the kernel before this one; the activations are.
      const long long ahead = total < STAGES ? total : STAGES;
      Walk ww, wa;
      start(ww);
      start(wa);
      for (long long item = 0; item < ahead; ++item, step(ww)) issue_w(ww);
      pdl_wait();
      for (long long item = 0; item < ahead; ++item, step(wa)) issue_a(wa);
      for (long long item = ahead; item < total && ok; ++item, step(ww)) {
        ok = tma::mbar_wait(&empty_bar[ww.s], ww.phase ^ 1);      // the products of the round before have read the stage
        if (!ok) break;
        issue_w(ww);
        issue_a(ww);
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
      if (ok) ok = tma::mbar_wait(&acc_full[buf], (uint32_t)((i >> 1) & 1));
      tc5::fence_after_sync();
      const uint32_t acc = tmem + ((uint32_t)lane_base << 16) + buf * BN;
      const bool vec = (ldc * sizeof(TO)) % 16 == 0 && (n0 * sizeof(TO)) % 16 == 0 && ((uintptr_t)C & 15) == 0;
      if (ok) {
        auto load = [&](int col, float (&v)[32]) { tc5::ld_32cols(acc + col, v); };
        auto fix = [](int, float (&)[32]) {};
        write_rows<EPI, TO, OUT_COLS>(load, fix, smem + STAGES * STAGE_BYTES + (warp & 3) * 4096, C, ldc, M, N, m0, n0, lane_base, lane, vec);
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

// ---- work shared out evenly ---------------------------------------------------------------------------------
// The persistent form gives a block whole tiles: with 1.3 or 2.2 tiles an SM most SMs idle through the last round.  Here
// a block takes whole tiles in that same order (tile blockIdx.x, + gridDim.x, ...) for all rounds but the last one or
// two; the stages of the tiles that remain (at least one tile a block where there are that many, fewer than two; 64 of K
// a stage, tile after tile) are one sequence, cut into gridDim.x ranges of the same length: there a block computes the
// end of one tile and the beginning of the next.  (All tiles in one such sequence was tried first: the blocks then work on
// 148 different tiles of W at a time, which L2 does not hold, and the products ran a third slower.)  The block with a
// tile's beginning owns the tile: it adds what the blocks after it computed of it, in the order of the blocks (float32
// sums through ``partials``, a flag for each of a block's four epilogue warps once they are written), and applies the
// epilogue.  A contributing block's part is the FIRST thing it computes in the shared rounds and the owner wants it at the
// END of its own range, so no block waits long, and none waits for a block that waits for it; the waits are bounded.
// The owner's epilogue warps bring a contributor's sums into the (by then idle) ring of stages with one bulk copy a warp and
// add them from shared memory: read by plain loads, 32 columns at a time, they took 10 us and more of a product of 30.
// partials: gridDim.x x 4 x BN / 32 x 8 x 32 float4 (block, epilogue warp, 32 columns, four of them, row); flags: 4 ints a
// block, zero between launches.
template <int BN, int EPI, typename TO>
__global__ void __launch_bounds__(TG_THREADS, 1)
gemm_tcgen05_shared_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                           TO* __restrict__ C, int64_t ldc, int M, int N, int K, float* __restrict__ partials,
                           int* __restrict__ flags, int* __restrict__ err) {
  constexpr int STAGES = tp_stages<BN>();
  constexpr int B_BYTES = BN * TG_BK * 2, STAGE_BYTES = TG_A_BYTES + B_BYTES;
  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
  constexpr uint32_t TMEM_COLS = 2 * BN;             // two accumulators
  constexpr int CHUNKS = BN / 32, WARP_VECS = CHUNKS * 8 * 32;      // what an epilogue warp leaves: 32 rows x BN columns as float4
  extern __shared__ unsigned char tg_smem_raw[];
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2], fix_bar[4];
  __shared__ uint32_t tmem_slot;
  unsigned char* smem = tg_smem_raw + ((1024u - (tma::smem_addr(tg_smem_raw) & 1023u)) & 1023u);
  const int warp = tc5::uniform_warp_index(), lane = threadIdx.x & 31;
  const int m_tiles = (M + TG_BM - 1) / TG_BM, n_tiles = (N + OUT_COLS - 1) / OUT_COLS, num_kb = (K + TG_BK - 1) / TG_BK;
  const int tiles = m_tiles * n_tiles, G = (int)gridDim.x;
  const int whole_rounds = tiles / G > 1 ? tiles / G - 1 : 0;                  // rounds in which a block takes a whole tile
  const int first_shared = whole_rounds * G;                                   // the tiles from here on are shared out
  const long long shared_total = (long long)(tiles - first_shared) * num_kb;   // their stages
  auto begin_of = [&](int block) { return shared_total * block / (long long)G; };
  const long long s0 = begin_of(blockIdx.x), s1 = begin_of(blockIdx.x + 1);
  const long long whole_items = (long long)whole_rounds * num_kb, my_items = whole_items + (s1 - s0);
  // the part of a tile that starts at this block's stage ``idx``: K blocks kb0 .. kb1 - 1 of ``tile``
  auto segment = [&](long long idx, int& tile, int& kb0, int& kb1) {
    if (idx < whole_items) {
      const int round = (int)(idx / num_kb);
      tile = round * G + (int)blockIdx.x;
      kb0 = (int)(idx - (long long)round * num_kb);
      kb1 = num_kb;
    } else {
      const long long at = s0 + (idx - whole_items);
      const int t = (int)(at / num_kb);
      tile = first_shared + t;
      kb0 = (int)(at - (long long)t * num_kb);
      kb1 = (int)(s1 - at < (long long)(num_kb - kb0) ? kb0 + (s1 - at) : num_kb);
    }
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tma::mbar_init(&full_bar[s], 1);
      tma::mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tma::mbar_init(&acc_full[i], 1);
      tma::mbar_init(&acc_empty[i], 4);
    }
    for (int i = 0; i < 4; ++i) tma::mbar_init(&fix_bar[i], 1);
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
      // A place in this block's sequence of stages, moved on without a division inside a segment (one thread feeds the SM).
      struct Walk { long long idx; int kb, kb1, m0, n0, s; uint32_t phase; };
      auto enter = [&](Walk& w) {                      // the segment that starts at w.idx
        int tile;
        segment(w.idx, tile, w.kb, w.kb1);
        w.m0 = (tile % m_tiles) * TG_BM;
        w.n0 = (tile / m_tiles) * OUT_COLS;
      };
      auto start = [&](Walk& w) {
        w.idx = 0;
        w.s = 0;
        w.phase = 0;
        if (my_items > 0) enter(w);
      };
      auto step = [&](Walk& w) {
        ++w.idx;
        if (++w.kb == w.kb1 && w.idx < my_items) enter(w);
        if (++w.s == STAGES) {
          w.s = 0;
          w.phase ^= 1;
        }
      };
      auto issue_w = [&](const Walk& w) {
        unsigned char* b_dst = smem + w.s * STAGE_BYTES + TG_A_BYTES;
        tma::mbar_expect_tx(&full_bar[w.s], STAGE_BYTES);
        if (EPI == 1) {
          tma::load_2d(b_dst, &map_w, w.kb * TG_BK, w.n0, &full_bar[w.s]);
          tma::load_2d(b_dst + B_BYTES / 2, &map_w, w.kb * TG_BK, N + w.n0, &full_bar[w.s]);
        } else {
          tma::load_2d(b_dst, &map_w, w.kb * TG_BK, w.n0, &full_bar[w.s]);
        }
      };
      auto issue_a = [&](const Walk& w) { tma::load_2d(smem + w.s * STAGE_BYTES, &map_a, w.kb * TG_BK, w.m0, &full_bar[w.s]); };
      // The weights are no output of the kernel before this one; the activations are.
      const long long ahead = my_items < STAGES ? my_items : STAGES;
      Walk ww, wa;
      start(ww);
      start(wa);
      for (long long i = 0; i < ahead; ++i, step(ww)) issue_w(ww);
      pdl_wait();
      for (long long i = 0; i < ahead; ++i, step(wa)) issue_a(wa);
      for (long long i = ahead; i < my_items && ok; ++i, step(ww)) {
        ok = tma::mbar_wait(&empty_bar[ww.s], ww.phase ^ 1);      // the products of the round before have read the stage
        if (!ok) break;
        issue_w(ww);
        issue_a(ww);
      }
    }
  } else if (warp == 1) {
    // all lanes run the loop, an elected one issues
    constexpr uint32_t idesc = tc5::instr_desc_bf16(TG_BM, BN);
    const tc5::DescWords a_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(smem));
    const tc5::DescWords b_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(smem + TG_A_BYTES));
    uint32_t s = 0, phase = 0;                       // the ring's stage and the parity of its round
    int seg = 0;
    for (long long idx = 0; idx < my_items; ++seg) {
      int tile, kb0, kb1;
      segment(idx, tile, kb0, kb1);
      const int buf = seg & 1;
      if (seg >= 2 && ok) ok = tc5::mbar_wait_warp(&acc_empty[buf], (uint32_t)(((seg >> 1) - 1) & 1));      // read out by the epilogue
      tc5::fence_after_sync();
      for (int kb = kb0; kb < kb1; ++kb) {
        if (ok) ok = tc5::mbar_wait_warp(&full_bar[s], phase);
        tc5::fence_after_sync();
        if (ok) {
          const uint32_t stage = (s * (uint32_t)STAGE_BYTES) >> 4;
#pragma unroll
          for (int k = 0; k < TG_BK / 16; ++k)       // 32 bytes further along K per step: +2 in units of 16 bytes
            tc5::mma_f16_elect(tmem + buf * BN, a_desc, stage + 2 * k, b_desc, stage + 2 * k, idesc, kb > kb0 || k > 0);
        }
        tc5::commit_elect(&empty_bar[s]);            // the stage is free once these MMAs have read it
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
      tc5::commit_elect(&acc_full[buf]);             // the segment's sums are complete
      idx += kb1 - kb0;
    }
  } else {
    // Epilogue: warp w reads lanes 32 (w % 4) .. +31 of tensor memory; a lane is a row of the tile.
    const int quad = warp & 3, lane_base = quad * 32;
    int seg = 0;
    for (long long idx = 0; idx < my_items; ++seg) {
      int tile, kb0, kb1;
      segment(idx, tile, kb0, kb1);
      idx += kb1 - kb0;
      const int buf = seg & 1;
      const int m0 = (tile % m_tiles) * TG_BM, n0 = (tile / m_tiles) * OUT_COLS;
      if (ok) ok = tma::mbar_wait(&acc_full[buf], (uint32_t)((seg >> 1) & 1));
      tc5::fence_after_sync();
      const uint32_t acc = tmem + ((uint32_t)lane_base << 16) + buf * BN;
      if (kb0 > 0) {
        // the tile's beginning is another block's: leave the sums for it
        if (ok) {
          float4* dst = reinterpret_cast<float4*>(partials) + ((size_t)blockIdx.x * 4 + quad) * WARP_VECS + lane;
#pragma unroll 1
          for (int c = 0; c < CHUNKS; ++c) {
            float v[32];
            tc5::ld_32cols(acc + c * 32, v);
            tc5::wait_ld();
#pragma unroll
            for (int q = 0; q < 8; ++q) dst[(c * 8 + q) * 32] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          }
          __threadfence();
          __syncwarp();
          if (lane == 0) asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(flags + blockIdx.x * 4 + quad), "r"(1) : "memory");
        }
      } else {
        // the blocks after this one that hold the rest of the tile (none if it ends here)
        int c_end = blockIdx.x + 1;
        if (kb1 < num_kb)
          while (c_end < G && begin_of(c_end) < (long long)(tile - first_shared + 1) * num_kb) ++c_end;
        // This is the block's last segment and its products are over: the ring of stages is idle, and this warp's quarter
        // of its first 128 KB is where the contributors' sums of the warp's 32 rows land, one contributor at a time.
        const float4* land = reinterpret_cast<const float4*>(smem + quad * (WARP_VECS * 16)) + lane;
        int landed = 0;                                      // copies this warp has waited for
        auto bring = [&](int cc) {                           // wait for block cc's sums, copy them in, wait for the copy
          const int* f = flags + cc * 4 + quad;
          bool there = false;
          for (unsigned i = 0; i < (1u << 21) && !there; ++i) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(f) : "memory");
            there = v != 0;
            if (!there) __nanosleep(64);
          }
          ok = __all_sync(0xffffffffu, there);
          if (!ok) return;
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // (this warp's loads of the copy before are over)
          __syncwarp();
          if (lane == 0) {
            tma::mbar_expect_tx(&fix_bar[quad], WARP_VECS * 16);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                         ::"r"(tma::smem_addr(smem + quad * (WARP_VECS * 16))),
                           "l"(reinterpret_cast<const float4*>(partials) + ((size_t)cc * 4 + quad) * WARP_VECS), "r"(WARP_VECS * 16),
                           "r"(tma::smem_addr(&fix_bar[quad])) : "memory");
          }
          ok = __all_sync(0xffffffffu, tma::mbar_wait(&fix_bar[quad], landed & 1));
          ++landed;
        };
        auto add_landed = [&](int chunk, float (&v)[32]) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 t = land[(chunk * 8 + q) * 32];
            v[q * 4] += t.x;
            v[q * 4 + 1] += t.y;
            v[q * 4 + 2] += t.z;
            v[q * 4 + 3] += t.w;
          }
        };
        // all contributors but the last are added into tensor memory, in their order; the last one on the way out
        for (int cc = blockIdx.x + 1; cc + 1 < c_end && ok; ++cc) {
          bring(cc);
          if (!ok) break;
#pragma unroll 1
          for (int c = 0; c < CHUNKS; ++c) {
            float v[32];
            tc5::ld_32cols(acc + c * 32, v);
            tc5::wait_ld();
            add_landed(c, v);
            tc5::st_32cols(acc + c * 32, v);
          }
          tc5::wait_st();
        }
        const bool last = c_end > (int)blockIdx.x + 1;
        if (last && ok) bring(c_end - 1);
        auto load = [&](int col, float (&v)[32]) { tc5::ld_32cols(acc + col, v); };
        auto fix = [&](int col, float (&v)[32]) {
          if (last) add_landed(col / 32, v);
        };
        const bool vec = (ldc * sizeof(TO)) % 16 == 0 && (n0 * sizeof(TO)) % 16 == 0 && ((uintptr_t)C & 15) == 0;
        if (ok) {
          // (the staging rows lie behind the ring: the last contributor's sums are still being read from the ring itself)
          write_rows<EPI, TO, OUT_COLS>(load, fix, smem + STAGES * STAGE_BYTES + quad * 4096, C, ldc, M, N, m0, n0, lane_base, lane, vec);
          __syncwarp();
          if (lane == 0)
            for (int cc = blockIdx.x + 1; cc < c_end; ++cc) flags[cc * 4 + quad] = 0;      // zero again for the next launch
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
int launch_ts(const void* map_a, const void* map_w, void* C, int64_t ldc, int M, int N, int K, float* partials, int* flags, int* err,
              cudaStream_t stream) {
  const size_t smem = (size_t)tp_stages<BN>() * (TG_A_BYTES + BN * TG_BK * 2) + 4 * 4096 + 1024;      // the ring, the epilogue warps' staging rows
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_shared_kernel<BN, EPI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_gemm_tcgen05: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
  const long long tiles = (long long)((N + OUT_COLS - 1) / OUT_COLS) * ((M + TG_BM - 1) / TG_BM);
  ME_REQUIRE(tiles < (1ll << 30), "me_gemm_tcgen05: too many tiles");
  const long long total = tiles * ((K + TG_BK - 1) / TG_BK);
  const int blocks = (int)(total < me_sm_count() ? total : me_sm_count());
  me_launch(gemm_tcgen05_shared_kernel<BN, EPI, TO>, dim3(blocks), dim3(TG_THREADS), smem, stream,
            *reinterpret_cast<const CUtensorMap*>(map_a), *reinterpret_cast<const CUtensorMap*>(map_w), (TO*)C, ldc, M, N, K, partials,
            flags, err);
  return 0;
}

template <int BN, int EPI, typename TO>
int launch_tp(const void* map_a, const void* map_w, void* C, int64_t ldc, int M, int N, int K, int* err, cudaStream_t stream) {
  const size_t smem = (size_t)tp_stages<BN>() * (TG_A_BYTES + BN * TG_BK * 2) + 4 * 4096 + 1024;      // the ring, the epilogue warps' staging rows
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

// The form that shares the work out evenly over the SMs (same operands as the persistent form): ``partials`` has room for
// me_gemm_tcgen05_shared_partial_floats() floats, ``flags`` for me_gemm_tcgen05_shared_flag_ints() ints that are zero
// between launches (the kernel leaves them so unless a bounded wait runs out).  Launches that share them must not overlap.
ME_API int me_gemm_tcgen05_shared_partial_floats() { return me_sm_count() * 256 * 128; }
ME_API int me_gemm_tcgen05_shared_flag_ints() { return 4 * me_sm_count(); }
ME_API int me_gemm_tcgen05_shared(const void* map_a, const void* map_w, void* C, int c_dtype, int64_t ldc, int M, int N,
                                  int K, int epi, int bn, float* partials, int* flags, int* err, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  ME_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0, "me_gemm_tcgen05_shared: bad sizes M=%d N=%d K=%d (K must be a multiple of 8)", M, N, K);
  ME_REQUIRE(map_a != nullptr && map_w != nullptr && err != nullptr && partials != nullptr && flags != nullptr,
             "me_gemm_tcgen05_shared: tensor maps, work buffers and the error word are required");
  ME_REQUIRE(epi == 0 || (epi == 1 && c_dtype == ME_BF16), "me_gemm_tcgen05_shared: epilogue %d", epi);
  ME_REQUIRE(bn == 128 || bn == 256, "me_gemm_tcgen05_shared: tile width %d is not 128 or 256", bn);
  int rc = 1;
#define ME_TS_CASE(BN_)                                                                                                    \
  if (bn == BN_) {                                                                                                         \
    if (epi == 1) rc = launch_ts<BN_, 1, bf16>(map_a, map_w, C, ldc, M, N, K, partials, flags, err, stream);              \
    else if (c_dtype == ME_BF16) rc = launch_ts<BN_, 0, bf16>(map_a, map_w, C, ldc, M, N, K, partials, flags, err, stream); \
    else rc = launch_ts<BN_, 0, float>(map_a, map_w, C, ldc, M, N, K, partials, flags, err, stream);                      \
  }
  ME_TS_CASE(128) ME_TS_CASE(256)
#undef ME_TS_CASE
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_gemm_tcgen05_shared");
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
