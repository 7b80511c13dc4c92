// Paged attention for portions of prompts on tcgen05 / tensor memory (bfloat16, head_dim 64 or 128,
// page sizes that divide 128).
//
// Semantics as in csrc/attention_prefill_mma.cu and the reference's csrc/paged_prefill.cu:177-247:
// a tile of queries against tiles of cached keys found through the block table, online softmax in
// float32, P rounded to bfloat16 before P V, O / l at the end; optional window.
//
// One block = 128 rows = (128 / GP query tokens) x (GP heads of one key/value head), row r being head
// r / TQ, token r % TQ.  Key tiles of 128 keys at absolute multiples of 128.
//   warps 0 and 10: TMA.  Q once (a box per head and 64-column half), then per key tile the pages of K (warp 0)
//     and of V (warp 10), a box per page and half with the 128-byte swizzle, each into a ring of two buffers of
//     its own: a K buffer is handed back when Q K^T has read it, a V buffer when P V has, so the next K is on
//     its way a tile's time before the next V.
//   warp 1, one thread: tcgen05.mma.  S[128x128] = Q K^T into one of two S buffers in tensor memory
//     (K-major operands), one tile ahead of the softmax; after the softmax warps have written P:
//     O_tile[128 x head_dim] = P V, with V as an MN-major operand.
//   warps 2..9 (256 threads, two per row, each with half of the columns): read S from tensor memory, mask,
//     maximum and sum, write P (bfloat16) into one of two buffers in shared memory in the swizzled K-major
//     layout.  O stays in tensor memory, where P V accumulates over the key tiles; a row's reference
//     maximum is only raised when the new maximum exceeds it by more than 2^8 (the values of P stay below
//     256 meanwhile), and then the row of O is rescaled in tensor memory.  So the softmax of a tile does not
//     wait for the P V of the tile before; at the end O is read once and divided by the row's sum.
// Blocks take the query tiles from the last to the first, the ones with most keys first.
// That is the kernel for key tiles of 64; for key tiles of 128 a second kernel further down keeps the roles and the
// tiles but splits the softmax warps into two groups that take the key tiles in turn, and keeps P in tensor memory.
// All waits are bounded; a wait that gives up sets flag 1 of ``err`` and the block frees its tensor
// memory and exits.
#include "tcgen05.cuh"

namespace {

constexpr int TA_ROWS = 128, TA_THREADS = 352;      // warp 0: K loads, 1: MMA, 2..9: softmax, 10: V loads

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tma::smem_addr(bar)) : "memory");
}

template <int HD, int TA_KEYS>
__global__ void __launch_bounds__(TA_THREADS)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                            bf16* __restrict__ out, int64_t out_row_stride, const int* __restrict__ block_tables,
                            int bt_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                            const int* __restrict__ tiles, int nh, int nkv, int gp, int page_size, float scale_log2,
                            int window, int* __restrict__ err) {
  constexpr int HALVES = HD / 64;
  constexpr int Q_BYTES = TA_ROWS * HD * 2, KV_BYTES = TA_KEYS * HD * 2, P_BYTES = TA_ROWS * TA_KEYS * 2;
  constexpr int HALF_BYTES = 128 * 128;                 // one [128][64] bfloat16 block
  constexpr int KB_BYTES = TA_KEYS * 128;               // one [TA_KEYS][64] bfloat16 block of K or V
  constexpr uint32_t TMEM_COLS = TA_KEYS == 128 ? 512 : 256;   // two S buffers of TA_KEYS columns, then the O tile
  extern __shared__ unsigned char ta_smem_raw[];
  __shared__ __align__(8) unsigned long long q_bar, k_full[2], k_empty[2], v_full[2], v_empty[2], s_ready[2], p_ready, p_free[2], o_ready;
  __shared__ uint32_t tmem_slot;
  __shared__ float l_other[TA_ROWS];
  __shared__ float m_half[2][TA_ROWS];                  // the two threads of a row tell each other their half's maximum
  unsigned char* smem = ta_smem_raw + ((1024u - (tma::smem_addr(ta_smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + Q_BYTES;                   // 2 buffers
  unsigned char* v_s = k_s + 2 * KV_BYTES;              // 2 buffers
  unsigned char* p_s = v_s + 2 * KV_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int G = nh / nkv, packs = G / gp, tq = TA_ROWS / gp;
  // grid.x runs over the head packs and grid.y over the query tiles from the last to the first, so blocks are
  // handed out with the most keys first across all heads.
  const int tile = gridDim.y - 1 - blockIdx.y;
  const int b = tiles[2 * tile], q0 = tiles[2 * tile + 1];
  const int kvh = blockIdx.x / packs, head0 = kvh * G + (blockIdx.x % packs) * gp;
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int L = context_lens[b], start = L - q_len;
  const int n_tok = min(tq, q_len - q0);
  const int p_lo = start + q0, p_hi = p_lo + n_tok - 1, hi = p_hi + 1;
  int lo = window > 0 ? max(0, p_lo - window + 1) : 0;
  const int lo_seen = lo;                                // keys below this are seen by no row of the tile
  lo = (lo / TA_KEYS) * TA_KEYS;
  const int n_tiles = (hi - lo + TA_KEYS - 1) / TA_KEYS;
  const int* bt = block_tables + (int64_t)b * bt_stride;

  if (threadIdx.x == 0) {
    tma::mbar_init(&q_bar, 1);
    for (int s = 0; s < 2; ++s) {
      tma::mbar_init(&k_full[s], 1);                      // K and V have rings of their own: a K buffer is free again as soon
      tma::mbar_init(&k_empty[s], 1);                     // as Q K^T has read it, a V buffer only after P V, a tile's time later
      tma::mbar_init(&v_full[s], 1);
      tma::mbar_init(&v_empty[s], 1);
    }
    tma::mbar_init(&s_ready[0], 1);
    tma::mbar_init(&s_ready[1], 1);
    tma::mbar_init(&p_ready, 8);                          // one arrival per softmax warp
    tma::mbar_init(&p_free[0], 1);
    tma::mbar_init(&p_free[1], 1);
    tma::mbar_init(&o_ready, 1);
    tma::mbar_fence_init();
    tma::prefetch_map(&q_map);
    tma::prefetch_map(&kv_map);
  }
  if (warp == 1) tc5::tmem_alloc(&tmem_slot, TMEM_COLS);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + 2 * TA_KEYS;
  pdl_wait();                                            // q, and the newest keys and values, come from the kernel before
  bool ok = true;

  if (warp == 0 || warp == 10) {
    // Two warps stream the pages of a key tile: warp 0 K (and Q, once), warp 10 V.  Lane l issues the box of page
    // l / HALVES, half l % HALVES, so a tile's boxes leave in one warp instruction (a tensor-map copy is a
    // per-thread instruction).
    const bool is_v = warp == 10;
    if (!is_v && lane == 0) {
      // Q: head h of the pack, 64-column half c -> block c of the A operand, rows h * tq ...
      tma::mbar_expect_tx(&q_bar, (unsigned)(gp * HALVES * tq * 128));
      for (int h = 0; h < gp; ++h)
        for (int c = 0; c < HALVES; ++c)
          tma::load_2d(q_s + c * HALF_BYTES + h * tq * 128, &q_map, (head0 + h) * HD + c * 64, tok0 + q0, &q_bar);
    }
    const int boxes = (TA_KEYS / page_size) * HALVES;              // <= 32 for pages of 8 and more
    const unsigned box_bytes = (unsigned)page_size * 128;
    const int row_off = is_v ? nkv * page_size : 0;
    unsigned char* dst0 = is_v ? v_s : k_s;
    const int pg = lane / HALVES, hf = lane % HALVES;
    unsigned long long* const full = is_v ? v_full : k_full;
    unsigned long long* const empty = is_v ? v_empty : k_empty;
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int s = it & 1, kt = lo + it * TA_KEYS;
      ok = tma::mbar_wait(&empty[s], ((it >> 1) & 1) ^ 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      int first_row = -1;
      if (lane < boxes) {
        const int j0 = kt + pg * page_size;
        if (j0 < hi && j0 + page_size > lo_seen) {
          const int page = bt[j0 / page_size];
          if (page >= 0) first_row = ((page * 2) * nkv + kvh) * page_size + row_off;
        }
      }
      const unsigned n_boxes = __popc(__ballot_sync(0xffffffffu, first_row >= 0));
      if (lane == 0) tma::mbar_expect_tx(&full[s], n_boxes * box_bytes);
      __syncwarp();
      if (first_row >= 0)
        tma::load_2d(dst0 + s * KV_BYTES + hf * KB_BYTES + pg * page_size * 128, &kv_map, hf * 64, first_row, &full[s]);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc5::instr_desc_bf16(TA_ROWS, TA_KEYS);
      constexpr uint32_t idesc_o = tc5::instr_desc_bf16(TA_ROWS, HD, true);
      ok = tma::mbar_wait(&q_bar, 0);
      // S(it) = Q K(it)^T into S buffer it % 2.  The buffer was last read by the softmax of tile it - 2, which
      // arrived on p_ready(it - 2) before this thread issued P V (it - 2).
      auto issue_qk = [&](int it) -> bool {
        const int s = it & 1;
        if (!tma::mbar_wait(&k_full[s], (it >> 1) & 1)) return false;
        tc5::fence_after_sync();
#pragma unroll
        for (int c = 0; c < HALVES; ++c) {
          const uint64_t a_desc = tc5::smem_desc_k_major_sw128(q_s + c * HALF_BYTES);
          const uint64_t b_desc = tc5::smem_desc_k_major_sw128(k_s + s * KV_BYTES + c * KB_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc5::mma_f16(tmem_s + s * TA_KEYS, a_desc + 2 * k, b_desc + 2 * k, idesc_s, c > 0 || k > 0);
        }
        tc5::commit(&s_ready[s]);
        tc5::commit(&k_empty[s]);                          // the K buffer may be refilled while the softmax and P V of the tile run
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int s = it & 1;
        if (it + 1 < n_tiles) {                            // one tile ahead: runs while the softmax works on tile it
          ok = issue_qk(it + 1);
          if (!ok) break;
        }
        ok = tma::mbar_wait(&p_ready, it & 1);             // P(it) is in shared memory, O is rescaled if it had to be
        if (ok) ok = tma::mbar_wait(&v_full[s], (it >> 1) & 1);
        if (!ok) break;
        tc5::fence_after_sync();
        // O += P V: A = P [128 rows][TA_KEYS] K-major (blocks of 64 keys); B = V [TA_KEYS][HD], MN-major:
        // 16 keys per MMA are 2048 bytes further in every 64-column half, the halves are KB_BYTES apart.
#pragma unroll
        for (int k = 0; k < TA_KEYS / 16; ++k) {
          const uint64_t a_desc = tc5::smem_desc_k_major_sw128(p_s + s * P_BYTES + (k >> 2) * HALF_BYTES) + 2 * (k & 3);
          const uint64_t b_desc = tc5::smem_desc_mn_major_sw128(v_s + s * KV_BYTES + k * 2048, KB_BYTES);
          tc5::mma_f16(tmem_o, a_desc, b_desc, idesc_o, it > 0 || k > 0);     // O accumulates over the key tiles
        }
        tc5::commit(&o_ready);                             // P V (it) and everything before it are done
        tc5::commit(&p_free[s]);
        tc5::commit(&v_empty[s]);
      }
    }
  } else {
    // Two threads per row: warps 2..5 take columns 0..63 of S, P and the first half of O's columns, warps 6..9
    // the other halves.  (A warp may read the 32 lanes of tensor memory given by its index modulo 4.)
    constexpr int OC = HD / 2;                            // O columns per thread
    const int lane_base = (warp & 3) * 32, half = (warp - 2) >> 2;
    const int r = lane_base + lane;
    const int hh = r / tq, tk = r % tq;
    const bool row_ok = tk < n_tok;
    const int pos = p_lo + tk;
    const uint32_t t_o = tmem_o + ((uint32_t)lane_base << 16) + half * OC;
    float m = -INFINITY, l = 0.f;                          // m: the row's reference maximum (may lag behind the true one)
    const float neg_inf = -INFINITY;
    // Every softmax warp runs every tile's barriers, also after a wait has given up (ok == false): then only the
    // work is skipped, so no warp is left waiting at a barrier for a partner that has gone.
    for (int it = 0; it < n_tiles; ++it) {
      const int s = it & 1, kt = lo + it * TA_KEYS;
      const uint32_t t_s = tmem_s + s * TA_KEYS + ((uint32_t)lane_base << 16);
      constexpr int KH = TA_KEYS / 2;
      float sv[KH];
      float mx = neg_inf;
      const bool need_mask = kt + TA_KEYS - 1 > p_lo || (window > 0 && kt <= p_hi - window) || n_tok * gp < TA_ROWS;
      if (ok) ok = tma::mbar_wait(&s_ready[s], (it >> 1) & 1);
      if (kt + TA_KEYS > hi || kt < lo_seen) {
        // Rows of V that hold no key this tile may use must be zero (0 * anything-else would not be 0):
        // thread (r, half) clears its 64-column half of key row r, once the tile's pages have landed.  (The wait
        // stands after the one for S: Q K^T of this tile was issued after P V of the tile two before, so the
        // buffer's load before this one is over and the parity cannot be mistaken for it.)
        if (ok) ok = tma::mbar_wait(&v_full[s], (it >> 1) & 1);
        const int j = kt + r;
        if (ok && r < TA_KEYS && (j >= hi || j < lo_seen) && half < HALVES) {
          uint4* row = reinterpret_cast<uint4*>(v_s + s * KV_BYTES + half * KB_BYTES + r * 128);
#pragma unroll
          for (int q = 0; q < 8; ++q) row[q] = make_uint4(0, 0, 0, 0);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc5::fence_after_sync();
        // This thread's half of the row's scores, read once and kept.
        if (KH == 64) {
          tc5::ld_64cols(t_s + half * KH, *reinterpret_cast<float(*)[64]>(sv));
        } else {
          tc5::ld_32cols(t_s + half * KH, *reinterpret_cast<float(*)[32]>(sv));
        }
        tc5::wait_ld();
        if (need_mask) {
#pragma unroll
          for (int jj = 0; jj < KH; ++jj) {
            const int j = kt + half * KH + jj;
            if (!(row_ok && j <= pos && (window <= 0 || j > pos - window))) sv[jj] = neg_inf;
            mx = fmaxf(mx, sv[jj]);
          }
        } else {
#pragma unroll
          for (int jj = 0; jj < KH; ++jj) mx = fmaxf(mx, sv[jj]);
        }
      }
      // The half's maximum goes to the partner thread (same row, other half: four warps further).
      m_half[half][r] = mx;
      asm volatile("bar.sync %0, 64;\n" ::"r"(2 + (warp & 3)) : "memory");
      mx = fmaxf(mx, m_half[half ^ 1][r]);
      asm volatile("bar.sync %0, 64;\n" ::"r"(2 + (warp & 3)) : "memory");      // read before the next tile overwrites
      if (ok) {
        // Raise the reference maximum only on the first tile with a seen key and when the new maximum is more
        // than 2^8 (in the exponent's units) above it; both threads of a row decide alike.
        const bool raise = mx > neg_inf && (m == neg_inf || (mx - m) * scale_log2 > 8.0f);
        float alpha = 1.f;
        if (raise) {
          alpha = ex2((m - mx) * scale_log2);                // m = -inf gives 0
          m = mx;
          l *= alpha;
        }
        if (it > 0 && __any_sync(0xffffffffu, raise)) {
          // Rescale this thread's half of its row of O in tensor memory, after P V (it - 1) has finished.
          ok = tma::mbar_wait(&o_ready, (it - 1) & 1);
          if (ok) {
            tc5::fence_after_sync();
            float v[OC];
            if (OC == 64) tc5::ld_64cols(t_o, *reinterpret_cast<float(*)[64]>(v));
            else tc5::ld_32cols(t_o, *reinterpret_cast<float(*)[32]>(v));
            tc5::wait_ld();
#pragma unroll
            for (int jj = 0; jj < OC; ++jj) v[jj] *= alpha;
            if (OC == 64) tc5::st_64cols(t_o, *reinterpret_cast<float(*)[64]>(v));
            else tc5::st_32cols(t_o, *reinterpret_cast<float(*)[32]>(v));
            tc5::wait_st();
          }
        }
      }
      if (ok) ok = tma::mbar_wait(&p_free[s], ((it >> 1) & 1) ^ 1);      // P V (it - 2) has read this P buffer
      if (ok) {
        const float mu_s = (m == neg_inf ? 0.f : m) * scale_log2;
        // p = 2^(s * scale - reference * scale) (masked scores are -inf and give 0), rounded to bfloat16 into P:
        // keys c .. c+31 of row r are in block c / 64, 16-byte pieces (c % 64) / 8 .. +3, swizzled by the row
#pragma unroll
        for (int c0 = 0; c0 < KH; c0 += 32) {
          const int c = half * KH + c0;
          uint32_t pk[16];
#pragma unroll
          for (int jj = 0; jj < 32; jj += 2) {
            const float p0 = ex2(fmaf(sv[c0 + jj], scale_log2, -mu_s)), p1 = ex2(fmaf(sv[c0 + jj + 1], scale_log2, -mu_s));
            l += p0 + p1;
            __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
            pk[jj >> 1] = *reinterpret_cast<uint32_t*>(&h2);
          }
          unsigned char* row = p_s + s * P_BYTES + (c >> 6) * HALF_BYTES + r * 128;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int piece = ((c & 63) >> 3) + q;
            *reinterpret_cast<uint4*>(row + ((piece ^ (r & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
          }
        }
        // P (and the zeroed rows of V) were written by ordinary stores: make them visible to the tensor core's reads.
        fence_async_smem();
        tc5::fence_before_sync();
      }
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&p_ready);            // ok is the same in all lanes of a warp here
    }
    // the row's sum is the two threads' sums; softmax warps meet at a named barrier of their own
    if (half == 1) l_other[r] = l;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    if (half == 0) l += l_other[r];
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    if (half == 0) l_other[r] = l;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    l = l_other[r];
    if (ok) ok = tma::mbar_wait(&o_ready, (n_tiles - 1) & 1);          // the last P V is done
    float o_acc[OC];
    if (ok) {
      tc5::fence_after_sync();
      if (OC == 64) tc5::ld_64cols(t_o, *reinterpret_cast<float(*)[64]>(o_acc));
      else tc5::ld_32cols(t_o, *reinterpret_cast<float(*)[32]>(o_acc));
      tc5::wait_ld();
    }
    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = out + (int64_t)(tok0 + q0 + tk) * out_row_stride + (int64_t)(head0 + hh) * HD + half * OC;
#pragma unroll
      for (int q = 0; q < OC / 8; ++q) {
        uint4 pk;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) h2[jj] = __floats2bfloat162_rn(o_acc[q * 8 + 2 * jj] * inv, o_acc[q * 8 + 2 * jj + 1] * inv);
        *reinterpret_cast<uint4*>(dst + q * 8) = pk;
      }
    }
  }
  if (!ok) atomicOr(err + 1, 1);
  pdl_launch_dependents();
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tmem_slot, TMEM_COLS);
}

// ---- two softmax groups ---------------------------------------------------------------------------------------
// The same block of 128 rows, key tiles of 128, but the eight softmax warps work as two groups of four (a thread
// per row) that take the key tiles in turn: while group 0 computes the exponentials of tile t, group 1 reads and
// reduces tile t + 1, so a tile's chain of waits (S ready, tensor-memory loads, P handed over) overlaps with the
// other group's arithmetic instead of adding to it.
//   tensor memory: three S buffers of 128 columns (Q K^T runs two tiles ahead), then the O tile;
//   shared memory: Q, rings of three K and three V buffers.
// A thread reads its row of S twice, in pieces of 32 columns: once for the maximum, once for the exponentials.
// P never goes through shared memory: the thread writes it, rounded to bfloat16 and two to a column, over the
// first 64 columns of the S buffer it came from (the writes trail the reads), and P V takes its A operand from
// tensor memory.  Shared memory, whose 128 bytes a clock the operands of the products, the arriving K and V
// tiles and, before, P shared, is what bounds a tile's time; this takes P's 64 KB a tile off it.
// The row's reference maximum is a chain through the tiles: the group of tile t publishes reference(t) in shared
// memory as soon as it has the tile's maximum (named barriers 2 and 3: the publishing group arrives, the other
// waits), and raises it only when the tile's maximum exceeds it by more than 2^8, rescaling O in tensor memory
// after P V (t - 1).  Each group keeps the sum of its own tiles relative to the last reference it used; the two
// are brought to the final reference and added at the end.
// Parities: a wait names a phase of its barrier by parity, which is only right while the phase before it is
// over.  Every wait below stands where that is known (the comment beside it says why).
template <int HD>
__global__ void __launch_bounds__(TA_THREADS)
attn_prefill_tcgen05_two_groups_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kv_map,
                                       bf16* __restrict__ out, int64_t out_row_stride, const int* __restrict__ block_tables,
                                       int bt_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                                       const int* __restrict__ tiles, int nh, int nkv, int gp, int page_size, float scale_log2,
                                       int window, int* __restrict__ err) {
  constexpr int KEYS = 128, HALVES = HD / 64;
  constexpr int Q_BYTES = TA_ROWS * HD * 2, KV_BYTES = KEYS * HD * 2, RING = 3;
  constexpr int HALF_BYTES = 128 * 128, KB_BYTES = KEYS * 128;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ unsigned char ta_smem_raw[];
  __shared__ __align__(8) unsigned long long q_bar, k_full[RING], k_empty[RING], v_full[RING], v_empty[RING], s_ready[3], p_ready[2],
      o_ready[2];
  __shared__ uint32_t tmem_slot;
  __shared__ float ref_m[2][TA_ROWS];                   // reference(t) of every row, for t even and odd
  unsigned char* smem = ta_smem_raw + ((1024u - (tma::smem_addr(ta_smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + Q_BYTES;
  unsigned char* v_s = k_s + RING * KV_BYTES;
  const int warp = tc5::uniform_warp_index(), lane = threadIdx.x & 31;

  const int G = nh / nkv, packs = G / gp, tq = TA_ROWS / gp;
  const int tile = gridDim.y - 1 - blockIdx.y;
  const int b = tiles[2 * tile], q0 = tiles[2 * tile + 1];
  const int kvh = blockIdx.x / packs, head0 = kvh * G + (blockIdx.x % packs) * gp;
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int L = context_lens[b], start = L - q_len;
  const int n_tok = min(tq, q_len - q0);
  const int p_lo = start + q0, p_hi = p_lo + n_tok - 1, hi = p_hi + 1;
  int lo = window > 0 ? max(0, p_lo - window + 1) : 0;
  const int lo_seen = lo;
  lo = (lo / KEYS) * KEYS;
  const int n_tiles = (hi - lo + KEYS - 1) / KEYS;
  const int* bt = block_tables + (int64_t)b * bt_stride;

  if (threadIdx.x == 0) {
    tma::mbar_init(&q_bar, 1);
    for (int s = 0; s < RING; ++s) {
      tma::mbar_init(&k_full[s], 1);
      tma::mbar_init(&k_empty[s], 1);
      tma::mbar_init(&v_full[s], 1);
      tma::mbar_init(&v_empty[s], 1);
      tma::mbar_init(&s_ready[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      tma::mbar_init(&p_ready[s], 4);                     // one arrival per warp of the group
      tma::mbar_init(&o_ready[s], 1);
    }
    tma::mbar_fence_init();
    tma::prefetch_map(&q_map);
    tma::prefetch_map(&kv_map);
  }
  if (warp == 1) tc5::tmem_alloc(&tmem_slot, TMEM_COLS);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + 3 * KEYS;
  // The two producing warps look the first tile's pages up before the wait: block tables are written by the host.
  const bool is_v = warp == 10;
  const int boxes = (KEYS / page_size) * HALVES;
  const int row_off = is_v ? nkv * page_size : 0;
  const int pg = lane / HALVES, hf = lane % HALVES;
  auto first_row_of = [&](int kt) {
    int first_row = -1;
    if (lane < boxes) {
      const int j0 = kt + pg * page_size;
      if (j0 < hi && j0 + page_size > lo_seen) {
        const int page = bt[j0 / page_size];
        if (page >= 0) first_row = ((page * 2) * nkv + kvh) * page_size + row_off;
      }
    }
    return first_row;
  };
  int first_row_0 = -1;
  if (warp == 0 || warp == 10) first_row_0 = first_row_of(lo);
  pdl_wait();
  bool ok = true;

  if (warp == 0 || warp == 10) {
    if (!is_v) {
      // Q: head h of the pack, 64-column half c -> block c of the A operand, rows h * tq ...; a box a lane
      if (lane == 0) tma::mbar_expect_tx(&q_bar, (unsigned)(gp * HALVES * tq * 128));
      __syncwarp();
      if (lane < gp * HALVES) {
        const int h = lane / HALVES, c = lane % HALVES;
        tma::load_2d(q_s + c * HALF_BYTES + h * tq * 128, &q_map, (head0 + h) * HD + c * 64, tok0 + q0, &q_bar);
      }
    }
    const unsigned box_bytes = (unsigned)page_size * 128;
    unsigned char* dst0 = is_v ? v_s : k_s;
    unsigned long long* const full = is_v ? v_full : k_full;
    unsigned long long* const empty = is_v ? v_empty : k_empty;
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int s = it % RING, kt = lo + it * KEYS;
      ok = tma::mbar_wait(&empty[s], ((it / RING) & 1) ^ 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int first_row = it == 0 ? first_row_0 : first_row_of(kt);
      const unsigned n_boxes = __popc(__ballot_sync(0xffffffffu, first_row >= 0));
      if (lane == 0) tma::mbar_expect_tx(&full[s], n_boxes * box_bytes);
      __syncwarp();
      if (first_row >= 0)
        tma::load_2d(dst0 + s * KV_BYTES + hf * KB_BYTES + pg * page_size * 128, &kv_map, hf * 64, first_row, &full[s]);
    }
  } else if (warp == 1) {
    // The issuing warp: all lanes run the loop with the same values, an elected lane issues.
    constexpr uint32_t idesc_s = tc5::instr_desc_bf16(TA_ROWS, KEYS);
    constexpr uint32_t idesc_o = tc5::instr_desc_bf16(TA_ROWS, HD, true);
    const tc5::DescWords q_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(q_s));
    const tc5::DescWords k_desc = tc5::words_of(tc5::smem_desc_k_major_sw128(k_s));
    const tc5::DescWords v_desc = tc5::words_of(tc5::smem_desc_mn_major_sw128(v_s, KB_BYTES));
    ok = tc5::mbar_wait_warp(&q_bar, 0);
    // S(it) = Q K(it)^T into S buffer it % 3, which held S and then P of tile it - 3: P V (it - 3) was issued an
    // iteration ago, and the tensor core runs this warp's products in the order of their issue.
    auto issue_qk = [&](int it) -> bool {
      const int s = it % RING;
      if (!tc5::mbar_wait_warp(&k_full[s], (it / RING) & 1)) return false;
      tc5::fence_after_sync();
#pragma unroll
      for (int c = 0; c < HALVES; ++c) {
#pragma unroll
        for (int k = 0; k < 4; ++k)                          // (offsets in units of 16 bytes)
          tc5::mma_f16_elect(tmem_s + s * KEYS, q_desc, (c * HALF_BYTES >> 4) + 2 * k, k_desc,
                             ((s * KV_BYTES + c * KB_BYTES) >> 4) + 2 * k, idesc_s, c > 0 || k > 0);
      }
      tc5::commit_elect(&s_ready[s]);
      tc5::commit_elect(&k_empty[s]);
      return true;
    };
    if (ok) ok = issue_qk(0);
    if (ok && n_tiles > 1) ok = issue_qk(1);
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int s = it % RING, g = it & 1;
      if (it + 2 < n_tiles) {                              // two tiles ahead: one for each softmax group
        ok = issue_qk(it + 2);
        if (!ok) break;
      }
      ok = tc5::mbar_wait_warp(&p_ready[g], (it >> 1) & 1);  // P(it) is in tensor memory, O is rescaled if it had to be
      if (ok) ok = tc5::mbar_wait_warp(&v_full[s], (it / RING) & 1);
      if (!ok) break;
      tc5::fence_after_sync();
      // O += P V: A = P, 8 columns of tensor memory for the 16 keys of a step; B = V [KEYS][HD], MN-major: 16 keys
      // are 2048 bytes further in every 64-column half, the halves are KB_BYTES apart.
#pragma unroll
      for (int k = 0; k < KEYS / 16; ++k)
        tc5::mma_f16_a_in_tmem_elect(tmem_o, tmem_s + s * KEYS + k * 8, v_desc, (s * KV_BYTES + k * 2048) >> 4, idesc_o, it > 0 || k > 0);
      tc5::commit_elect(&o_ready[g]);                      // P V (it) and everything before it are done
      tc5::commit_elect(&v_empty[s]);
    }
  } else {
    const int lane_base = (warp & 3) * 32, g = (warp - 2) >> 2;
    const int r = lane_base + lane;
    const int hh = r / tq, tk = r % tq;
    const bool row_ok = tk < n_tok;
    const int pos = p_lo + tk;
    const uint32_t t_row = (uint32_t)lane_base << 16;
    const float neg_inf = -INFINITY;
    float m_mine = neg_inf, l = 0.f;                       // l: the sum over this group's tiles, relative to m_mine
    // the keys this row sees: j_min .. j_max (none for a row beyond the tile's tokens)
    const int j_max = row_ok ? pos : -(1 << 30), j_min = window > 0 ? pos - window + 1 : -(1 << 30);
    // Both groups run every named barrier of every tile, also after a wait has given up (ok == false): then only
    // the work is skipped, so no warp is left waiting for a partner that has gone.
    for (int it = g; it < n_tiles; it += 2) {
      const int kt = lo + it * KEYS;
      const uint32_t t_s = tmem_s + (it % 3) * KEYS + t_row;
      const bool need_mask = kt + KEYS - 1 > p_lo || (window > 0 && kt <= p_hi - window) || n_tok * gp < TA_ROWS;
      // Q K^T (it) was issued after Q K^T (it - 3), which this group's last tile (it - 2) waited for in its turn.
      if (ok) ok = tma::mbar_wait(&s_ready[it % 3], (it / 3) & 1);
      ok = __all_sync(0xffffffffu, ok);
      float mx = neg_inf;
      const int c_min = j_min - kt, c_max = j_max - kt;      // the same as columns of this tile
      auto seen = [&](int col) { return col >= c_min && col <= c_max; };
      // A masked tile by pieces of 32 columns: the rows of a warp are consecutive tokens (of one or two heads), so
      // most pieces are seen whole, or not at all, by the whole warp; only the others are tested column by column.
      // 0: all rows of the warp see all of the piece, 1: none sees any of it, 2: mixed.
      auto piece_kind = [&](int c0) {
        if (!need_mask) return 0;
        if (__all_sync(0xffffffffu, c_min <= c0 && c_max >= c0 + 31)) return 0;
        if (__all_sync(0xffffffffu, c_max < c0 || c_min > c0 + 31)) return 1;
        return 2;
      };
      // The thread's whole row of S, 128 scores, stays in registers from the maximum to the exponentials: tensor
      // memory is read once, and the reads' latency is paid once a tile.
      float s_lo[64], s_hi[64];
      auto piece = [](float (&half)[64], int q) -> float (&)[32] { return *reinterpret_cast<float(*)[32]>(&half[32 * q]); };
      if (ok) {
        tc5::fence_after_sync();
        auto piece_max = [&](const float (&sv)[32], int c0) {
          const int kind = piece_kind(c0);
          if (kind == 0) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) mx = fmaxf(mx, sv[jj]);
          } else if (kind == 2) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              if (seen(c0 + jj)) mx = fmaxf(mx, sv[jj]);
          }
        };
        tc5::ld_64cols(t_s, s_lo);
        tc5::wait_ld();
        tc5::ld_64cols(t_s + 64, s_hi);                      // on its way while the first half is worked on
        piece_max(piece(s_lo, 0), 0);
        piece_max(piece(s_lo, 1), 32);
        tc5::wait_ld();
        piece_max(piece(s_hi, 0), 64);
        piece_max(piece(s_hi, 1), 96);
      }
      // reference(it - 1) from the other group, reference(it) to it
      float m_prev = neg_inf;
      if (it > 0) {
        asm volatile("bar.sync %0, 256;\n" ::"r"(2 + ((it - 1) & 1)) : "memory");
        m_prev = ref_m[(it - 1) & 1][r];
      }
      const bool raise = ok && mx > neg_inf && (m_prev == neg_inf || (mx - m_prev) * scale_log2 > 8.0f);
      const float m_new = raise ? mx : m_prev;
      ref_m[it & 1][r] = m_new;
      __threadfence_block();
      asm volatile("bar.arrive %0, 256;\n" ::"r"(2 + (it & 1)) : "memory");
      if (ok) {
        if (m_new != m_mine) {                               // m_mine = -inf: nothing summed yet
          l *= ex2((m_mine - m_new) * scale_log2);
          m_mine = m_new;
        }
        if (it > 0 && __any_sync(0xffffffffu, raise)) {
          // Rescale this row of O after P V (it - 1).  P V (it - 3), the phase before on that barrier, is over:
          // Q K^T (it) was issued after it, and S(it) has been waited for.
          ok = tma::mbar_wait(&o_ready[(it - 1) & 1], ((it - 1) >> 1) & 1);
          if (ok) {
            tc5::fence_after_sync();
            const float alpha = raise ? ex2((m_prev - m_new) * scale_log2) : 1.f;      // m_prev = -inf gives 0
#pragma unroll
            for (int c0 = 0; c0 < HD; c0 += 16) {             // (a rare path: small pieces, the row of S is held meanwhile)
              float v[16];
              tc5::ld_16cols(tmem_o + t_row + c0, v);
              tc5::wait_ld();
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) v[jj] *= alpha;
              tc5::st_16cols(tmem_o + t_row + c0, *reinterpret_cast<uint32_t(*)[16]>(v));
            }
            tc5::wait_st();
          }
        }
      }
      if (kt + KEYS > hi || kt < lo_seen) {
        // Rows of V that hold no key this tile may use must be zero (0 * anything-else would not be 0).  The load
        // before this one into the buffer, V (it - 3), is over: P V (it - 3) was issued before Q K^T (it).
        if (ok) ok = tma::mbar_wait(&v_full[it % RING], (it / RING) & 1);
        const int j = kt + r;
        if (ok && (j >= hi || j < lo_seen)) {
#pragma unroll
          for (int hf = 0; hf < HALVES; ++hf) {
            uint4* row = reinterpret_cast<uint4*>(v_s + (it % RING) * KV_BYTES + hf * KB_BYTES + r * 128);
#pragma unroll
            for (int q = 0; q < 8; ++q) row[q] = make_uint4(0, 0, 0, 0);
          }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        const float mu_s = (m_new == neg_inf ? 0.f : m_new) * scale_log2;
        // p = 2^(s * scale - reference * scale), 0 for a key the row does not see (its score is set to -inf), rounded
        // to bfloat16: keys c .. c+31 of the row go to columns c / 2 .. c / 2 + 15 of the S buffer, which are read already.
        auto piece_of_p = [&](float (&sv)[32], int c) {
          const int kind = piece_kind(c);
          uint32_t pk[16];
          if (kind == 1) {
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) pk[jj] = 0u;
          } else {
            if (kind == 2) {
#pragma unroll
              for (int jj = 0; jj < 32; ++jj)
                if (!seen(c + jj)) sv[jj] = neg_inf;
            }
#pragma unroll
            for (int jj = 0; jj < 32; jj += 2) {
              const float p0 = ex2(fmaf(sv[jj], scale_log2, -mu_s)), p1 = ex2(fmaf(sv[jj + 1], scale_log2, -mu_s));
              l += p0 + p1;
              __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
              pk[jj >> 1] = *reinterpret_cast<uint32_t*>(&h2);
            }
          }
          tc5::st_16cols(t_s + (c >> 1), pk);
        };
        piece_of_p(piece(s_lo, 0), 0);
        piece_of_p(piece(s_lo, 1), 32);
        piece_of_p(piece(s_hi, 0), 64);
        piece_of_p(piece(s_hi, 1), 96);
        tc5::wait_st();
        fence_async_smem();                                  // the zeroed rows of V were written by ordinary stores
        tc5::fence_before_sync();
      }
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&p_ready[g]);
    }
    // The group that did not take the last tile takes the last reference off its barrier.
    if (g == (n_tiles & 1)) asm volatile("bar.sync %0, 256;\n" ::"r"(2 + ((n_tiles - 1) & 1)) : "memory");
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    const float m_fin = ref_m[(n_tiles - 1) & 1][r];
    // The two groups' sums meet in the first K buffer: every Q K^T is over (the group of the last tile waited for
    // its S, and both groups have met since), and the block's shared memory has no room to spare.
    float* l_part = reinterpret_cast<float*>(k_s);
    l_part[g * TA_ROWS + r] = m_mine == neg_inf ? 0.f : l * ex2((m_mine - m_fin) * scale_log2);
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    l = l_part[r] + l_part[TA_ROWS + r];
    // The last P V.  The phase before it on that barrier is P V (n - 3), which nothing so far has waited for: Q K^T
    // (n - 1) was issued after P V (n - 4) only, the phase before P V (n - 2) on the other barrier.  So that one first
    // (the group of the last tile waited for S (n - 1), and both groups have met since); the products end in order.
    if (ok && n_tiles > 1) ok = tma::mbar_wait(&o_ready[(n_tiles - 2) & 1], ((n_tiles - 2) >> 1) & 1);
    if (ok) ok = tma::mbar_wait(&o_ready[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
    ok = __all_sync(0xffffffffu, ok);
    // O / l goes through Q's place in shared memory (every Q K^T is over) so that it leaves in whole rows: a thread
    // holds one row of 128 lanes, and 32 threads storing 32 different rows would be 32 separate lines a store.
    constexpr int OC = HD / 2, PIECES = HD / 8;              // group 0 takes the first half of the row's columns, group 1 the other
    if (ok) {
      tc5::fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int c0 = 0; c0 < OC; c0 += 32) {
        float o_acc[32];
        tc5::ld_32cols(tmem_o + t_row + g * OC + c0, o_acc);
        tc5::wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 pk;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) h2[jj] = __floats2bfloat162_rn(o_acc[q * 8 + 2 * jj] * inv, o_acc[q * 8 + 2 * jj + 1] * inv);
          const int piece = (g * OC + c0) / 8 + q;
          *reinterpret_cast<uint4*>(q_s + r * (HD * 2) + ((piece ^ (r & 7)) << 4)) = pk;
        }
      }
    }
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    if (ok) {
      constexpr int ROWS_AT_ONCE = 32 / PIECES;
      const int piece = lane % PIECES;
      for (int row = (warp - 2) * 16 + lane / PIECES; row < (warp - 1) * 16; row += ROWS_AT_ONCE) {
        const int tok = row % tq;
        if (tok < n_tok) {
          const uint4 pk = *reinterpret_cast<const uint4*>(q_s + row * (HD * 2) + ((piece ^ (row & 7)) << 4));
          *reinterpret_cast<uint4*>(out + (int64_t)(tok0 + q0 + tok) * out_row_stride + (int64_t)(head0 + row / tq) * HD + piece * 8) = pk;
        }
      }
    }
  }
  if (!ok) atomicOr(err + 1, 1);
  pdl_launch_dependents();
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tmem_slot, TMEM_COLS);
}

template <int HD, int KT, bool TWO_GROUPS>
int launch_ta(const void* q_map, const void* kv_map, void* out, int64_t out_row_stride, const int* block_tables, int bt_stride,
              const int* cu_seqlens, const int* context_lens, const int* tiles, int num_tiles, int nh, int nkv, int gp,
              int page_size, float scale, int window, int* err, cudaStream_t stream) {
  const size_t smem = TWO_GROUPS ? (size_t)TA_ROWS * HD * 2 + 6 * (size_t)KT * HD * 2 + 1024
                                 : (size_t)TA_ROWS * HD * 2 + 4 * (size_t)KT * HD * 2 + 2 * (size_t)TA_ROWS * KT * 2 + 1024;
  auto kernel = TWO_GROUPS ? attn_prefill_tcgen05_two_groups_kernel<HD> : attn_prefill_tcgen05_kernel<HD, KT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_attn_prefill_tcgen05: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  // Heads fastest, tiles (the ones with the most keys first) slowest: the long tiles of all heads start in the first round.
  // (Tiles fastest, so that the blocks of a round share one or two heads' keys in L2, measured the same at 16,384 tokens
  // and 16% slower at 2,048, where the last round then holds long tiles.)
  dim3 grid(nkv * (nh / nkv / gp), num_tiles);
  me_launch(kernel, grid, dim3(TA_THREADS), smem, stream, *reinterpret_cast<const CUtensorMap*>(q_map),
            *reinterpret_cast<const CUtensorMap*>(kv_map), (bf16*)out, out_row_stride, block_tables, bt_stride, cu_seqlens,
            context_lens, tiles, nh, nkv, gp, page_size, scale * 1.4426950408889634f, window, err);
  return 0;
}

}  // namespace

// How many heads of a group share a block of the tcgen05 prefill kernel (a block covers 128 / that many
// query tokens); 0 if the kernel refuses the shape.
ME_API int me_attn_prefill_tcgen05_heads_per_block(int nh, int nkv, int hd, int page_size) {
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv || page_size < 8 || 128 % page_size) return 0;
  const int G = nh / nkv;
  for (int gp = 16; gp >= 1; gp >>= 1)
    if (G % gp == 0) return gp;
  return 1;
}

// q_map: the step's packed q|k|v rows as [tokens][row width], boxes (128 / heads-per-block) x 64; kv_map: the cache
// slot as [pages * 2 * kv_heads * page_size][head_dim], boxes page_size x 64; both with the 128-byte swizzle.
// ``tiles``: (request, first local query) per block, each covering 128 / heads-per-block query tokens.
ME_API int me_attn_prefill_tcgen05(const void* q_map, const void* kv_map, void* out, int64_t out_row_stride,
                                   const int* block_tables, int bt_stride, const int* cu_seqlens, const int* context_lens,
                                   const int* tiles, int num_tiles, int nh, int nkv, int hd, int page_size, float scale,
                                   int window, int key_tile, int* err, cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  const int gp = me_attn_prefill_tcgen05_heads_per_block(nh, nkv, hd, page_size);
  ME_REQUIRE(gp > 0, "me_attn_prefill_tcgen05: head_dim %d, %d/%d heads, pages of %d are not taken", hd, nh, nkv, page_size);
  ME_REQUIRE(q_map != nullptr && kv_map != nullptr && err != nullptr, "me_attn_prefill_tcgen05: tensor maps and the error word are required");
  ME_REQUIRE((out_row_stride * 2) % 16 == 0 && ((uintptr_t)out & 15) == 0, "me_attn_prefill_tcgen05: output rows must be 16-byte aligned");
  ME_REQUIRE(num_tiles <= 65535, "me_attn_prefill_tcgen05: %d query tiles in one step are too many", num_tiles);
  // key_tile: keys per step of the loop.  128 (and 0): the kernel with two softmax groups and P in tensor memory, the
  // faster one; 64: the kernel with one group and P in shared memory, which needs less of both memories.
  if (key_tile == 0) key_tile = 128;
  ME_REQUIRE((key_tile == 64 || key_tile == 128) && key_tile % page_size == 0, "me_attn_prefill_tcgen05: key tile %d with pages of %d",
             key_tile, page_size);
  int rc;
#define ME_TA_ARGS q_map, kv_map, out, out_row_stride, block_tables, bt_stride, cu_seqlens, context_lens, tiles, num_tiles, nh, nkv, gp, \
                   page_size, scale, window, err, stream
  if (hd == 64) rc = key_tile == 64 ? launch_ta<64, 64, false>(ME_TA_ARGS) : launch_ta<64, 128, true>(ME_TA_ARGS);
  else rc = key_tile == 64 ? launch_ta<128, 64, false>(ME_TA_ARGS) : launch_ta<128, 128, true>(ME_TA_ARGS);
#undef ME_TA_ARGS
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_attn_prefill_tcgen05");
  return 0;
}
