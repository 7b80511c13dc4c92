// Paged attention for portions of prompts on the tensor cores (bfloat16, head_dim 64 or 128).
//
// Same semantics as csrc/attention_chunk.cu (the reference's csrc/paged_prefill.cu:177-247 in
// spirit: a tile of queries against tiles of cached keys gathered through the block table,
// online softmax in float32, O accumulated in float32, P rounded to bfloat16 before P V).
// One block = 64 rows x one group of query heads of one key/value head: the rows are
// (64 / GP query tokens) x (GP heads), so a K/V tile is loaded once for GP heads
// (the reference packs 32 tokens x 2 heads, csrc/paged_prefill.cu:18-19).  Four warps, each a
// strip of 16 rows; S = Q K^T and O += P V with mma.sync m16n8k16 (Q and P as register
// fragments, K and V from shared memory by ldmatrix); K/V tiles of 64 keys arrive by cp.async
// in two buffers, 16-byte pieces XOR-swizzled against bank conflicts.  Key tiles start at
// multiples of 64 from position 0, so a query's sums do not depend on how the prompt was cut.
#include "common.cuh"
#include "mma_prims.cuh"

namespace {

using namespace mma_prims;

constexpr int PF_ROWS = 64, PF_KEYS = 64, PF_THREADS = 128;

// Thread t copies piece (t % PIECES) of rows (t / PIECES) + k * (128 / PIECES): its piece and its swizzle
// term are the same for all its rows, so the loop is one table lookup and two copies per row.
template <int HD>
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const bf16* __restrict__ pool, const PageMap& pm,
                                             int64_t v_off, int kt, int hi) {
  constexpr int PIECES = HD / 8, ROWS_PER_PASS = PF_THREADS / PIECES;
  const int piece = threadIdx.x % PIECES, r0 = threadIdx.x / PIECES;
#pragma unroll
  for (int row = r0; row < PF_KEYS; row += ROWS_PER_PASS) {
    const int j = kt + row;
    const int64_t base = j < hi ? pm.row(j) : -1;
    const bool ok = base >= 0;
    const bf16* src = ok ? pool + base + piece * 8 : pool;
    cp_async16(tile_ptr<HD>(ks, row, piece), src, ok);
    cp_async16(tile_ptr<HD>(vs, row, piece), ok ? src + v_off : pool, ok);
  }
}

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_mma_kernel(const bf16* __restrict__ qkv, int64_t q_row_stride, bf16* __restrict__ out,
                        int64_t out_row_stride, const bf16* __restrict__ pool,
                        const int* __restrict__ block_tables, int bt_stride,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                        const int* __restrict__ tiles, int nh, int nkv, int gp, int page_size,
                        float scale_log2, int window) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);          // [64][HD]
  bf16* kv = qs + PF_ROWS * HD;                           // 2 x (K [64][HD], V [64][HD])
  constexpr int PIECES = HD / 8, KSTEPS = HD / 16, NT_S = PF_KEYS / 8, NT_O = HD / 8;
  pdl_wait();
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = nh / nkv, packs = G / gp, tq = PF_ROWS / gp;
  const int b = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
  const int kvh = blockIdx.y / packs, head0 = kvh * G + (blockIdx.y % packs) * gp;
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int L = context_lens[b], start = L - q_len;
  const int n_tok = min(tq, q_len - q0);                 // query tokens of this tile
  const int64_t v_off = (int64_t)nkv * page_size * HD;
  const PageMap pm{block_tables + (int64_t)b * bt_stride, page_size, log2_if_pow2(page_size), 2 * v_off,
                   (int64_t)kvh * page_size * HD, HD};

  // Q tile: row r = token (r / gp), head (r % gp)
  for (int c = tid; c < PF_ROWS * PIECES; c += PF_THREADS) {
    const int row = c / PIECES, piece = c % PIECES;
    const int tk = row / gp, hh = row % gp;
    const bool ok = tk < n_tok;
    const bf16* src = ok ? qkv + (int64_t)(tok0 + q0 + tk) * q_row_stride + (int64_t)(head0 + hh) * HD + piece * 8 : qkv;
    cp_async16(tile_ptr<HD>(qs, row, piece), src, ok);
  }
  const int p_lo = start + q0, p_hi = start + q0 + n_tok - 1;   // positions of the tile's queries
  const int hi = p_hi + 1;                                      // keys [lo, hi) can be seen by some row
  int lo = window > 0 ? max(0, p_lo - window + 1) : 0;
  lo = (lo / PF_KEYS) * PF_KEYS;
  const int n_tiles = (hi - lo + PF_KEYS - 1) / PF_KEYS;
  load_kv_tile<HD>(kv, kv + PF_KEYS * HD, pool, pm, v_off, lo, hi);
  cp_async_commit();

  uint32_t qf[KSTEPS][4];
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;       // rows g and g+8 of the warp's strip
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  const int pos0 = p_lo + r0 / gp, pos1 = p_lo + r1 / gp;
  const bool ok0 = r0 / gp < n_tok, ok1 = r1 / gp < n_tok;

  for (int it = 0; it < n_tiles; ++it) {
    const int kt = lo + it * PF_KEYS;
    bf16* ks = kv + (it & 1) * 2 * PF_KEYS * HD;
    bf16* vs = ks + PF_KEYS * HD;
    if (it + 1 < n_tiles) {
      bf16* kn = kv + ((it + 1) & 1) * 2 * PF_KEYS * HD;
      load_kv_tile<HD>(kn, kn + PF_KEYS * HD, pool, pm, v_off, kt + PF_KEYS, hi);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int mi = lane >> 3;
        ldmatrix_x4(qf[kk], tile_ptr<HD>(qs, warp * 16 + (mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1)));
      }
    }
    // S = Q K^T for the warp's 16 rows x 64 keys
    float s[NT_S][4];
#pragma unroll
    for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int np = 0; np < NT_S / 2; ++np) {
        uint32_t bfr[4];
        const int mi = lane >> 3;
        ldmatrix_x4(bfr, tile_ptr<HD>(ks, np * 16 + (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
        mma_bf16(s[2 * np], qf[kk], bfr[0], bfr[1]);
        mma_bf16(s[2 * np + 1], qf[kk], bfr[2], bfr[3]);
      }
    }
    // mask (only tiles that touch the diagonal, the end of the keys or the window's edge)
    const bool need_mask = kt + PF_KEYS - 1 > p_lo || (window > 0 && kt <= p_hi - window) || n_tok * gp < PF_ROWS;
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < NT_S; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = kt + i * 8 + 2 * t4 + (e & 1);
          const int pos = e < 2 ? pos0 : pos1;
          const bool okr = e < 2 ? ok0 : ok1;
          const bool seen = okr && j <= pos && (window <= 0 || j > pos - window);
          if (!seen) s[i][e] = -INFINITY;
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < NT_S; ++i) {
      mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
      mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
    const float a0 = exp2f((m0 - mu0) * scale_log2), a1 = exp2f((m1 - mu1) * scale_log2);   // m = -inf gives 0
    m0 = mn0;
    m1 = mn1;
    l0 *= a0;
    l1 *= a1;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      o[i][0] *= a0;
      o[i][1] *= a0;
      o[i][2] *= a1;
      o[i][3] *= a1;
    }
    uint32_t pf[PF_KEYS / 16][4];
#pragma unroll
    for (int i = 0; i < NT_S; ++i) {
      const float p0 = exp2f((s[i][0] - mu0) * scale_log2), p1 = exp2f((s[i][1] - mu0) * scale_log2);
      const float p2 = exp2f((s[i][2] - mu1) * scale_log2), p3 = exp2f((s[i][3] - mu1) * scale_log2);
      l0 += p0 + p1;
      l1 += p2 + p3;
      pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < PF_KEYS / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        uint32_t bfr[4];
        const int mi = lane >> 3;
        ldmatrix_x4_trans(bfr, tile_ptr<HD>(vs, kk * 16 + (mi & 1) * 8 + (lane & 7), np * 2 + (mi >> 1)));
        mma_bf16(o[2 * np], pf[kk], bfr[0], bfr[1]);
        mma_bf16(o[2 * np + 1], pf[kk], bfr[2], bfr[3]);
      }
    }
    __syncthreads();          // everyone is done with this buffer before the next load overwrites it
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
  if (ok0) {
    bf16* dst = out + (int64_t)(tok0 + q0 + r0 / gp) * out_row_stride + (int64_t)(head0 + r0 % gp) * HD;
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = pack_bf16(o[i][0] * i0, o[i][1] * i0);
  }
  if (ok1) {
    bf16* dst = out + (int64_t)(tok0 + q0 + r1 / gp) * out_row_stride + (int64_t)(head0 + r1 % gp) * HD;
#pragma unroll
    for (int i = 0; i < NT_O; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = pack_bf16(o[i][2] * i1, o[i][3] * i1);
  }
}

template <int HD>
int launch_prefill(const void* qkv, int64_t q_row_stride, void* out, int64_t out_row_stride, const void* pool,
                   const int* block_tables, int bt_stride, const int* cu_seqlens, const int* context_lens,
                   const int* tiles, int num_tiles, int nh, int nkv, int gp, int page_size, float scale, int window,
                   cudaStream_t stream) {
  const size_t smem = (size_t)(PF_ROWS + 4 * PF_KEYS) * HD * sizeof(bf16);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_attn_prefill: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  dim3 grid(num_tiles, nkv * (nh / nkv / gp));
  me_launch(attn_prefill_mma_kernel<HD>, grid, dim3(PF_THREADS), smem, stream,
      (const bf16*)qkv, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)pool, block_tables, bt_stride, cu_seqlens,
      context_lens, tiles, nh, nkv, gp, page_size, scale * 1.4426950408889634f, window);
  return 0;
}

}  // namespace

// Whether the tensor-core kernel takes this shape; if so, how many heads of a group share a block.
ME_API int me_attn_prefill_heads_per_block(int nh, int nkv, int hd) {
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv) return 0;
  const int G = nh / nkv;
  for (int gp = 8; gp >= 1; gp >>= 1)
    if (G % gp == 0) return gp;
  return 1;
}

// ``tiles``: (request, first local query) per block, each covering 64 / heads_per_block query tokens.
ME_API int me_attn_prefill(const void* qkv, int64_t q_row_stride, void* out, int64_t out_row_stride,
                           const void* pool, const int* block_tables, int bt_stride, const int* cu_seqlens,
                           const int* context_lens, const int* tiles, int num_tiles, int nh, int nkv, int hd,
                           int page_size, float scale, int window, cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  const int gp = me_attn_prefill_heads_per_block(nh, nkv, hd);
  ME_REQUIRE(gp > 0, "me_attn_prefill: head_dim %d with %d/%d heads is not taken by the tensor-core kernel", hd, nh, nkv);
  ME_REQUIRE((q_row_stride * 2) % 16 == 0 && (out_row_stride * 2) % 4 == 0, "me_attn_prefill: rows must be 16-byte aligned");
  ME_REQUIRE((int64_t)nkv * (nh / nkv / gp) <= 65535, "me_attn_prefill: too many heads");
  int rc;
  if (hd == 64)
    rc = launch_prefill<64>(qkv, q_row_stride, out, out_row_stride, pool, block_tables, bt_stride, cu_seqlens,
                            context_lens, tiles, num_tiles, nh, nkv, gp, page_size, scale, window, stream);
  else
    rc = launch_prefill<128>(qkv, q_row_stride, out, out_row_stride, pool, block_tables, bt_stride, cu_seqlens,
                             context_lens, tiles, num_tiles, nh, nkv, gp, page_size, scale, window, stream);
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_attn_prefill");
  return 0;
}
