// Paged attention for requests that bring one token: split over the keys, then merged.
//
// Reference (csrc/paged_decode.cu:247-334): the context is cut into partitions of 256 keys (128 here) at
// fixed absolute positions; a block handles one request, one key/value head and one
// partition, all query heads of the group sharing every K/V load; it writes an un-normalised
// output with its maximum and exponential sum, and a second kernel merges the partitions
// (M = max m_p, l = sum e^(m_p-M) l_p, o = sum e^(m_p-M) o_p, out = o / l).
//
// Here 8 lanes share a key (each holds 8-element pieces of the head), 16 keys are in flight
// per block, every 8-lane group keeps an online softmax of its own over the keys
// j = first + group + 16 i, and the groups are merged in index order, so the result depends
// only on the request's own keys.  Any head size that is a multiple of 8 up to 256, any
// group size, any page size, optional window (keys j > position - window).
#include "common.cuh"
#include "mma_prims.cuh"
#include "tma.cuh"

constexpr int DEC_PART = 128, DEC_THREADS = 128, DEC_LANES = 8, DEC_GROUPS = DEC_THREADS / DEC_LANES;

template <typename T> struct Vec8;
template <> struct Vec8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&x)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
};

// GT query heads per block, CH 8-element pieces per lane (head_dim <= 64 * CH).
template <typename T, int GT, int CH>
__global__ void __launch_bounds__(DEC_THREADS)
decode_partition_kernel(const T* __restrict__ qkv, int64_t q_row_stride, const T* __restrict__ pool,
                        const int* __restrict__ block_tables, int bt_stride,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                        int nh, int nkv, int hd, int page_size, float scale, int window,
                        float* __restrict__ tmp_out, float* __restrict__ tmp_m,
                        float* __restrict__ tmp_l, int max_parts) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int G = nh / nkv, head_tiles = (G + GT - 1) / GT;
  const int b = blockIdx.x, kvh = blockIdx.y / head_tiles, g0 = (blockIdx.y % head_tiles) * GT;
  const int z = blockIdx.z;
  const int L = context_lens[b];
  const int tid = threadIdx.x, kg = tid / DEC_LANES, lg = tid % DEC_LANES;
  const int n_g = min(GT, G - g0);
  const int lo_w = window > 0 ? max(0, L - window) : 0;
  const int part_lo = z * DEC_PART, part_hi = min(L, part_lo + DEC_PART);
  const int64_t slot0 = ((int64_t)b * nh + kvh * G + g0) * max_parts + z;   // + g * max_parts per head

  if (part_hi <= part_lo || part_hi <= lo_w) {        // nothing of this request in the partition
    if (part_lo < L || z == 0)
      for (int g = tid; g < n_g; g += DEC_THREADS) {
        tmp_m[slot0 + (int64_t)g * max_parts] = -INFINITY;
        tmp_l[slot0 + (int64_t)g * max_parts] = 0.f;
      }
    return;
  }
  float* q_s = smem;                                   // [GT][hd], scaled
  float* s_m = q_s + GT * hd;                          // [DEC_GROUPS][GT]
  float* s_l = s_m + DEC_GROUPS * GT;                  // [DEC_GROUPS][GT]
  float* s_acc = s_l + DEC_GROUPS * GT;                // [DEC_GROUPS][GT][hd]
  const int64_t tok = cu_seqlens[b];
  for (int idx = tid; idx < GT * hd; idx += DEC_THREADS) {
    const int g = idx / hd, d = idx - g * hd;
    q_s[idx] = g < n_g ? to_f<T>(qkv[tok * q_row_stride + (int64_t)(kvh * G + g0 + g) * hd + d]) * scale : 0.f;
  }
  __syncthreads();

  float m[GT], l[GT], acc[GT][CH][8];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int u = 0; u < CH; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][u][e] = 0.f;
  }
  const int* bt = block_tables + (int64_t)b * bt_stride;
  // The 8 lanes of a key group run the key loop together; other groups of the warp may not.
  const unsigned gmask = 0xFFu << ((tid & 31) & ~7);
  const int64_t v_off = (int64_t)nkv * page_size * hd;
  for (int j = part_lo + kg; j < part_hi; j += DEC_GROUPS) {
    if (j < lo_w) continue;
    const int page = bt[j / page_size];
    if (page < 0) continue;                            // given back: behind every window
    const T* kp = pool + (((int64_t)page * 2) * nkv + kvh) * page_size * hd + (int64_t)(j % page_size) * hd;
    float kx[CH][8], vx[CH][8];
#pragma unroll
    for (int u = 0; u < CH; ++u) {
      const int d0 = (lg + DEC_LANES * u) * 8;
      if (d0 < hd) {
        Vec8<T>::load(kp + d0, kx[u]);
        Vec8<T>::load(kp + v_off + d0, vx[u]);
      }
    }
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float dot = 0.f;
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const int d0 = (lg + DEC_LANES * u) * 8;
        if (d0 < hd) {
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(q_s[g * hd + d0 + e], kx[u][e], dot);
        }
      }
#pragma unroll
      for (int o = 1; o < DEC_LANES; o <<= 1) dot += __shfl_xor_sync(gmask, dot, o);
      const float m_new = fmaxf(m[g], dot);
      const float alpha = expf(m[g] - m_new), p = expf(dot - m_new);
      l[g] = l[g] * alpha + p;
      m[g] = m_new;
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const int d0 = (lg + DEC_LANES * u) * 8;
        if (d0 < hd) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[g][u][e] = fmaf(p, vx[u][e], acc[g][u][e] * alpha);
        }
      }
    }
  }
  // Merge the 16 key groups in index order.
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (lg == 0) {
      s_m[kg * GT + g] = m[g];
      s_l[kg * GT + g] = l[g];
    }
#pragma unroll
    for (int u = 0; u < CH; ++u) {
      const int d0 = (lg + DEC_LANES * u) * 8;
      if (d0 < hd) {
#pragma unroll
        for (int e = 0; e < 8; ++e) s_acc[((int64_t)kg * GT + g) * hd + d0 + e] = acc[g][u][e];
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < n_g * hd; idx += DEC_THREADS) {
    const int g = idx / hd, d = idx - g * hd;
    float M = -INFINITY;
    for (int k = 0; k < DEC_GROUPS; ++k) M = fmaxf(M, s_m[k * GT + g]);
    float lt = 0.f, o = 0.f;
    if (M > -INFINITY) {
      for (int k = 0; k < DEC_GROUPS; ++k) {
        const float mk = s_m[k * GT + g];
        const float f = mk == -INFINITY ? 0.f : expf(mk - M);
        lt += f * s_l[k * GT + g];
        o += f * s_acc[((int64_t)k * GT + g) * hd + d];
      }
    }
    const int64_t slot = slot0 + (int64_t)g * max_parts;
    tmp_out[slot * hd + d] = o;
    if (d == 0) {
      tmp_m[slot] = M;
      tmp_l[slot] = lt;
    }
  }
}

// The end of a partition step on the tensor cores: the four warps' (m, l, O) for the rows that are real heads, merged in
// warp order and written as the partition's result.  The results [4][16][HD] float32 go over the K tile ``po`` (every warp
// is done with it), the 8-float pieces of row r at piece ^ (r & 7): the eight rows that a warp's store touches then lie in
// different banks (unswizzled, rows 512 bytes apart, they shared them all).  The weight of warp w's share of row r,
// exp2((m_w - M) scale) with M the row's maximum over the warps, is computed once per (w, r), not once per element.
template <int HD>
__device__ __forceinline__ void merge_warps_of_partition(float* po, float (*w_m)[16], float (*w_l)[16], float (*w_f)[16],
                                                         float (*w_fl)[16], const float (&o)[HD / 8][4], float mx0, float l0,
                                                         float mx1, float l1, int n_g, float sl2, float scale,
                                                         float* __restrict__ tmp_out, float* __restrict__ tmp_m,
                                                         float* __restrict__ tmp_l, int64_t slot0, int max_parts) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  auto po_at = [&](int w, int r, int d) -> float* { return po + (w * 16 + r) * HD + ((((d >> 3) ^ (r & 7)) << 3) | (d & 7)); };
  if (t4 == 0) {
    w_m[warp][g] = mx0;
    w_l[warp][g] = l0;
    w_m[warp][g + 8] = mx1;
    w_l[warp][g + 8] = l1;
  }
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    if (g < n_g) *reinterpret_cast<float2*>(po_at(warp, g, i * 8 + 2 * t4)) = make_float2(o[i][0], o[i][1]);
    if (g + 8 < n_g) *reinterpret_cast<float2*>(po_at(warp, g + 8, i * 8 + 2 * t4)) = make_float2(o[i][2], o[i][3]);
  }
  __syncthreads();
  if (tid < 64) {
    const int w = tid >> 4, r = tid & 15;
    const float M = fmaxf(fmaxf(w_m[0][r], w_m[1][r]), fmaxf(w_m[2][r], w_m[3][r]));
    const float mw = w_m[w][r];
    const float f = (M == -INFINITY || mw == -INFINITY) ? 0.f : exp2f((mw - M) * sl2);
    w_f[w][r] = f;
    w_fl[w][r] = f * w_l[w][r];
    if (w == 0 && r < n_g) tmp_m[slot0 + (int64_t)r * max_parts] = M == -INFINITY ? -INFINITY : M * scale;   // natural-log units, as the merge kernel expects
  }
  __syncthreads();
  if (tid < n_g) tmp_l[slot0 + (int64_t)tid * max_parts] = ((w_fl[0][tid] + w_fl[1][tid]) + w_fl[2][tid]) + w_fl[3][tid];
  for (int idx = tid; idx < n_g * (HD / 4); idx += DEC_THREADS) {
    const int r = idx / (HD / 4), d = (idx - r * (HD / 4)) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = w_f[w][r];
      const float4 v = *reinterpret_cast<const float4*>(po_at(w, r, d));
      acc.x += f * v.x;
      acc.y += f * v.y;
      acc.z += f * v.z;
      acc.w += f * v.w;
    }
    *reinterpret_cast<float4*>(tmp_out + (slot0 + (int64_t)r * max_parts) * HD + d) = acc;
  }
}

// ---- the partition step on the tensor cores -----------------------------------------------------
// The query heads of one key/value head (up to 16) form the rows of an m16 strip; each of the four
// warps takes 32 keys of the 128-key partition: S = Q K^T and O = P V with mma.sync m16n8k16, softmax
// in float32 on the accumulator fragments, then the four warps' (m, l, O) are merged in index order.
// K and V arrive by cp.async (zero fill outside the request's keys) in two groups, so the scores are
// computed while V is still on its way.  bfloat16, head_dim 64 or 128, any page size.
template <int HD>
__global__ void __launch_bounds__(DEC_THREADS)
decode_partition_mma_kernel(const bf16* __restrict__ qkv, int64_t q_row_stride, const bf16* __restrict__ pool,
                            const int* __restrict__ block_tables, int bt_stride,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                            int nh, int nkv, int page_size, float scale, int window,
                            float* __restrict__ tmp_out, float* __restrict__ tmp_m,
                            float* __restrict__ tmp_l, int max_parts) {
  using namespace mma_prims;
  extern __shared__ __align__(128) unsigned char dec_smem[];
  __shared__ float w_m[4][16], w_l[4][16], w_f[4][16], w_fl[4][16];
  constexpr int PIECES = HD / 8, KSTEPS = HD / 16, NT_O = HD / 8;
  const int G = nh / nkv, head_tiles = (G + 15) / 16;
  const int b = blockIdx.x, kvh = blockIdx.y / head_tiles, g0 = (blockIdx.y % head_tiles) * 16;
  const int z = blockIdx.z;
  const int L = context_lens[b];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, t4 = lane & 3;
  const int n_g = min(16, G - g0);
  const int lo_w = window > 0 ? max(0, L - window) : 0;
  const int part_lo = z * DEC_PART, part_hi = min(L, part_lo + DEC_PART);
  const int64_t slot0 = ((int64_t)b * nh + kvh * G + g0) * max_parts + z;
  if (part_hi <= part_lo || part_hi <= lo_w) {
    pdl_wait();
    pdl_launch_dependents();
    if (part_lo < L || z == 0)
      for (int r = tid; r < n_g; r += DEC_THREADS) {
        tmp_m[slot0 + (int64_t)r * max_parts] = -INFINITY;
        tmp_l[slot0 + (int64_t)r * max_parts] = 0.f;
      }
    return;
  }
  bf16* qs = reinterpret_cast<bf16*>(dec_smem);     // [16][HD]
  bf16* ks = qs + 16 * HD;                           // [128][HD]; later the warps' partial outputs
  bf16* vs = ks + DEC_PART * HD;                     // [128][HD]
  const int* bt = block_tables + (int64_t)b * bt_stride;
  const int64_t tok = cu_seqlens[b];
  // Only the partition that holds the request's newest key depends on the kernel before this one (which
  // wrote that key); the others fetch their keys and values while that kernel is still running.
  const bool has_new = part_hi == L;
  // Thread t copies piece (t % PIECES) of rows (t / PIECES) + k * (128 / PIECES); the rows' places in the
  // pool are looked up once and serve both K (first group) and V (second group).
  const int64_t v_off = (int64_t)nkv * page_size * HD;
  const PageMap pm{bt, page_size, log2_if_pow2(page_size), 2 * v_off, (int64_t)kvh * page_size * HD, HD};
  constexpr int ROWS_PER_PASS = DEC_THREADS / PIECES, PASSES = DEC_PART / ROWS_PER_PASS;
  const int piece = tid % PIECES, r0 = tid / PIECES;
  int64_t base[PASSES];
#pragma unroll
  for (int k = 0; k < PASSES; ++k) {
    const int j = part_lo + r0 + k * ROWS_PER_PASS;
    base[k] = (j < part_hi && j >= lo_w) ? pm.row(j) : -1;
  }
  if (has_new) {
    pdl_wait();
    pdl_launch_dependents();
  }
#pragma unroll
  for (int k = 0; k < PASSES; ++k)
    cp_async16(tile_ptr<HD>(ks, r0 + k * ROWS_PER_PASS, piece), base[k] >= 0 ? pool + base[k] + piece * 8 : pool, base[k] >= 0);
  cp_async_commit();
#pragma unroll
  for (int k = 0; k < PASSES; ++k)
    cp_async16(tile_ptr<HD>(vs, r0 + k * ROWS_PER_PASS, piece), base[k] >= 0 ? pool + base[k] + v_off + piece * 8 : pool,
               base[k] >= 0);
  cp_async_commit();
  if (!has_new) {
    pdl_wait();
    pdl_launch_dependents();
  }
  for (int c = tid; c < 16 * PIECES; c += DEC_THREADS) {       // q is written by the kernel before this one
    const int row = c / PIECES, piece = c % PIECES;
    const bool ok = row < n_g;
    cp_async16(tile_ptr<HD>(qs, row, piece),
               ok ? qkv + tok * q_row_stride + (int64_t)(kvh * G + g0 + row) * HD + piece * 8 : qkv, ok);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  const float sl2 = scale * 1.4426950408889634f;
  const int mi = lane >> 3;
  float s[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
    uint32_t qf[4];
    ldmatrix_x4(qf, tile_ptr<HD>(qs, (mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1)));
#pragma unroll
    for (int np = 0; np < 2; ++np) {
      uint32_t bfr[4];
      ldmatrix_x4(bfr, tile_ptr<HD>(ks, warp * 32 + np * 16 + (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
      mma_bf16(s[2 * np], qf, bfr[0], bfr[1]);
      mma_bf16(s[2 * np + 1], qf, bfr[2], bfr[3]);
    }
  }
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int j = part_lo + warp * 32 + i * 8 + 2 * t4 + e;
      if (j >= part_hi || j < lo_w) s[i][e] = s[i][e + 2] = -INFINITY;
    }
    mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
    mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mu0 = mx0 == -INFINITY ? 0.f : mx0, mu1 = mx1 == -INFINITY ? 0.f : mx1;
  float l0 = 0.f, l1 = 0.f;
  uint32_t pf[2][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float p0 = exp2f((s[i][0] - mu0) * sl2), p1 = exp2f((s[i][1] - mu0) * sl2);
    const float p2 = exp2f((s[i][2] - mu1) * sl2), p3 = exp2f((s[i][3] - mu1) * sl2);
    l0 += p0 + p1;
    l1 += p2 + p3;
    pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
    pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();                                   // every warp is done reading K
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
    for (int np = 0; np < NT_O / 2; ++np) {
      uint32_t bfr[4];
      ldmatrix_x4_trans(bfr, tile_ptr<HD>(vs, warp * 32 + kk * 16 + (mi & 1) * 8 + (lane & 7), np * 2 + (mi >> 1)));
      mma_bf16(o[2 * np], pf[kk], bfr[0], bfr[1]);
      mma_bf16(o[2 * np + 1], pf[kk], bfr[2], bfr[3]);
    }
  }
  merge_warps_of_partition<HD>(reinterpret_cast<float*>(ks), w_m, w_l, w_f, w_fl, o, mx0, l0, mx1, l1, n_g, sl2, scale, tmp_out,
                               tmp_m, tmp_l, slot0, max_parts);
}

template <int HD>
static int launch_partition_mma(int num_reqs, int max_parts, cudaStream_t stream, const void* qkv, int64_t q_row_stride,
                                const void* pool, const int* bt, int bt_stride, const int* cu, const int* cl, int nh,
                                int nkv, int page_size, float scale, int window, float* to, float* tm, float* tl) {
  const size_t smem = (size_t)(16 + 2 * DEC_PART) * HD * sizeof(bf16);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(decode_partition_mma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_attn_decode: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  const int G = nh / nkv;
  dim3 grid(num_reqs, nkv * ((G + 15) / 16), max_parts);
  me_launch(decode_partition_mma_kernel<HD>, grid, dim3(DEC_THREADS), smem, stream,
      (const bf16*)qkv, q_row_stride, (const bf16*)pool, bt, bt_stride, cu, cl, nh, nkv, page_size, scale, window, to, tm, tl,
      max_parts);
  return 0;
}

// ---- the tensor-core partition step fed by tensor-map loads ------------------------------------------
// As above, but K and V come by TMA: the pool of one cache slot is a 2-D tensor [pages * 2 * kv_heads *
// page_size][head_dim]; a box is one page of one head, 64 columns wide, written with the 128-byte swizzle
// that ldmatrix wants.  One thread issues every box of the partition (K on one mbarrier, V on another),
// so the block has its 64 KB in flight as a few dozen requests instead of four thousand 16-byte copies.
// Rows of V that are not keys of the request (a page's tail, keys behind the window) are zeroed before
// P V, because 0 * (whatever the page holds there) must be 0.  Page sizes that divide 128.
// RMSNorm over one head and the rotary embedding, exactly as csrc/qk_rope_kv.cu does them for a whole step
// (models/qwen3.py:34-36 and layers/rotary_embedding.py:20-25 in the reference): one warp per head, lane l owns
// HD/64 consecutive elements of each half.  The lane's norm weights (wa, wb) and its cosines and sines of the
// token's position were read ahead; ``norm`` / ``rope`` say which of the two steps exist.
template <int HD>
__device__ __forceinline__ void norm_rope_head(const bf16* __restrict__ x, bool norm, const float (&wa)[HD / 64],
                                               const float (&wb)[HD / 64], float eps, bool rope, const float (&c)[HD / 64],
                                               const float (&sn)[HD / 64], int lane, bf16 (&ra)[HD / 64], bf16 (&rb)[HD / 64]) {
  constexpr int VEC = HD / 64, half = HD / 2;
  const int i0 = lane * VEC;
  float a[VEC], b[VEC], ss = 0.f;
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    a[j] = __bfloat162float(x[i0 + j]);
    b[j] = __bfloat162float(x[half + i0 + j]);
    ss += a[j] * a[j] + b[j] * b[j];
  }
  float inv = 1.f;
  if (norm) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)HD + eps);
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    float y1 = a[j], y2 = b[j];
    if (norm) {
      y1 = (y1 * inv) * wa[j];
      y2 = (y2 * inv) * wb[j];
    }
    float o1 = y1, o2 = y2;
    if (rope) {
      o1 = y1 * c[j] - y2 * sn[j];
      o2 = y2 * c[j] + y1 * sn[j];
    }
    ra[j] = __float2bfloat16_rn(o1);
    rb[j] = __float2bfloat16_rn(o2);
  }
}

// What the kernel needs to prepare q and the newest key and value itself (FUSED): then no kernel runs between
// the q|k|v product and this one, and no block's loads depend on the kernel before it.
struct DecodePrep {
  const float* qw;            // q and k norm weights [HD] (both null: no norm)
  const float* kw;
  float eps;
  const float* cos_sin;       // rotary table [positions][HD] (cos | sin) or null; the token's position is context - 1
  const int* slot_mapping;    // [tokens] cache slot of the token's key and value; null: another layer wrote them
  bf16* pool;                 // the cache slot, [page][k|v][kv_head][offset][HD]
};

// The two products are mma.sync m16n8k16 with ldmatrix.
// VBUF says how much shared memory V has of its own: 2 a whole tile (three blocks an SM); 0
// none: V passes through K's tile, requested once every warp has its scores (six blocks an SM with an 8-row Q tile:
// a block lives one load longer, but more of them are loading at any time: large batches); 1 half a tile: the
// first 64 keys' values come with K, the other 64 pass through K's tile (four blocks an SM: a batch of 8 at 1,000
// tokens then fits the GPU in one wave with most of its loads in flight before the dependency resolves).
// With at most 8 query heads a group the Q tile keeps 8 rows (the upper half of the m16 strip reads one chunk of
// zeros), and with VBUF 0 the registers are held to what lets six blocks share an SM.
// TILED: a block walks ``tiles`` tiles of 128 keys, one after the other with a running softmax (else one: what the
// loop carries, the output's 64 registers above all, would not fit the registers of six blocks an SM; four share it then).
template <int HD, bool FUSED, int VBUF, int QROWS, bool TILED>
__global__ void __launch_bounds__(DEC_THREADS, (VBUF == 0 && QROWS == 8) ? (TILED ? 4 : 6) : 1)
decode_partition_tma_mma_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ qkv,
                                int64_t q_row_stride, const int* __restrict__ block_tables, int bt_stride,
                                const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                                int nh, int nkv, int page_size, float scale, int window,
                                float* __restrict__ tmp_out, float* __restrict__ tmp_m,
                                float* __restrict__ tmp_l, int max_parts, int tiles, int* __restrict__ err, DecodePrep prep) {
  using namespace mma_prims;
  extern __shared__ unsigned char dec_smem_raw[];
  __shared__ float w_m[4][16], w_l[4][16], w_f[4][16], w_fl[4][16];
  __shared__ __align__(8) unsigned long long bar_k, bar_v, bar_v2;
  __shared__ __align__(16) bf16 zero_chunk[8];
  constexpr int PIECES = HD / 8, KSTEPS = HD / 16, NT_O = HD / 8, HALVES = HD / 64;
  const int G = nh / nkv, head_tiles = (G + 15) / 16;
  const int b = blockIdx.x, kvh = blockIdx.y / head_tiles, g0 = (blockIdx.y % head_tiles) * 16;
  const int z = blockIdx.z;
  const int L = context_lens[b];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, t4 = lane & 3;
  const int n_g = min(16, G - g0);
  // The page of this lane's piece of the partition is asked for together with the context length (which page it
  // is depends on the partition alone; whether it holds keys of the request is decided afterwards): one
  // round trip to memory before the loads can be issued, not two.
  const int part_keys = (TILED ? tiles : 1) * DEC_PART;      // keys of a block: tiles of 128, walked one after the other
  const int n_pages = DEC_PART / page_size;
  auto page_of = [&](int tile_lo_) -> int {          // warp 0, lane < n_pages: the page of this lane's piece of a tile
    const int pi = tile_lo_ / page_size + lane;
    return pi < bt_stride ? block_tables[(int64_t)b * bt_stride + pi] : -1;
  };
  int page_ahead = -1;
  if (warp == 0 && lane < n_pages) page_ahead = page_of(z * part_keys);
  const int lo_w = window > 0 ? max(0, L - window) : 0;
  const int part_lo = z * part_keys, part_hi = min(L, part_lo + part_keys);
  const int64_t slot0 = ((int64_t)b * nh + kvh * G + g0) * max_parts + z;
  if (part_hi <= part_lo || part_hi <= lo_w) {
    pdl_wait();
    pdl_launch_dependents();
    if (part_lo < L || z == 0)
      for (int r = tid; r < n_g; r += DEC_THREADS) {
        tmp_m[slot0 + (int64_t)r * max_parts] = -INFINITY;
        tmp_l[slot0 + (int64_t)r * max_parts] = 0.f;
      }
    return;
  }
  // Shared memory from a 1024-byte boundary: K halves [HALVES][128][64], V halves, then Q [16][HD].
  unsigned char* aligned = dec_smem_raw + ((1024u - (tma::smem_addr(dec_smem_raw) & 1023u)) & 1023u);
  bf16* ks = reinterpret_cast<bf16*>(aligned);
  constexpr int HALF = DEC_PART / 2;
  bf16* vs = VBUF == 0 ? ks : ks + DEC_PART * HD;      // VBUF 1: the values of keys 0..63; those of 64..127 go to ks
  bf16* qs = vs + (VBUF == 2 ? DEC_PART : (VBUF == 1 ? HALF : 0)) * HD + (VBUF == 0 ? DEC_PART * HD : 0);
  // Row ``row`` (a key of the partition), 16-byte piece ``piece`` of the V tile(s)
  auto v_at = [&](int row, int piece) -> bf16* {
    if (VBUF == 1) {
      const int hi_half = row >= HALF;
      return tma::swz128((hi_half ? ks : vs) + (piece >> 3) * HALF * 64, row - hi_half * HALF, piece & 7);
    }
    return tma::swz128(vs + (piece >> 3) * DEC_PART * 64, row, piece & 7);
  };
  // Element i of row ``row`` of the Q tile: a [16][HD] tile with XOR-swizzled pieces.
  auto q_at = [&](int row, int i) -> bf16* { return tile_ptr<HD>(qs, row, i >> 3) + (i & 7); };
  const int64_t tok = cu_seqlens[b];
  // Only the partition that holds the request's newest key depends on the kernel before this one (which
  // wrote that key); the others fetch their keys and values while that kernel is still running.  A block
  // that makes the newest key and value itself (FUSED) loads the slot's old content and replaces it in
  // shared memory, so it does not wait either.
  const bool has_new = part_hi == L;
  const bool makes_new = FUSED && has_new && prep.slot_mapping != nullptr;
  const bool wait_first = has_new && !makes_new;
  // the tiles of the partition that hold keys the request sees: [t_first, n_tiles)
  const int t_first = (TILED && lo_w > part_lo) ? (lo_w - part_lo) / DEC_PART : 0;
  const int n_tiles = TILED ? (part_hi - part_lo + DEC_PART - 1) / DEC_PART : 1;
  int tile_lo = part_lo + t_first * DEC_PART, tile_hi = min(part_hi, tile_lo + DEC_PART);
  if (t_first > 0 && warp == 0 && lane < n_pages) page_ahead = page_of(tile_lo);
  if (wait_first) {
    pdl_wait();
    pdl_launch_dependents();
  }
  if (tid < 8) zero_chunk[tid] = __float2bfloat16_rn(0.f);
  if (tid == 0) {
    tma::mbar_init(&bar_k, 1);
    tma::mbar_init(&bar_v, 1);
    tma::mbar_init(&bar_v2, 1);
    tma::mbar_fence_init();
  }
  // A tensor-map copy is issued per thread, so the lanes of one warp issue the partition's boxes together: lane i
  // looks up page i, lane 0 announces the bytes, then box x = ((k|v) * HALVES + half) * pages + page goes out from
  // lane x % 32.
  int first_row = -1;                                  // warp 0: row of the pool's 2-D view where this lane's page keeps K
  auto rows_of_tile = [&]() {
    first_row = -1;
    if (warp == 0 && lane < n_pages) {
      const int j0 = tile_lo + lane * page_size;
      const int page = (j0 < tile_hi && j0 + page_size > lo_w) ? page_ahead : -1;
      if (page >= 0) first_row = ((page * 2) * nkv + kvh) * page_size;
    }
  };
  rows_of_tile();
  // what: bit 0 K, bit 1 the values of the partition's first half of pages, bit 2 those of the second half
  auto request = [&](int what) {                       // warp 0
    const unsigned box_bytes = (unsigned)page_size * 64 * sizeof(bf16);
    const unsigned present = __ballot_sync(0xffffffffu, first_row >= 0);
    const unsigned lo_pages = (1u << (n_pages / 2)) - 1u;
    if (lane == 0) {
      if (what & 1) tma::mbar_expect_tx(&bar_k, (unsigned)__popc(present) * HALVES * box_bytes);
      if (VBUF == 1) {
        if (what & 2) tma::mbar_expect_tx(&bar_v, (unsigned)__popc(present & lo_pages) * HALVES * box_bytes);
        if (what & 4) tma::mbar_expect_tx(&bar_v2, (unsigned)__popc(present & ~lo_pages) * HALVES * box_bytes);
      } else if (what & 6) {
        tma::mbar_expect_tx(&bar_v, (unsigned)__popc(present) * HALVES * box_bytes);
      }
    }
    __syncwarp();
    const int v_rows = nkv * page_size;
    for (int x0 = 0; x0 < 2 * HALVES * n_pages; x0 += 32) {
      const int x = x0 + lane;
      const int i = x % n_pages, h = (x / n_pages) % HALVES, v = x / (n_pages * HALVES);
      const int row = __shfl_sync(0xffffffffu, first_row, i);
      if (x >= 2 * HALVES * n_pages || row < 0) continue;
      if (!v) {
        if (what & 1) tma::load_2d(ks + h * DEC_PART * 64 + i * page_size * 64, &kv_map, h * 64, row, &bar_k);
      } else if (VBUF == 1) {
        const bool second = i >= n_pages / 2;
        if (what & (second ? 4 : 2))
          tma::load_2d((second ? ks : vs) + h * HALF * 64 + (i - (second ? n_pages / 2 : 0)) * page_size * 64, &kv_map, h * 64,
                       row + v_rows, second ? &bar_v2 : &bar_v);
      } else if (what & 6) {
        tma::load_2d(vs + h * DEC_PART * 64 + i * page_size * 64, &kv_map, h * 64, row + v_rows, &bar_v);
      }
    }
  };
  if (warp == 0) request(VBUF == 2 ? 7 : (VBUF == 1 ? 3 : 1));
  constexpr int VEC = HD / 64;
  // what the preparation of q and of the newest key needs besides the rows themselves is no kernel's output:
  // read it while the kernel before this one is still running
  float qwa[VEC], qwb[VEC], kwa[VEC], kwb[VEC], rc[VEC], rs[VEC];
  const bool norm = FUSED && prep.qw != nullptr, rope = FUSED && prep.cos_sin != nullptr;
  if (FUSED) {
    const float* cs = rope ? prep.cos_sin + (int64_t)(L - 1) * HD : nullptr;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int i = lane * VEC + j;
      qwa[j] = norm ? prep.qw[i] : 1.f;
      qwb[j] = norm ? prep.qw[HD / 2 + i] : 1.f;
      kwa[j] = norm ? prep.kw[i] : 1.f;
      kwb[j] = norm ? prep.kw[HD / 2 + i] : 1.f;
      rc[j] = rope ? cs[i] : 1.f;
      rs[j] = rope ? cs[HD / 2 + i] : 0.f;
    }
  }
  // (the slot of the newest key and value is the host's data as well)
  const int new_slot = makes_new ? prep.slot_mapping[tok] : -1;
  if (!wait_first) {
    pdl_wait();
    pdl_launch_dependents();
  }
  bf16 new_a[VEC], new_b[VEC];                       // warp 0: the newest key; warp 1: the newest value (makes_new)
  if (FUSED) {
    // q as the product before left it: norm and rotation here, one warp per head, into the swizzled tile
    for (int row = warp; row < QROWS; row += 4) {
      bf16 ra[VEC], rb[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) ra[j] = rb[j] = __float2bfloat16_rn(0.f);
      if (row < n_g)
        norm_rope_head<HD>(qkv + tok * q_row_stride + (int64_t)(kvh * G + g0 + row) * HD, norm, qwa, qwb, prep.eps, rope, rc, rs,
                           lane, ra, rb);
      const int i0 = lane * VEC;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        *q_at(row, i0 + j) = ra[j];
        *q_at(row, HD / 2 + i0 + j) = rb[j];
      }
    }
    if (makes_new) {
      if (warp == 0) {
        norm_rope_head<HD>(qkv + tok * q_row_stride + (int64_t)(nh + kvh) * HD, norm, kwa, kwb, prep.eps, rope, rc, rs, lane,
                           new_a, new_b);
      } else if (warp == 1) {
        const bf16* v = qkv + tok * q_row_stride + (int64_t)(nh + nkv + kvh) * HD;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          new_a[j] = v[lane * VEC + j];
          new_b[j] = v[HD / 2 + lane * VEC + j];
        }
      }
    }
  } else {
    for (int c = tid; c < QROWS * PIECES; c += DEC_THREADS) {  // q is written by the kernel before this one
      const int row = c / PIECES, piece = c % PIECES;
      const bool ok = row < n_g;
      cp_async16(q_at(row, piece * 8),
                 ok ? qkv + tok * q_row_stride + (int64_t)(kvh * G + g0 + row) * HD + piece * 8 : qkv, ok);
    }
    cp_async_commit();
    cp_async_wait<0>();
  }
  __syncthreads();                                   // barriers initialised, Q in place
  // The newest key and value go to their row of the tiles (over whatever the slot held) and to the cache.
  auto put_new = [&](bf16* tile, int kv) {
    const int row = L - 1 - tile_lo, i0 = lane * VEC;
    const int slot = new_slot;
    bf16* dst = nullptr;
    if (slot >= 0 && g0 == 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      dst = prep.pool + ((((int64_t)page * 2 + kv) * nkv + kvh) * page_size + off) * HD;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const int ia = i0 + j, ib = HD / 2 + i0 + j;
      (kv ? v_at(row, ia >> 3) : tma::swz128(tile + (ia >> 6) * DEC_PART * 64, row, (ia & 63) >> 3))[ia & 7] = new_a[j];
      (kv ? v_at(row, ib >> 3) : tma::swz128(tile + (ib >> 6) * DEC_PART * 64, row, (ib & 63) >> 3))[ib & 7] = new_b[j];
      if (dst) {
        dst[ia] = new_a[j];
        dst[ib] = new_b[j];
      }
    }
  };
  const float sl2 = scale * 1.4426950408889634f;
  const int mi = lane >> 3;
  // Each warp keeps the running maximum, sum and output of its 32 keys of every tile (rows g and g + 8 of the strip);
  // the sums stay per thread until the end (the factor a new maximum brings is the same for the four threads of a row).
  float mx0 = -INFINITY, mx1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  bool landed = true;
  for (int t = t_first; t < n_tiles; ++t) {
    const int phase = (t - t_first) & 1;
    const bool newest_here = makes_new && tile_hi == L;
    if (t > t_first) {
      // the tile before is read by every warp (the barrier at its end): its place takes this tile's keys
      rows_of_tile();
      if (warp == 0) {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // (rows of the tile were written by threads)
        request(VBUF == 2 ? 7 : (VBUF == 1 ? 3 : 1));
      }
    }
    // the pages of the tile after this one: asked for now, needed at the end of this tile
    int page_next = -1;
    if (t + 1 < n_tiles && warp == 0 && lane < n_pages) page_next = page_of(tile_lo + DEC_PART);
    landed = tma::mbar_wait(&bar_k, phase) && landed;
    if (newest_here) {
      if (warp == 0) put_new(ks, 0);
      __syncthreads();                               // the row is in place before any warp reads K
    }
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t qf[4];
      ldmatrix_x4(qf, (QROWS == 8 && (mi & 1)) ? zero_chunk : tile_ptr<HD>(qs, (mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1)));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t bfr[4];
        const int piece = kk * 2 + (mi & 1);
        ldmatrix_x4(bfr, tma::swz128(ks + (piece >> 3) * DEC_PART * 64, warp * 32 + np * 16 + (mi >> 1) * 8 + (lane & 7), piece & 7));
        mma_bf16(s[2 * np], qf, bfr[0], bfr[1]);
        mma_bf16(s[2 * np + 1], qf, bfr[2], bfr[3]);
      }
    }
    if (VBUF < 2) {
      __syncthreads();                               // every warp has its scores: K's tile is free for V
      if (warp == 0) {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // (the newest key's row was written by threads)
        request(VBUF == 1 ? 4 : 6);
      }
    }
    float tm0 = -INFINITY, tm1 = -INFINITY;          // the tile's maxima
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = tile_lo + warp * 32 + i * 8 + 2 * t4 + e;
        if (j >= tile_hi || j < lo_w) s[i][e] = s[i][e + 2] = -INFINITY;
      }
      tm0 = fmaxf(tm0, fmaxf(s[i][0], s[i][1]));
      tm1 = fmaxf(tm1, fmaxf(s[i][2], s[i][3]));
    }
    tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
    tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
    tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
    tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
    const float nm0 = fmaxf(mx0, tm0), nm1 = fmaxf(mx1, tm1);
    const float mu0 = nm0 == -INFINITY ? 0.f : nm0, mu1 = nm1 == -INFINITY ? 0.f : nm1;
    if (t > t_first) {                               // what the tiles before left, at the new maximum (0 while there was none)
      const float a0 = exp2f((mx0 - mu0) * sl2), a1 = exp2f((mx1 - mu1) * sl2);
      l0 *= a0;
      l1 *= a1;
#pragma unroll
      for (int i = 0; i < NT_O; ++i) {
        o[i][0] *= a0;
        o[i][1] *= a0;
        o[i][2] *= a1;
        o[i][3] *= a1;
      }
    }
    mx0 = nm0;
    mx1 = nm1;
    uint32_t pf[2][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p0 = exp2f((s[i][0] - mu0) * sl2), p1 = exp2f((s[i][1] - mu0) * sl2);
      const float p2 = exp2f((s[i][2] - mu1) * sl2), p3 = exp2f((s[i][3] - mu1) * sl2);
      l0 += p0 + p1;
      l1 += p2 + p3;
      pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    landed = tma::mbar_wait(&bar_v, phase) && landed;
    if (VBUF == 1) landed = tma::mbar_wait(&bar_v2, phase) && landed;
    if (newest_here && warp == 1) put_new(vs, 1);
    {                                                // rows of V that are no keys of this request: zero
      const int j = tile_lo + tid;                   // 128 threads, 128 rows
      if (j >= tile_hi || j < lo_w)
        for (int p = 0; p < PIECES; ++p) *reinterpret_cast<uint4*>(v_at(tid, p)) = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();                                 // V complete and cleaned; every warp is done reading K
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        uint32_t bfr[4];
        const int piece = np * 2 + (mi >> 1);
        ldmatrix_x4_trans(bfr, v_at(warp * 32 + kk * 16 + (mi & 1) * 8 + (lane & 7), piece));
        mma_bf16(o[2 * np], pf[kk], bfr[0], bfr[1]);
        mma_bf16(o[2 * np + 1], pf[kk], bfr[2], bfr[3]);
      }
    }
    if (t + 1 < n_tiles) {
      __syncthreads();                               // every warp is done with this tile's V (and K)
      tile_lo += DEC_PART;
      tile_hi = min(part_hi, tile_lo + DEC_PART);
      page_ahead = page_next;
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (VBUF < 2) __syncthreads();                     // every warp is done reading V: K's tile now takes the warps' results
  if (!landed && tid == 0) atomicOr(err + 1, 1);     // a load did not land in time: the result is reported as invalid
  merge_warps_of_partition<HD>(reinterpret_cast<float*>(ks), w_m, w_l, w_f, w_fl, o, mx0, l0, mx1, l1, n_g, sl2, scale, tmp_out,
                               tmp_m, tmp_l, slot0, max_parts);
}

template <int HD, bool FUSED, int VBUF, int QROWS, bool TILED = false>
static int launch_partition_tma_mma(const void* kv_map, int num_reqs, int max_parts, cudaStream_t stream, const void* qkv,
                                    int64_t q_row_stride, const int* bt, int bt_stride, const int* cu, const int* cl, int nh,
                                    int nkv, int page_size, float scale, int window, float* to, float* tm, float* tl, int tiles,
                                    int* err, const DecodePrep& prep) {
  const size_t smem = (size_t)(QROWS + DEC_PART + VBUF * DEC_PART / 2) * HD * sizeof(bf16) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(decode_partition_tma_mma_kernel<HD, FUSED, VBUF, QROWS, TILED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "me_attn_decode: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  const int G = nh / nkv;
  dim3 grid(num_reqs, nkv * ((G + 15) / 16), max_parts);
  me_launch(decode_partition_tma_mma_kernel<HD, FUSED, VBUF, QROWS, TILED>, grid, dim3(DEC_THREADS), smem, stream,
      *reinterpret_cast<const CUtensorMap*>(kv_map), (const bf16*)qkv, q_row_stride, bt, bt_stride, cu, cl, nh, nkv, page_size,
      scale, window, to, tm, tl, max_parts, tiles, err, prep);
  return 0;
}

// One block per (request, head) adds the partitions' results.  Loads that do not depend on one another are
// issued together (a partition per thread for the maxima and sums, eight partitions at a time for the
// outputs): a loop of dependent loads would pay the L2 latency once per partition.
template <typename T>
__global__ void decode_merge_kernel(T* __restrict__ out, int64_t out_row_stride,
                                    const int* __restrict__ cu_seqlens,
                                    const int* __restrict__ context_lens,
                                    const float* __restrict__ tmp_out, const float* __restrict__ tmp_m,
                                    const float* __restrict__ tmp_l, int nh, int hd, int max_parts, int part_keys) {
  constexpr int CHUNK = 128;                         // partitions whose factors are held in shared memory at a time
  __shared__ float f_s[CHUNK], red[32];
  const int b = blockIdx.x, h = blockIdx.y;
  const int L = context_lens[b];                     // written by the host, not by a kernel of this step
  const int64_t tok = cu_seqlens[b];
  pdl_wait();
  pdl_launch_dependents();
  const int P = max(1, min(max_parts, (L + part_keys - 1) / part_keys));
  const int64_t row0 = ((int64_t)b * nh + h) * max_parts;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = (blockDim.x + 31) >> 5;
  if (P <= 16 && hd <= (int)blockDim.x) {
    // The usual case in one round trip to memory: every thread asks for all maxima and sums (the same few words
    // for all threads) and for its column of every partition at once, then needs no other thread.
    float mv[16], lv[16], ov[16];
#pragma unroll
    for (int p = 0; p < 16; ++p) {
      mv[p] = p < P ? tmp_m[row0 + p] : -INFINITY;
      lv[p] = p < P ? tmp_l[row0 + p] : 0.f;
      ov[p] = (p < P && tid < hd) ? tmp_out[(row0 + p) * hd + tid] : 0.f;     // (never written where mv is -inf: not used then)
    }
    float M = -INFINITY;
#pragma unroll
    for (int p = 0; p < 16; ++p) M = fmaxf(M, mv[p]);
    float lt = 0.f, acc = 0.f;
#pragma unroll
    for (int p = 0; p < 16; ++p) {                   // partitions in index order
      if (mv[p] == -INFINITY) continue;
      const float f = expf(mv[p] - M);
      lt += f * lv[p];
      acc += f * ov[p];
    }
    if (tid < hd) out[tok * out_row_stride + (int64_t)h * hd + tid] = from_f<T>(lt > 0.f ? acc / lt : 0.f);
    return;
  }
  // the largest maximum: a partition per thread, then lanes, then warps
  float mx = -INFINITY;
  for (int p = tid; p < P; p += blockDim.x) mx = fmaxf(mx, tmp_m[row0 + p]);
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < nwarps; ++w) M = fmaxf(M, red[w]);
  float lt = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};      // thread t owns columns t, t + blockDim, ... (hd <= 4 blockDim)
  for (int p0 = 0; p0 < P && M > -INFINITY; p0 += CHUNK) {
    const int n = min(CHUNK, P - p0);
    __syncthreads();
    for (int p = tid; p < n; p += blockDim.x) {
      const float mp = tmp_m[row0 + p0 + p];
      f_s[p] = mp == -INFINITY ? 0.f : expf(mp - M);
    }
    __syncthreads();
    if (hd <= (int)blockDim.x) {
      // a column a thread (the usual head sizes): 32 partitions' loads at a time, so that a long context's dozens of
      // partitions cost two or three trips to memory and not one per eight
      for (int q0 = 0; q0 < n; q0 += 32) {
        float lv[32], ov[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool ok = q0 + i < n && f_s[q0 + i] != 0.f;
          lv[i] = ok ? tmp_l[row0 + p0 + q0 + i] : 0.f;
          ov[i] = ok && tid < hd ? tmp_out[(row0 + p0 + q0 + i) * hd + tid] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {               // partitions in index order
          const float f = q0 + i < n ? f_s[q0 + i] : 0.f;
          if (f != 0.f) {
            lt += f * lv[i];
            acc[0] += f * ov[i];
          }
        }
      }
      continue;
    }
    for (int q0 = 0; q0 < n; q0 += 8) {
      float lv[8], ov[4][8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool ok = q0 + i < n && f_s[q0 + i] != 0.f;
        lv[i] = ok ? tmp_l[row0 + p0 + q0 + i] : 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int d = tid + c * (int)blockDim.x;
          ov[c][i] = ok && d < hd ? tmp_out[(row0 + p0 + q0 + i) * hd + d] : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {                  // partitions in index order
        const float f = q0 + i < n ? f_s[q0 + i] : 0.f;
        if (f != 0.f) {
          lt += f * lv[i];
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[c] += f * ov[c][i];
        }
      }
    }
  }
  T* o = out + tok * out_row_stride + (int64_t)h * hd;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int d = tid + c * (int)blockDim.x;
    if (d < hd) o[d] = from_f<T>(lt > 0.f ? acc[c] / lt : 0.f);
  }
}

ME_API int me_attn_decode_partition() { return DEC_PART; }

// Scratch (caller-provided): tmp_out [D * nh * max_parts * hd] floats, tmp_m and tmp_l
// [D * nh * max_parts] floats each, with max_parts >= ceil(max context / 256).
template <typename T, int GT, int CH>
static void launch_partition(dim3 grid, size_t smem, cudaStream_t stream, const void* qkv,
                             int64_t q_row_stride, const void* pool, const int* bt, int bt_stride,
                             const int* cu, const int* cl, int nh, int nkv, int hd, int page_size,
                             float scale, int window, float* to, float* tm, float* tl, int max_parts) {
  me_launch(decode_partition_kernel<T, GT, CH>, grid, dim3(DEC_THREADS), smem, stream,
      (const T*)qkv, q_row_stride, (const T*)pool, bt, bt_stride, cu, cl, nh, nkv, hd, page_size, scale,
      window, to, tm, tl, max_parts);
}

ME_API int me_attn_decode(const void* qkv, int dtype, int64_t q_row_stride, void* out,
                          int64_t out_row_stride, const void* pool, const int* block_tables,
                          int bt_stride, const int* cu_seqlens, const int* context_lens,
                          int num_reqs, int nh, int nkv, int hd, int page_size, float scale,
                          int window, float* tmp_out, float* tmp_m, float* tmp_l, int max_parts,
                          int* err, int kind, const void* kv_map, cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  ME_REQUIRE(hd % 8 == 0 && hd >= 8 && hd <= 256, "me_attn_decode: head_dim %d is not a multiple of 8 up to 256", hd);
  ME_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "me_attn_decode: %d heads, %d kv heads", nh, nkv);
  ME_REQUIRE(max_parts >= 1 && max_parts <= 65535, "me_attn_decode: max_parts %d", max_parts);
  ME_REQUIRE((q_row_stride * (dtype == ME_BF16 ? 2 : 4)) % 16 == 0 && (hd * (dtype == ME_BF16 ? 2 : 4)) % 16 == 0,
             "me_attn_decode: rows must be 16-byte aligned");
  const int G = nh / nkv;
  const int CH = hd <= 64 ? 1 : (hd <= 128 ? 2 : 4);
  int GT = G >= 4 ? 4 : (G >= 2 ? 2 : 1);
  if (CH == 4 && GT > 2) GT = 2;
  const int head_tiles = (G + GT - 1) / GT;
  ME_REQUIRE((int64_t)nkv * head_tiles <= 65535, "me_attn_decode: too many heads");
  dim3 grid(num_reqs, nkv * head_tiles, max_parts);
  const size_t smem = sizeof(float) * ((size_t)GT * hd + 2 * DEC_GROUPS * GT + (size_t)DEC_GROUPS * GT * hd);
  // kind: 0 = the fastest kernel that takes the shape, 1 = CUDA cores,
  // 3 = tensor cores fed by cp.async, 4 = tensor cores fed by tensor-map loads (needs ``kv_map``, made by
  // me_tma_encode_2d over the cache slot: rows = pages * 2 * kv_heads * page_size, boxes page_size x 64).
  const bool mma_ok = dtype == ME_BF16 && (hd == 64 || hd == 128);
  const bool tma_mma_ok = mma_ok && kv_map != nullptr && err != nullptr && page_size >= 8 && DEC_PART % page_size == 0;
  ME_REQUIRE(kind >= 0 && kind <= 4 && kind != 2 && (kind != 4 || tma_mma_ok) && (kind != 3 || mma_ok),
             "me_attn_decode: kernel kind %d does not take this shape", kind);
  const bool tma_mma = kind == 4 || (kind == 0 && tma_mma_ok);
  const bool mma = !tma_mma && (kind == 3 || (kind == 0 && mma_ok));
  if (tma_mma) {
    const DecodePrep none = {};
    int rc = hd == 64 ? launch_partition_tma_mma<64, false, 2, 16>(kv_map, num_reqs, max_parts, stream, qkv, q_row_stride, block_tables, bt_stride,
                                                            cu_seqlens, context_lens, nh, nkv, page_size, scale, window, tmp_out, tmp_m, tmp_l, 1, err, none)
                      : launch_partition_tma_mma<128, false, 2, 16>(kv_map, num_reqs, max_parts, stream, qkv, q_row_stride, block_tables, bt_stride,
                                                             cu_seqlens, context_lens, nh, nkv, page_size, scale, window, tmp_out, tmp_m, tmp_l, 1, err, none);
    if (rc) return rc;
  }
  if (mma) {
    ME_REQUIRE((int64_t)nkv * ((G + 15) / 16) <= 65535, "me_attn_decode: too many heads");
    int rc = hd == 64 ? launch_partition_mma<64>(num_reqs, max_parts, stream, qkv, q_row_stride, pool, block_tables, bt_stride,
                                                 cu_seqlens, context_lens, nh, nkv, page_size, scale, window, tmp_out, tmp_m, tmp_l)
                      : launch_partition_mma<128>(num_reqs, max_parts, stream, qkv, q_row_stride, pool, block_tables, bt_stride,
                                                  cu_seqlens, context_lens, nh, nkv, page_size, scale, window, tmp_out, tmp_m, tmp_l);
    if (rc) return rc;
  }
  const bool simt = !tma_mma && !mma;
#define ME_DEC_CASE(GT_, CH_)                                                                       \
  if (simt && GT == GT_ && CH == CH_) {                                                             \
    ME_DISPATCH_DTYPE(dtype, T, (launch_partition<T, GT_, CH_>(grid, smem, stream, qkv, q_row_stride, \
        pool, block_tables, bt_stride, cu_seqlens, context_lens, nh, nkv, hd, page_size, scale,     \
        window, tmp_out, tmp_m, tmp_l, max_parts)));                                                \
  }
  ME_DEC_CASE(1, 1) ME_DEC_CASE(2, 1) ME_DEC_CASE(4, 1)
  ME_DEC_CASE(1, 2) ME_DEC_CASE(2, 2) ME_DEC_CASE(4, 2)
  ME_DEC_CASE(1, 4) ME_DEC_CASE(2, 4)
#undef ME_DEC_CASE
  ME_LAUNCH_CHECK("me_attn_decode (partitions)");
  dim3 mgrid(num_reqs, nh);
  const int mthreads = hd >= 128 ? 128 : (hd >= 64 ? 64 : 32);
  ME_DISPATCH_DTYPE(dtype, T, (me_launch(decode_merge_kernel<T>, mgrid, dim3(mthreads), 0, stream,
      (T*)out, out_row_stride, cu_seqlens, context_lens, tmp_out, tmp_m, tmp_l, nh, hd, max_parts, DEC_PART)));
  ME_LAUNCH_CHECK("me_attn_decode (merge)");
  return 0;
}

// Whether me_attn_decode_fused takes the shape (bfloat16 only; the tensor map is the caller's to provide).
ME_API int me_attn_decode_fused_takes(int hd, int page_size) {
  return (hd == 64 || hd == 128) && page_size >= 8 && DEC_PART % page_size == 0;
}

// Decode attention straight from the q|k|v product's bfloat16 rows: the per-head norm of q and k, the rotary
// embedding and the write of the newest key and value to the cache (what me_qk_norm_rope_kv_write does for a
// whole step) happen inside the partition kernel, for requests [0, num_reqs) that bring one token each
// (token row = cu_seqlens[request], position = context_lens[request] - 1).  q_weight/k_weight (both or neither), cos_sin and slot_mapping may be
// null; with a null slot_mapping the newest key and value are expected in the cache already.  The q rows of
// ``qkv`` are left as the product wrote them.  Scratch as for me_attn_decode, with max_parts >= ceil(max context /
// (128 tiles)).  form (of the partition kernel): 0 K and V through one tile, 2 a tile each, 3 half a tile for V beside
// K's.  tiles: how many tiles of 128 keys a block walks, one after the other with a running softmax: what a block does
// once (q's norm and rotation, the merge of its warps, its partial result and the merge kernel's share of it) is then
// spread over that many keys; for batches whose blocks are many times what the device holds at once.
ME_API int me_attn_decode_fused(const void* qkv, int64_t q_row_stride, void* out, int64_t out_row_stride, void* pool,
                                const void* kv_map, const int* block_tables, int bt_stride, const int* cu_seqlens,
                                const int* context_lens, int num_reqs, int nh, int nkv, int hd, int page_size, float scale,
                                int window, const float* q_weight, const float* k_weight, float eps, const float* cos_sin,
                                const int* slot_mapping, float* tmp_out, float* tmp_m, float* tmp_l, int max_parts, int form,
                                int tiles, int* err, cudaStream_t stream) {
  if (num_reqs == 0) return 0;
  ME_REQUIRE(me_attn_decode_fused_takes(hd, page_size), "me_attn_decode_fused: head_dim %d with pages of %d is not taken", hd, page_size);
  ME_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "me_attn_decode_fused: %d heads, %d kv heads", nh, nkv);
  ME_REQUIRE(max_parts >= 1 && max_parts <= 65535, "me_attn_decode_fused: max_parts %d", max_parts);
  ME_REQUIRE(kv_map != nullptr && err != nullptr && pool != nullptr, "me_attn_decode_fused: missing operand");
  ME_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "me_attn_decode_fused: q and k norm weights go together");
  ME_REQUIRE((q_row_stride * 2) % 16 == 0, "me_attn_decode_fused: rows must be 16-byte aligned");
  const int G = nh / nkv;
  ME_REQUIRE((int64_t)nkv * ((G + 15) / 16) <= 65535, "me_attn_decode_fused: too many heads");
  DecodePrep prep = {q_weight, k_weight, eps, cos_sin, slot_mapping, (bf16*)pool};
  ME_REQUIRE(form == 0 || form == 2 || form == 3, "me_attn_decode_fused: unknown form %d", form);
  ME_REQUIRE(tiles >= 1 && tiles <= 64, "me_attn_decode_fused: %d tiles a block", tiles);
  int rc = 1;
#define ME_FUSED(HD_, VBUF_, Q_)                                                                                    \
  rc = launch_partition_tma_mma<HD_, true, VBUF_, Q_>(kv_map, num_reqs, max_parts, stream, qkv, q_row_stride, block_tables, \
                                                           bt_stride, cu_seqlens, context_lens, nh, nkv, page_size, scale, window, \
                                                           tmp_out, tmp_m, tmp_l, tiles, err, prep)
  const bool few_heads = G <= 8;                     // a group's query heads fit the lower half of the m16 strip
  ME_REQUIRE(form != 3 || (DEC_PART / 2) % page_size == 0, "me_attn_decode_fused: pages of %d do not fit half a partition", page_size);
#define ME_FUSED_Q(HD_, VBUF_)                                                                                           \
  do { if (few_heads) ME_FUSED(HD_, VBUF_, 8); else ME_FUSED(HD_, VBUF_, 16); } while (0)
#define ME_FUSED_TILED(HD_, Q_)                                                                                          \
  rc = launch_partition_tma_mma<HD_, true, 0, Q_, true>(kv_map, num_reqs, max_parts, stream, qkv, q_row_stride, block_tables, \
                                                        bt_stride, cu_seqlens, context_lens, nh, nkv, page_size, scale, window, \
                                                        tmp_out, tmp_m, tmp_l, tiles, err, prep)
  ME_REQUIRE(tiles == 1 || form == 0, "me_attn_decode_fused: several tiles a block go with form 0 only");
  if (tiles > 1) {
    if (hd == 64) { if (few_heads) ME_FUSED_TILED(64, 8); else ME_FUSED_TILED(64, 16); }
    else { if (few_heads) ME_FUSED_TILED(128, 8); else ME_FUSED_TILED(128, 16); }
  } else
  if (hd == 64 && form == 2) ME_FUSED(64, 2, 16);
  else if (hd == 64 && form == 3) ME_FUSED_Q(64, 1);
  else if (hd == 64) ME_FUSED_Q(64, 0);
  else if (form == 2) ME_FUSED(128, 2, 16);
  else if (form == 3) ME_FUSED_Q(128, 1);
  else ME_FUSED_Q(128, 0);
#undef ME_FUSED_TILED
#undef ME_FUSED_Q
#undef ME_FUSED
  if (rc) return rc;
  ME_LAUNCH_CHECK("me_attn_decode_fused (partitions)");
  dim3 mgrid(num_reqs, nh);
  me_launch(decode_merge_kernel<bf16>, mgrid, dim3(hd >= 128 ? 128 : 64), 0, stream, (bf16*)out, out_row_stride, cu_seqlens,
            context_lens, tmp_out, tmp_m, tmp_l, nh, hd, max_parts, DEC_PART * tiles);
  ME_LAUNCH_CHECK("me_attn_decode_fused (merge)");
  return 0;
}
