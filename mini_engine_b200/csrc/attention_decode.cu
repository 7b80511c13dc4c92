// Paged attention for requests that bring one token: split over the keys, then merged.
//
// Reference (csrc/paged_decode.cu:247-334): the context is cut into partitions of 256 keys at
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

constexpr int DEC_PART = 256, DEC_THREADS = 128, DEC_LANES = 8, DEC_GROUPS = DEC_THREADS / DEC_LANES;

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

template <typename T>
__global__ void decode_merge_kernel(T* __restrict__ out, int64_t out_row_stride,
                                    const int* __restrict__ cu_seqlens,
                                    const int* __restrict__ context_lens,
                                    const float* __restrict__ tmp_out, const float* __restrict__ tmp_m,
                                    const float* __restrict__ tmp_l, int nh, int hd, int max_parts) {
  const int b = blockIdx.x, h = blockIdx.y;
  const int L = context_lens[b];
  const int P = max(1, min(max_parts, (L + DEC_PART - 1) / DEC_PART));
  const int64_t row0 = ((int64_t)b * nh + h) * max_parts;
  float M = -INFINITY;
  for (int p = 0; p < P; ++p) M = fmaxf(M, tmp_m[row0 + p]);
  T* o = out + (int64_t)cu_seqlens[b] * out_row_stride + (int64_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float lt = 0.f, acc = 0.f;
    if (M > -INFINITY) {
      for (int p = 0; p < P; ++p) {
        const float mp = tmp_m[row0 + p];
        if (mp == -INFINITY) continue;
        const float f = expf(mp - M);
        lt += f * tmp_l[row0 + p];
        acc += f * tmp_out[(row0 + p) * hd + d];
      }
    }
    o[d] = from_f<T>(lt > 0.f ? acc / lt : 0.f);
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
  decode_partition_kernel<T, GT, CH><<<grid, DEC_THREADS, smem, stream>>>(
      (const T*)qkv, q_row_stride, (const T*)pool, bt, bt_stride, cu, cl, nh, nkv, hd, page_size, scale,
      window, to, tm, tl, max_parts);
}

ME_API int me_attn_decode(const void* qkv, int dtype, int64_t q_row_stride, void* out,
                          int64_t out_row_stride, const void* pool, const int* block_tables,
                          int bt_stride, const int* cu_seqlens, const int* context_lens,
                          int num_reqs, int nh, int nkv, int hd, int page_size, float scale,
                          int window, float* tmp_out, float* tmp_m, float* tmp_l, int max_parts,
                          cudaStream_t stream) {
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
#define ME_DEC_CASE(GT_, CH_)                                                                       \
  if (GT == GT_ && CH == CH_) {                                                                     \
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
  ME_DISPATCH_DTYPE(dtype, T, (decode_merge_kernel<T><<<mgrid, mthreads, 0, stream>>>(
      (T*)out, out_row_stride, cu_seqlens, context_lens, tmp_out, tmp_m, tmp_l, nh, hd, max_parts)));
  ME_LAUNCH_CHECK("me_attn_decode (merge)");
  return 0;
}
