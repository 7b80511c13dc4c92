// Fused per-head RMSNorm of q and k, rotary embedding, and the write of k and v to their
// cache pages: one pass over the packed qkv rows of a step.
//
// Reference, as three separate steps: models/qwen3.py:34-36 (q_norm, k_norm over head_dim
// with one weight vector for all heads, then rotary), layers/rotary_embedding.py:20-25
// (o[i] = x[i] cos - x[i+d/2] sin, o[i+d/2] = x[i+d/2] cos + x[i] sin), csrc/kv_cache.cu:10-31
// (row t goes to slot_mapping[t], negative slots are skipped).  Statistics, weights, angles
// and the rotation are float32; the result is rounded once.
//
// Cache layout of one cache slot: [page][k|v][kv_head][offset in page][head_dim].
#include "common.cuh"

constexpr int QK_WARPS = 4;
constexpr int MAX_PAIRS = 4;      // head_dim/2 <= 32 lanes * 4

template <typename T>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_rope_kv_kernel(T* __restrict__ qkv, int64_t row_stride, int n_tokens, int nh, int nkv, int hd,
                  const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                  const float* __restrict__ cos_sin, const int* __restrict__ positions,
                  const int* __restrict__ slot_mapping, T* __restrict__ pool, int page_size) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nh + 2 * nkv;
  const int64_t gw = (int64_t)blockIdx.x * QK_WARPS + warp;
  if (gw >= (int64_t)n_tokens * heads) return;
  const int t = (int)(gw / heads), head = (int)(gw % heads);
  T* x = qkv + (int64_t)t * row_stride + (int64_t)head * hd;
  const int half = hd >> 1;
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  const int kvh = is_q ? 0 : (is_k ? head - nh : head - nh - nkv);

  T* dst = nullptr;                       // where this head's row goes in the cache
  if (!is_q) {
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot >= 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      dst = pool + ((((int64_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * hd;
    }
  }
  if (!is_q && !is_k) {                   // v: copy to the cache
    if (dst)
      for (int i = lane; i < hd; i += 32) dst[i] = x[i];
    return;
  }
  float a[MAX_PAIRS], b[MAX_PAIRS];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAX_PAIRS; ++j) {
    const int i = lane + 32 * j;
    if (i < half) {
      a[j] = to_f<T>(x[i]);
      b[j] = to_f<T>(x[i + half]);
      ss += a[j] * a[j] + b[j] * b[j];
    } else {
      a[j] = b[j] = 0.f;
    }
  }
  const float* w = is_q ? qw : kw;
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  const int pos = positions[t];
#pragma unroll
  for (int j = 0; j < MAX_PAIRS; ++j) {
    const int i = lane + 32 * j;
    if (i < half) {
      float y1 = a[j], y2 = b[j];
      if (w) {
        y1 = (y1 * inv) * w[i];
        y2 = (y2 * inv) * w[i + half];
      }
      float o1 = y1, o2 = y2;
      if (cos_sin) {
        const float c = cos_sin[(int64_t)pos * hd + i], s = cos_sin[(int64_t)pos * hd + half + i];
        o1 = y1 * c - y2 * s;
        o2 = y2 * c + y1 * s;
      }
      const T r1 = from_f<T>(o1), r2 = from_f<T>(o2);
      x[i] = r1;
      x[i + half] = r2;
      if (dst) {
        dst[i] = r1;
        dst[i + half] = r2;
      }
    }
  }
}

// The same with vector accesses, for head sizes that are multiples of 64: lane l owns VEC consecutive
// elements of each half (VEC = head_dim / 64), so a warp reads and writes whole 128-byte lines.
template <typename T, int VEC> struct PackOf;
template <> struct PackOf<bf16, 1> { typedef unsigned short type; };
template <> struct PackOf<bf16, 2> { typedef uint32_t type; };
template <> struct PackOf<bf16, 4> { typedef uint2 type; };
template <> struct PackOf<float, 1> { typedef float type; };
template <> struct PackOf<float, 2> { typedef float2 type; };
template <> struct PackOf<float, 4> { typedef float4 type; };

template <typename T, int VEC>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_rope_kv_vec_kernel(T* __restrict__ qkv, int64_t row_stride, int n_tokens, int nh, int nkv,
                      const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                      const float* __restrict__ cos_sin, const int* __restrict__ positions,
                      const int* __restrict__ slot_mapping, T* __restrict__ pool, int page_size) {
  typedef typename PackOf<T, VEC>::type P;
  constexpr int hd = 64 * VEC, half = 32 * VEC;
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nh + 2 * nkv;
  const int64_t gw = (int64_t)blockIdx.x * QK_WARPS + warp;
  if (gw >= (int64_t)n_tokens * heads) return;
  const int t = (int)(gw / heads), head = (int)(gw % heads);
  T* x = qkv + (int64_t)t * row_stride + (int64_t)head * hd;
  const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
  const int kvh = is_q ? 0 : (is_k ? head - nh : head - nh - nkv);
  T* dst = nullptr;
  if (!is_q) {
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot >= 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      dst = pool + ((((int64_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * hd;
    }
  }
  const int i0 = lane * VEC;
  P pa = *reinterpret_cast<const P*>(x + i0), pb = *reinterpret_cast<const P*>(x + half + i0);
  if (!is_q && !is_k) {                   // v: copy to the cache
    if (dst) {
      *reinterpret_cast<P*>(dst + i0) = pa;
      *reinterpret_cast<P*>(dst + half + i0) = pb;
    }
    return;
  }
  const T* ea = reinterpret_cast<const T*>(&pa);
  const T* eb = reinterpret_cast<const T*>(&pb);
  float a[VEC], b[VEC], ss = 0.f;
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    a[j] = to_f<T>(ea[j]);
    b[j] = to_f<T>(eb[j]);
    ss += a[j] * a[j] + b[j] * b[j];
  }
  const float* w = is_q ? qw : kw;
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  const int pos = positions[t];
  P ra, rb;
  T* oa = reinterpret_cast<T*>(&ra);
  T* ob = reinterpret_cast<T*>(&rb);
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    const int i = i0 + j;
    float y1 = a[j], y2 = b[j];
    if (w) {
      y1 = (y1 * inv) * w[i];
      y2 = (y2 * inv) * w[i + half];
    }
    float o1 = y1, o2 = y2;
    if (cos_sin) {
      const float c = cos_sin[(int64_t)pos * hd + i], sn = cos_sin[(int64_t)pos * hd + half + i];
      o1 = y1 * c - y2 * sn;
      o2 = y2 * c + y1 * sn;
    }
    oa[j] = from_f<T>(o1);
    ob[j] = from_f<T>(o2);
  }
  *reinterpret_cast<P*>(x + i0) = ra;
  *reinterpret_cast<P*>(x + half + i0) = rb;
  if (dst) {
    *reinterpret_cast<P*>(dst + i0) = ra;
    *reinterpret_cast<P*>(dst + half + i0) = rb;
  }
}

ME_API int me_qk_norm_rope_kv_write(void* qkv, int dtype, int64_t row_stride, int n_tokens, int nh,
                                    int nkv, int hd, const float* qw, const float* kw, float eps,
                                    const float* cos_sin, const int* positions,
                                    const int* slot_mapping, void* pool, int page_size,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  ME_REQUIRE(hd % 2 == 0 && hd >= 2 && hd <= 64 * MAX_PAIRS,
             "me_qk_norm_rope_kv_write: head_dim %d is not an even number up to %d", hd, 64 * MAX_PAIRS);
  ME_REQUIRE(nh > 0 && nkv > 0 && page_size > 0, "me_qk_norm_rope_kv_write: bad sizes");
  ME_REQUIRE((qw == nullptr) == (kw == nullptr), "me_qk_norm_rope_kv_write: q and k norm weights go together");
  const int64_t warps = (int64_t)n_tokens * (nh + 2 * nkv);
  const int64_t blocks = (warps + QK_WARPS - 1) / QK_WARPS;
  ME_REQUIRE(blocks < 2147483647LL, "me_qk_norm_rope_kv_write: too many tokens");
  const int esize = dtype == ME_BF16 ? 2 : 4;
  const bool vec_ok = (hd == 64 || hd == 128 || hd == 256) && (row_stride * esize) % 16 == 0 && ((uintptr_t)qkv & 15) == 0;
#define ME_QK_VEC(V_)                                                                                   \
  ME_DISPATCH_DTYPE(dtype, T, (me_launch(qk_rope_kv_vec_kernel<T, V_>, dim3((unsigned)blocks), dim3(QK_WARPS * 32), 0, \
      stream, (T*)qkv, row_stride, n_tokens, nh, nkv, qw, kw, eps, cos_sin, positions, slot_mapping, (T*)pool, page_size)))
  if (vec_ok) {
    if (hd == 64) ME_QK_VEC(1);
    else if (hd == 128) ME_QK_VEC(2);
    else ME_QK_VEC(4);
    ME_LAUNCH_CHECK("me_qk_norm_rope_kv_write");
    return 0;
  }
#undef ME_QK_VEC
  ME_DISPATCH_DTYPE(dtype, T, (me_launch(qk_rope_kv_kernel<T>, dim3((unsigned)blocks), dim3(QK_WARPS * 32), 0, stream,
      (T*)qkv, row_stride, n_tokens, nh, nkv, hd, qw, kw, eps, cos_sin, positions, slot_mapping,
      (T*)pool, page_size)));
  ME_LAUNCH_CHECK("me_qk_norm_rope_kv_write");
  return 0;
}
