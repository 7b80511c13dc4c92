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
constexpr int QK_MAX_HD = 256;
constexpr int QK_PER_LANE = QK_MAX_HD / 32;

// Any even head size up to 256, and a rotation over the first ``rd`` <= head_dim elements only (the two halves of
// those rd elements are paired; elements from rd on pass through the rotation unchanged).  A lane owns elements
// lane, lane + 32, ...; the normalised values go through a per-warp row of shared memory so that a lane finds its
// element's partner wherever it lives.  With rd = head_dim this is the arithmetic of the vector kernel below.
template <typename T>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_rope_kv_kernel(T* __restrict__ qkv, int64_t row_stride, int n_tokens, int nh, int nkv, int hd, int rd,
                  const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                  const float* __restrict__ cos_sin, const int* __restrict__ positions,
                  const int* __restrict__ slot_mapping, T* __restrict__ pool, int page_size) {
  __shared__ float ys[QK_WARPS][QK_MAX_HD];
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
  float v[QK_PER_LANE];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < QK_PER_LANE; ++j) {
    const int i = lane + 32 * j;
    v[j] = i < hd ? to_f<T>(x[i]) : 0.f;
    ss += v[j] * v[j];
  }
  const float* w = is_q ? qw : kw;
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)hd + eps);
  }
#pragma unroll
  for (int j = 0; j < QK_PER_LANE; ++j) {
    const int i = lane + 32 * j;
    if (i < hd) {
      if (w) v[j] = (v[j] * inv) * w[i];
      ys[warp][i] = v[j];
    }
  }
  __syncwarp();
  const int pos = positions[t], rh = rd >> 1;
#pragma unroll
  for (int j = 0; j < QK_PER_LANE; ++j) {
    const int i = lane + 32 * j;
    if (i < hd) {
      float o = v[j];
      if (cos_sin && i < rd) {
        const int f = i < rh ? i : i - rh;                          // the pair's frequency
        const float c = cos_sin[(int64_t)pos * rd + f], s = cos_sin[(int64_t)pos * rd + rh + f];
        o = i < rh ? v[j] * c - ys[warp][i + rh] * s : v[j] * c + ys[warp][i - rh] * s;
      }
      const T r = from_f<T>(o);
      x[i] = r;
      if (dst) dst[i] = r;
    }
  }
}

// The same with 16-byte accesses, for head sizes 64, 128 and 256.  A lane owns E = 16 / sizeof(T) consecutive
// elements of each half of a head, so LPH = head_dim / 2 / E neighbouring lanes hold one head and a warp holds
// 32 / LPH heads of one token at a time; it takes QK_PASSES such sets, whose loads are issued together (bytes in
// flight are what a pass like this lives on).  The token's position, slot and rotation are read once per warp,
// before griddepcontrol.wait, like the norm weights.
constexpr int QK_PASSES = 2;

template <typename T, int HD>
__global__ void __launch_bounds__(QK_WARPS * 32)
qk_rope_kv_vec_kernel(T* __restrict__ qkv, int64_t row_stride, int n_tokens, int nh, int nkv,
                      const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                      const float* __restrict__ cos_sin, const int* __restrict__ positions,
                      const int* __restrict__ slot_mapping, T* __restrict__ pool, int page_size) {
  constexpr int E = 16 / sizeof(T), half = HD / 2, LPH = half / E, HPW = 32 / LPH;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nh + 2 * nkv, units = (heads + HPW * QK_PASSES - 1) / (HPW * QK_PASSES);
  const int64_t gw = (int64_t)blockIdx.x * QK_WARPS + warp;
  const bool active = gw < (int64_t)n_tokens * units;
  const int t = active ? (int)(gw / units) : 0, head0 = active ? (int)(gw % units) * (HPW * QK_PASSES) : heads;
  const int e0 = (lane % LPH) * E, sub = lane / LPH;
  float c[E], sn[E];
  const int pos = active ? positions[t] : 0;
  const int slot = active && slot_mapping ? slot_mapping[t] : -1;
#pragma unroll
  for (int j = 0; j < E; j += 4) {             // E is 4 or 8; the table's rows and e0 are multiples of 4 floats
    const float4 cv = cos_sin ? *reinterpret_cast<const float4*>(cos_sin + (int64_t)pos * HD + e0 + j) : make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 sv = cos_sin ? *reinterpret_cast<const float4*>(cos_sin + (int64_t)pos * HD + half + e0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    c[j] = cv.x; c[j + 1] = cv.y; c[j + 2] = cv.z; c[j + 3] = cv.w;
    sn[j] = sv.x; sn[j + 1] = sv.y; sn[j + 2] = sv.z; sn[j + 3] = sv.w;
  }
  pdl_wait();
  pdl_launch_dependents();
  T* row = qkv + (int64_t)t * row_stride;
  uint4 pa[QK_PASSES], pb[QK_PASSES];
#pragma unroll
  for (int r = 0; r < QK_PASSES; ++r) {
    const int head = head0 + r * HPW + sub;
    pa[r] = pb[r] = make_uint4(0, 0, 0, 0);
    if (head < heads) {
      pa[r] = *reinterpret_cast<const uint4*>(row + (int64_t)head * HD + e0);
      pb[r] = *reinterpret_cast<const uint4*>(row + (int64_t)head * HD + half + e0);
    }
  }
  const bool norm = qw != nullptr;
#pragma unroll
  for (int r = 0; r < QK_PASSES; ++r) {
    const int head = head0 + r * HPW + sub;
    const bool live = head < heads;
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    const int kvh = is_q ? 0 : (is_k ? head - nh : head - nh - nkv);
    T* dst = nullptr;
    if (live && !is_q && slot >= 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      dst = pool + ((((int64_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * HD;
    }
    const T* ea = reinterpret_cast<const T*>(&pa[r]);
    const T* eb = reinterpret_cast<const T*>(&pb[r]);
    float a[E], b[E], ss = 0.f;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      a[j] = to_f<T>(ea[j]);
      b[j] = to_f<T>(eb[j]);
      ss += a[j] * a[j] + b[j] * b[j];
    }
    float inv = 1.f;
    if (norm) {                               // every lane takes part; the lanes of one head add up
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = 1.0f / sqrtf(ss / (float)HD + eps);
    }
    uint4 ra = pa[r], rb = pb[r];             // v: copied as it is
    if (is_q || is_k) {
      T* oa = reinterpret_cast<T*>(&ra);
      T* ob = reinterpret_cast<T*>(&rb);
      const float* w = is_q ? qw : kw;         // a few hundred bytes that stay in L1
#pragma unroll
      for (int j = 0; j < E; ++j) {
        float y1 = a[j], y2 = b[j];
        if (norm) {
          y1 = (y1 * inv) * w[e0 + j];
          y2 = (y2 * inv) * w[half + e0 + j];
        }
        float o1 = y1, o2 = y2;
        if (cos_sin) {
          o1 = y1 * c[j] - y2 * sn[j];
          o2 = y2 * c[j] + y1 * sn[j];
        }
        oa[j] = from_f<T>(o1);
        ob[j] = from_f<T>(o2);
      }
      if (live) {
        *reinterpret_cast<uint4*>(row + (int64_t)head * HD + e0) = ra;
        *reinterpret_cast<uint4*>(row + (int64_t)head * HD + half + e0) = rb;
      }
    }
    if (dst) {
      *reinterpret_cast<uint4*>(dst + e0) = ra;
      *reinterpret_cast<uint4*>(dst + half + e0) = rb;
    }
  }
}

// Warps that a launch of the vector kernel needs.
template <typename T>
static int64_t vec_warps(int n_tokens, int heads, int hd) {
  const int hpw = 32 / (hd / 2 / (16 / (int)sizeof(T)));
  return (int64_t)n_tokens * ((heads + hpw * QK_PASSES - 1) / (hpw * QK_PASSES));
}

// cos_sin: float32 [positions][rotary_dim] (cos of the rotary_dim / 2 frequencies, then their sines), or null.
// rotary_dim: how many leading elements of a head are rotated (even, at most head_dim).
ME_API int me_qk_norm_rope_kv_write(void* qkv, int dtype, int64_t row_stride, int n_tokens, int nh,
                                    int nkv, int hd, const float* qw, const float* kw, float eps,
                                    const float* cos_sin, int rotary_dim, const int* positions,
                                    const int* slot_mapping, void* pool, int page_size,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  ME_REQUIRE(hd % 2 == 0 && hd >= 2 && hd <= QK_MAX_HD,
             "me_qk_norm_rope_kv_write: head_dim %d is not an even number up to %d", hd, QK_MAX_HD);
  if (cos_sin == nullptr) rotary_dim = hd;
  ME_REQUIRE(rotary_dim % 2 == 0 && rotary_dim >= 2 && rotary_dim <= hd,
             "me_qk_norm_rope_kv_write: rotary_dim %d is not an even number up to head_dim %d", rotary_dim, hd);
  ME_REQUIRE(nh > 0 && nkv > 0 && page_size > 0, "me_qk_norm_rope_kv_write: bad sizes");
  ME_REQUIRE((qw == nullptr) == (kw == nullptr), "me_qk_norm_rope_kv_write: q and k norm weights go together");
  const int64_t warps = (int64_t)n_tokens * (nh + 2 * nkv);
  const int64_t blocks = (warps + QK_WARPS - 1) / QK_WARPS;
  ME_REQUIRE(blocks < 2147483647LL, "me_qk_norm_rope_kv_write: too many tokens");
  const int esize = dtype == ME_BF16 ? 2 : 4;
  const bool vec_ok = (hd == 64 || hd == 128 || hd == 256) && rotary_dim == hd && (row_stride * esize) % 16 == 0 &&
                      ((uintptr_t)qkv & 15) == 0;
#define ME_QK_VEC(HD_)                                                                                  \
  ME_DISPATCH_DTYPE(dtype, T, (me_launch(qk_rope_kv_vec_kernel<T, HD_>,                                 \
      dim3((unsigned)((vec_warps<T>(n_tokens, nh + 2 * nkv, HD_) + QK_WARPS - 1) / QK_WARPS)), dim3(QK_WARPS * 32), 0, \
      stream, (T*)qkv, row_stride, n_tokens, nh, nkv, qw, kw, eps, cos_sin, positions, slot_mapping, (T*)pool, page_size)))
  if (vec_ok) {
    if (hd == 64) ME_QK_VEC(64);
    else if (hd == 128) ME_QK_VEC(128);
    else ME_QK_VEC(256);
    ME_LAUNCH_CHECK("me_qk_norm_rope_kv_write");
    return 0;
  }
#undef ME_QK_VEC
  ME_DISPATCH_DTYPE(dtype, T, (me_launch(qk_rope_kv_kernel<T>, dim3((unsigned)blocks), dim3(QK_WARPS * 32), 0, stream,
      (T*)qkv, row_stride, n_tokens, nh, nkv, hd, rotary_dim, qw, kw, eps, cos_sin, positions, slot_mapping,
      (T*)pool, page_size)));
  ME_LAUNCH_CHECK("me_qk_norm_rope_kv_write");
  return 0;
}
