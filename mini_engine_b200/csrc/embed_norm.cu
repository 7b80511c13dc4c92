// Embedding gather into the float32 residual stream; residual add + RMSNorm; SiLU-and-multiply.
//
// Reference formulas: layers/embed_head.py:11 (gather), layers/layernorm.py:11-23
// (y = x * rsqrt(mean(x^2) + eps) in float32, then the weight; with a residual the sum
// is normalised), layers/activation.py:4-7 (silu(gate) * up).
#include "common.cuh"

// A negative id ~j stands for ``feedback[j]``: the token that the step before drew for row j, still on the
// device.  That lets the host launch a decode step before it has read the step before it.
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ out, int H, int V, int* __restrict__ err,
                             const int* __restrict__ feedback, int n_feedback) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && feedback != nullptr && ~id < n_feedback) id = feedback[~id];
  const bool ok = id >= 0 && id < V;
  if (!ok && threadIdx.x == 0) atomicOr(err, 1);
  const TW* row = table + (int64_t)(ok ? id : 0) * H;
  float* o = out + (int64_t)t * H;
  for (int h = threadIdx.x; h < H; h += blockDim.x) o[h] = ok ? to_f<TW>(row[h]) : 0.f;
}

ME_API int me_embed(const int* ids, const void* table, int table_dtype, float* out, int T, int H,
                    int V, int* err, const int* feedback, int n_feedback, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && H > 0 && V > 0, "me_embed: bad sizes T=%d H=%d V=%d", T, H, V);
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  ME_DISPATCH_DTYPE(table_dtype, TW,
                    me_launch(embed_kernel<TW>, dim3(T), dim3(threads), 0, stream, ids, (const TW*)table, out, H, V, err,
                              feedback, n_feedback));
  ME_LAUNCH_CHECK("me_embed");
  return 0;
}

// One block per output row.  Both passes read res (+ delta); the second writes.  ``delta`` may
// come as ``splits`` partial results (a split-K product), each ``split_stride`` elements apart;
// they are added in order.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ res, const TD* __restrict__ delta,
                                   const float* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H, int write_res, int splits,
                                   int64_t split_stride) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r_out = blockIdx.x;
  const int64_t r = rows ? rows[r_out] : r_out;
  float* rr = res + r * H;
  const TD* dd = delta ? delta + r * H : nullptr;
  float ss = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = rr[h];
    if (dd) {
      float d = to_f<TD>(dd[h]);
      for (int s = 1; s < splits; ++s) d += to_f<TD>(dd[h + s * split_stride]);
      v += d;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* oo = out + (int64_t)r_out * H;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float v = rr[h];
    if (dd) {
      float d = to_f<TD>(dd[h]);
      for (int s = 1; s < splits; ++s) d += to_f<TD>(dd[h + s * split_stride]);
      v += d;
    }
    if (write_res) rr[h] = v;
    oo[h] = from_f<TO>((v * inv) * w[h]);
  }
}

// The same in one pass for rows of up to NV * blockDim elements: a thread keeps its NV sums in registers.
template <typename TD, typename TO, int NV>
__global__ void add_rmsnorm_regs_kernel(float* __restrict__ res, const TD* __restrict__ delta,
                                        const float* __restrict__ w, float eps, TO* __restrict__ out,
                                        const int* __restrict__ rows, int H, int write_res, int splits,
                                        int64_t split_stride) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r_out = blockIdx.x;
  const int64_t r = rows ? rows[r_out] : r_out;
  float* rr = res + r * H;
  const TD* dd = delta ? delta + r * H : nullptr;
  float v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int h = threadIdx.x + i * blockDim.x;
    v[i] = 0.f;
    if (h < H) {
      v[i] = rr[h];
      if (dd) {
        float d = to_f<TD>(dd[h]);
        for (int s = 1; s < splits; ++s) d += to_f<TD>(dd[h + s * split_stride]);
        v[i] += d;
      }
      ss += v[i] * v[i];
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* oo = out + (int64_t)r_out * H;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int h = threadIdx.x + i * blockDim.x;
    if (h < H) {
      if (write_res) rr[h] = v[i];
      oo[h] = from_f<TO>((v[i] * inv) * w[h]);
    }
  }
}

// The same with four consecutive elements per access (H a multiple of 4, up to 8 * blockDim).
template <typename TD, typename TO>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ res, const TD* __restrict__ delta,
                                        const float* __restrict__ w, float eps, TO* __restrict__ out,
                                        const int* __restrict__ rows, int H, int write_res, int splits,
                                        int64_t split_stride) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r_out = blockIdx.x;
  const int64_t r = rows ? rows[r_out] : r_out;
  float* rr = res + r * H;
  const TD* dd = delta ? delta + r * H : nullptr;
  float v[2][4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int h = (threadIdx.x + i * blockDim.x) * 4;
    v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    if (h < H) {
      const float4 a = *reinterpret_cast<const float4*>(rr + h);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
      if (dd) {
        for (int s = 0; s < splits; ++s) {
#pragma unroll
          for (int e = 0; e < 4; ++e) v[i][e] += to_f<TD>(dd[h + e + s * split_stride]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* oo = out + (int64_t)r_out * H;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int h = (threadIdx.x + i * blockDim.x) * 4;
    if (h < H) {
      if (write_res) *reinterpret_cast<float4*>(rr + h) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
      const float4 ww = *reinterpret_cast<const float4*>(w + h);
      oo[h] = from_f<TO>((v[i][0] * inv) * ww.x);
      oo[h + 1] = from_f<TO>((v[i][1] * inv) * ww.y);
      oo[h + 2] = from_f<TO>((v[i][2] * inv) * ww.z);
      oo[h + 3] = from_f<TO>((v[i][3] * inv) * ww.w);
    }
  }
}

// Eight consecutive elements with 16-byte (bfloat16) or 2 x 16-byte (float32) accesses.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h[k]);
    v[2 * k] = f.x;
    v[2 * k + 1] = f.y;
  }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// Many rows (a portion of a prompt): a warp per row, every load of the row issued before the first is used, no
// block-wide barrier.  H a multiple of 8 up to 256 * CH; the lane's chunks are elements 8 (lane + 32 i) .. + 7.
// ``splits`` partial results ``split_stride`` elements apart are added in order.
template <typename TD, typename TO, int CH>
__global__ void __launch_bounds__(128)
add_rmsnorm_rows_kernel(float* __restrict__ res, const TD* __restrict__ delta, const float* __restrict__ w, float eps,
                        TO* __restrict__ out, int n_rows, int H, int splits, int64_t split_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  float ww[CH][8];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int h = 8 * (lane + 32 * i);
    if (h < H) load8(w + h, ww[i]);
  }
  pdl_wait();
  pdl_launch_dependents();
  if (r >= n_rows) return;
  float* rr = res + r * H;
  float v[CH][8], d[CH][8];
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int h = 8 * (lane + 32 * i);
    if (h < H) {
      load8(rr + h, v[i]);
      if (delta) load8(delta + r * H + h, d[i]);
    }
  }
  if (delta) {
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      if (8 * (lane + 32 * i) < H) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += d[i][e];
      }
    }
  }
  for (int sp = 1; sp < splits; ++sp) {                 // the second and later partial results, in their order
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int h = 8 * (lane + 32 * i);
      if (h < H) {
        load8(delta + sp * split_stride + r * H + h, d[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += d[i][e];
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int h = 8 * (lane + 32 * i);
    if (h < H) {
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int h = 8 * (lane + 32 * i);
    if (h < H) {
      if (delta) store8(rr + h, v[i]);
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[i][e] * inv) * ww[i][e];
      store8(out + r * H + h, o);
    }
  }
}

ME_API int me_add_rmsnorm(float* res, const void* delta, int delta_dtype, const float* w, float eps,
                          void* out, int out_dtype, const int* rows, int n_rows, int H, int splits,
                          int64_t split_stride, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  ME_REQUIRE(n_rows > 0 && H > 0 && splits >= 1, "me_add_rmsnorm: bad sizes rows=%d H=%d splits=%d", n_rows, H, splits);
  const int write_res = rows == nullptr;     // gathered rows leave the residual as it is
  constexpr int NV = 8;
  // portions of prompts: a warp per row
  const bool aligned16 = (((uintptr_t)res | (uintptr_t)w | (uintptr_t)delta | (uintptr_t)out) & 15) == 0;
  if (n_rows >= 64 && rows == nullptr && (splits == 1 || (delta != nullptr && split_stride % 4 == 0)) && H % 8 == 0 && H <= 2048 &&
      aligned16) {
    const unsigned blocks = (unsigned)((n_rows + 3) / 4);
#define ME_ROWS(CH_)                                                                                              \
    ME_DISPATCH_DTYPE(delta_dtype, TD, ME_DISPATCH_DTYPE(out_dtype, TO,                                           \
        (me_launch(add_rmsnorm_rows_kernel<TD, TO, CH_>, dim3(blocks), dim3(128), 0, stream, res, (const TD*)delta, w, eps, \
                   (TO*)out, n_rows, H, splits, split_stride))))
    if (H <= 256) ME_ROWS(1); else if (H <= 512) ME_ROWS(2); else if (H <= 1024) ME_ROWS(4); else ME_ROWS(8);
#undef ME_ROWS
    ME_LAUNCH_CHECK("me_add_rmsnorm");
    return 0;
  }
  if (H % 4 == 0 && H <= 8 * 1024 && ((uintptr_t)res & 15) == 0 && ((uintptr_t)w & 15) == 0) {
    int threads = ((H / 4 + 1) / 2 + 31) / 32 * 32;
    if (threads < 32) threads = 32;
    ME_DISPATCH_DTYPE(delta_dtype, TD, ME_DISPATCH_DTYPE(out_dtype, TO,
        (me_launch(add_rmsnorm_vec4_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, stream,
                   res, (const TD*)delta, w, eps, (TO*)out, rows, H, write_res, splits, split_stride))));
  } else if (H <= NV * 1024) {
    int threads = ((H + NV - 1) / NV + 31) / 32 * 32;
    if (threads < 64) threads = 64;
    ME_DISPATCH_DTYPE(delta_dtype, TD, ME_DISPATCH_DTYPE(out_dtype, TO,
        (me_launch(add_rmsnorm_regs_kernel<TD, TO, NV>, dim3(n_rows), dim3(threads), 0, stream,
                   res, (const TD*)delta, w, eps, (TO*)out, rows, H, write_res, splits, split_stride))));
  } else {
    ME_DISPATCH_DTYPE(delta_dtype, TD, ME_DISPATCH_DTYPE(out_dtype, TO,
        (me_launch(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(1024), 0, stream,
                   res, (const TD*)delta, w, eps, (TO*)out, rows, H, write_res, splits, split_stride))));
  }
  ME_LAUNCH_CHECK("me_add_rmsnorm");
  return 0;
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t n, int I) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t t = i / I;
  const int c = (int)(i - t * I);
  const float g = to_f<T>(x[t * 2 * I + c]);
  const float u = to_f<T>(x[t * 2 * I + I + c]);
  out[i] = from_f<T>(g / (1.0f + expf(-g)) * u);
}

// Eight elements per thread with 16-byte accesses (bfloat16, I a multiple of 8).
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, int64_t n8, int I8) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const int64_t t = i / I8;
  const int c = (int)(i - t * I8);
  const uint4 g = *reinterpret_cast<const uint4*>(x + (t * 2 * I8 + c) * 8);
  const uint4 u = *reinterpret_cast<const uint4*>(x + (t * 2 * I8 + I8 + c) * 8);
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint4 r;
  __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]);
    rp[k] = __floats2bfloat162_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y);
  }
  *reinterpret_cast<uint4*>(out + i * 8) = r;
}

ME_API int me_silu_mul(const void* x, void* out, int dtype, int T, int I, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && I > 0, "me_silu_mul: bad sizes T=%d I=%d", T, I);
  if (dtype == ME_BF16 && I % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int64_t n8 = (int64_t)T * (I / 8);
    const int64_t blocks8 = (n8 + 255) / 256;
    ME_REQUIRE(blocks8 < 2147483647LL, "me_silu_mul: too many elements");
    me_launch(silu_mul_vec8_kernel, dim3((unsigned)blocks8), dim3(256), 0, stream, (const bf16*)x, (bf16*)out, n8, I / 8);
    ME_LAUNCH_CHECK("me_silu_mul");
    return 0;
  }
  const int64_t n = (int64_t)T * I;
  const int threads = 256;
  const int64_t blocks = (n + threads - 1) / threads;
  ME_REQUIRE(blocks < 2147483647LL, "me_silu_mul: too many elements");
  ME_DISPATCH_DTYPE(dtype, TT,
                    me_launch(silu_mul_kernel<TT>, dim3((unsigned)blocks), dim3(threads), 0, stream, (const TT*)x, (TT*)out, n, I));
  ME_LAUNCH_CHECK("me_silu_mul");
  return 0;
}
