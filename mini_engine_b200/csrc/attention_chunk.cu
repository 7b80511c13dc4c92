// Paged attention for portions of prompts (and, if asked, single tokens) on the CUDA cores:
// any head size that is a multiple of 8 up to 256, any number of heads and groups, any page
// size, an optional window.  This is the attention of the float32 engine and the fallback of
// the bfloat16 engine where its tensor-core kernel refuses a shape.
//
// Reference semantics (csrc/paged_prefill.cu:98-130,200-203, layers/attention.py:21-40):
// a request's portion of q_len tokens ends at context length L, so local query i sits at
// position start + i with start = L - q_len and sees cached keys j <= start + i; scores are
// scaled, softmax runs online in float32 over tiles of keys, the output is O / l.  With a
// window w only keys j > position - w are seen.  Key tiles start at multiples of ATT_BK
// counted from position 0 (from the first tile a window can reach), so the order of a
// query's sums does not depend on how the prompt was cut or what shares the batch.
//
// One block = 16 queries of one request x one query head; 128 threads; thread (r, c) owns
// row r = tid/8, keys c, c+8, c+16, c+24 of a tile and output dims c, c+8, ...
#include "common.cuh"

constexpr int ATT_BQ = 16, ATT_BK = 32, ATT_THREADS = 128, ATT_MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attn_chunk_kernel(const T* __restrict__ qkv, int64_t q_row_stride, T* __restrict__ out,
                  int64_t out_row_stride, const T* __restrict__ pool,
                  const int* __restrict__ block_tables, int bt_stride,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                  const int* __restrict__ tiles, int nh, int nkv, int hd, int page_size,
                  float scale, int window) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int ldh = hd + 1;
  float* Qs = smem;                          // [ATT_BQ][ldh]
  float* Ks = Qs + ATT_BQ * ldh;             // [ATT_BK][ldh]
  float* Vs = Ks + ATT_BK * ldh;             // [ATT_BK][ldh]
  float* Ps = Vs + ATT_BK * ldh;             // [ATT_BQ][ATT_BK + 1]
  const int tid = threadIdx.x, r = tid >> 3, c = tid & 7;
  const int b = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
  const int head = blockIdx.y, kvh = head / (nh / nkv);
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int L = context_lens[b], start = L - q_len;
  const int rows = min(ATT_BQ, q_len - q0);
  const int* bt = block_tables + (int64_t)b * bt_stride;

  for (int idx = tid; idx < ATT_BQ * hd; idx += ATT_THREADS) {
    const int rr = idx / hd, d = idx - rr * hd;
    Qs[rr * ldh + d] = rr < rows ? to_f<T>(qkv[(int64_t)(tok0 + q0 + rr) * q_row_stride + (int64_t)head * hd + d]) : 0.f;
  }
  const int p_r = start + q0 + r;            // position of this thread's query row
  const bool row_ok = r < rows;
  const int hi = min(L, start + q0 + rows);  // keys [lo, hi) can be seen by some row of the tile
  int lo = window > 0 ? max(0, start + q0 - window + 1) : 0;
  lo = (lo / ATT_BK) * ATT_BK;

  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAX_HD / 8];
#pragma unroll
  for (int k = 0; k < ATT_MAX_HD / 8; ++k) acc[k] = 0.f;

  for (int kt = lo; kt < hi; kt += ATT_BK) {
    __syncthreads();                          // previous tile fully consumed (and Q stored)
    for (int idx = tid; idx < ATT_BK * hd; idx += ATT_THREADS) {
      const int jj = idx / hd, d = idx - jj * hd;
      const int j = kt + jj;
      float kv = 0.f, vv = 0.f;
      if (j < hi) {
        const int page = bt[j / page_size];
        if (page >= 0) {
          const int64_t base = (((int64_t)page * 2) * nkv + kvh) * page_size * hd + (int64_t)(j % page_size) * hd + d;
          kv = to_f<T>(pool[base]);
          vv = to_f<T>(pool[base + (int64_t)nkv * page_size * hd]);
        }
      }
      Ks[jj * ldh + d] = kv;
      Vs[jj * ldh + d] = vv;
    }
    __syncthreads();
    float s[4];
    float tmax = -INFINITY;
#pragma unroll
    for (int mm = 0; mm < 4; ++mm) {
      const int jj = c + 8 * mm, j = kt + jj;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot = fmaf(Qs[r * ldh + d], Ks[jj * ldh + d], dot);
      const bool seen = row_ok && j <= p_r && j < L && (window <= 0 || j > p_r - window);
      s[mm] = seen ? dot * scale : -INFINITY;
      tmax = fmaxf(tmax, s[mm]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    const float m_new = fmaxf(m, tmax);
    float alpha = 1.f, psum = 0.f;
    if (m_new == -INFINITY) {
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) Ps[r * (ATT_BK + 1) + c + 8 * mm] = 0.f;
    } else {
      alpha = expf(m - m_new);                // m = -inf gives 0
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) {
        const float p = expf(s[mm] - m_new);  // masked scores give 0
        Ps[r * (ATT_BK + 1) + c + 8 * mm] = p;
        psum += p;
      }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l = l * alpha + psum;
    m = m_new;
    __syncwarp();                             // a row's 8 threads sit in one warp
#pragma unroll
    for (int k = 0; k < ATT_MAX_HD / 8; ++k) {
      const int d = c + 8 * k;
      if (d < hd) {
        float a = acc[k] * alpha;
        for (int jj = 0; jj < ATT_BK; ++jj) a = fmaf(Ps[r * (ATT_BK + 1) + jj], Vs[jj * ldh + d], a);
        acc[k] = a;
      }
    }
  }
  if (row_ok) {
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (int64_t)(tok0 + q0 + r) * out_row_stride + (int64_t)head * hd;
#pragma unroll
    for (int k = 0; k < ATT_MAX_HD / 8; ++k) {
      const int d = c + 8 * k;
      if (d < hd) o[d] = from_f<T>(acc[k] * inv);
    }
  }
}

ME_API int me_attn_chunk_tile_q() { return ATT_BQ; }

ME_API int me_attn_chunk(const void* qkv, int dtype, int64_t q_row_stride, void* out,
                         int64_t out_row_stride, const void* pool, const int* block_tables,
                         int bt_stride, const int* cu_seqlens, const int* context_lens,
                         const int* tiles, int num_tiles, int nh, int nkv, int hd, int page_size,
                         float scale, int window, cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  ME_REQUIRE(hd % 8 == 0 && hd >= 8 && hd <= ATT_MAX_HD,
             "me_attn_chunk: head_dim %d is not a multiple of 8 up to %d", hd, ATT_MAX_HD);
  ME_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0, "me_attn_chunk: %d heads, %d kv heads", nh, nkv);
  ME_REQUIRE(nh <= 65535, "me_attn_chunk: too many heads");
  const size_t smem = sizeof(float) * ((size_t)(ATT_BQ + 2 * ATT_BK) * (hd + 1) + ATT_BQ * (ATT_BK + 1));
  dim3 grid(num_tiles, nh);
  ME_DISPATCH_DTYPE(dtype, T, {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(attn_chunk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_attn_chunk: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
    me_launch(attn_chunk_kernel<T>, grid, dim3(ATT_THREADS), smem, stream,
        (const T*)qkv, q_row_stride, (T*)out, out_row_stride, (const T*)pool, block_tables, bt_stride,
        cu_seqlens, context_lens, tiles, nh, nkv, hd, page_size, scale, window);
  });
  ME_LAUNCH_CHECK("me_attn_chunk");
  return 0;
}
