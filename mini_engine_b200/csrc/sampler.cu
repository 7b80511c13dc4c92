// Greedy and temperature sampling: one block per row of float32 logits.
//
// Reference (layers/sampler.py:5-11): argmax where the temperature is 0, else
// argmax(softmax(logits/T) / E), E ~ Exp(1), which picks the same token as
// argmax(logits/T - log E).  E = -log(u), u in (0,1) from a counter-based hash of
// (seed, position, vocabulary index), restated on the host in sampling/sampler.py.
// Ties go to the lower index.
#include "common.cuh"

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

constexpr int SAMPLE_THREADS = 1024;

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int64_t row_stride, const float* __restrict__ temperature,
              const int* __restrict__ seeds, const int* __restrict__ positions, int* __restrict__ out, int V) {
  __shared__ float s_key[32];
  __shared__ int s_idx[32];
  const int row = blockIdx.x;
  const float* x = logits + (int64_t)row * row_stride;
  const float T = temperature[row];
  const uint32_t s = mix32((uint32_t)seeds[row] + 0x9E3779B9u);
  const uint32_t p = mix32((s ^ (uint32_t)positions[row]) + 0x85EBCA6Bu);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int v = threadIdx.x; v < V; v += SAMPLE_THREADS) {
    float key = x[v];
    if (T > 0.f) {
      const uint32_t h = mix32((p ^ (uint32_t)v) + 0xC2B2AE35u);
      const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
      key = key / T - logf(-logf(u));
    }
    if (key > best || (key == best && v < best_i)) {
      best = key;
      best_i = v;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ok = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ok > best || (ok == best && oi < best_i)) {
      best = ok;
      best_i = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_key[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
      if (s_key[w] > best || (s_key[w] == best && s_idx[w] < best_i)) {
        best = s_key[w];
        best_i = s_idx[w];
      }
    out[row] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

ME_API int me_sample(const float* logits, int64_t row_stride, const float* temperature, const int* seeds,
                     const int* positions, int* out, int S, int V, cudaStream_t stream) {
  if (S == 0) return 0;
  ME_REQUIRE(S > 0 && V > 0, "me_sample: bad sizes S=%d V=%d", S, V);
  sample_kernel<<<S, SAMPLE_THREADS, 0, stream>>>(logits, row_stride, temperature, seeds, positions, out, V);
  ME_LAUNCH_CHECK("me_sample");
  return 0;
}
