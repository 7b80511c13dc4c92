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

constexpr int SAMPLE_THREADS = 256;
constexpr int SAMPLE_CHUNK = 4096;        // vocabulary entries per block of the first pass

__device__ __forceinline__ bool better(float k, int i, float bk, int bi) { return k > bk || (k == bk && i < bi); }

// Reduce (key, index) over the block; the result is valid in thread 0.
__device__ __forceinline__ void block_best(float& best, int& best_i) {
  __shared__ float s_key[32];
  __shared__ int s_idx[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ok = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (better(ok, oi, best, best_i)) {
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
  if (threadIdx.x == 0)
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (better(s_key[w], s_idx[w], best, best_i)) {
        best = s_key[w];
        best_i = s_idx[w];
      }
}

// Pass 1: block (row, chunk) finds the best entry of its piece of the vocabulary.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_partial_kernel(const float* __restrict__ logits, int64_t row_stride, const float* __restrict__ temperature,
                      const int* __restrict__ seeds, const int* __restrict__ positions,
                      float* __restrict__ part_key, int* __restrict__ part_idx, int V, int chunks) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, chunk = blockIdx.y;
  const float* x = logits + (int64_t)row * row_stride;
  const float T = temperature[row];
  const uint32_t s = mix32((uint32_t)seeds[row] + 0x9E3779B9u);
  const uint32_t p = mix32((s ^ (uint32_t)positions[row]) + 0x85EBCA6Bu);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int v_end = min(V, (chunk + 1) * SAMPLE_CHUNK);
  for (int v = chunk * SAMPLE_CHUNK + threadIdx.x; v < v_end; v += SAMPLE_THREADS) {
    float key = x[v];
    if (T > 0.f) {
      const uint32_t h = mix32((p ^ (uint32_t)v) + 0xC2B2AE35u);
      const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
      key = key / T - logf(-logf(u));
    }
    if (better(key, v, best, best_i)) {
      best = key;
      best_i = v;
    }
  }
  block_best(best, best_i);
  if (threadIdx.x == 0) {
    part_key[(int64_t)row * chunks + chunk] = best;
    part_idx[(int64_t)row * chunks + chunk] = best_i;
  }
}

// Pass 2: one block per row picks the best of the chunks.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_final_kernel(const float* __restrict__ part_key, const int* __restrict__ part_idx, int* __restrict__ out, int chunks) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += SAMPLE_THREADS) {
    const float k = part_key[(int64_t)row * chunks + c];
    const int i = part_idx[(int64_t)row * chunks + c];
    if (better(k, i, best, best_i)) {
      best = k;
      best_i = i;
    }
  }
  block_best(best, best_i);
  if (threadIdx.x == 0) out[row] = best_i == 0x7fffffff ? 0 : best_i;
}

ME_API int me_sample_chunks(int V) { return (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK; }

// Scratch (caller-provided): part_key and part_idx of S * me_sample_chunks(V) entries each.
ME_API int me_sample(const float* logits, int64_t row_stride, const float* temperature, const int* seeds,
                     const int* positions, int* out, int S, int V, float* part_key, int* part_idx,
                     cudaStream_t stream) {
  if (S == 0) return 0;
  ME_REQUIRE(S > 0 && V > 0, "me_sample: bad sizes S=%d V=%d", S, V);
  const int chunks = me_sample_chunks(V);
  ME_REQUIRE(chunks <= 65535, "me_sample: vocabulary %d is too large", V);
  me_launch(sample_partial_kernel, dim3(S, chunks), dim3(SAMPLE_THREADS), 0, stream, logits, row_stride, temperature, seeds,
            positions, part_key, part_idx, V, chunks);
  ME_LAUNCH_CHECK("me_sample (pass 1)");
  me_launch(sample_final_kernel, dim3(S), dim3(SAMPLE_THREADS), 0, stream, part_key, part_idx, out, chunks);
  ME_LAUNCH_CHECK("me_sample (pass 2)");
  return 0;
}

// ---- the same two passes with the work buffer inside the library (see sampler_static.h) -------------
#include "sampler_static.h"
#include <mutex>

constexpr int SAMPLE_STATIC_ENTRIES = ME_SAMPLE_STATIC_MAX_ROWS * (ME_SAMPLE_STATIC_MAX_VOCAB / SAMPLE_CHUNK);

// Partial results of pass 1: SAMPLE_STATIC_ENTRIES keys (float) followed by as many indices (int).
// In host code this name is only a handle; the address a kernel can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_sample_static_scratch[SAMPLE_STATIC_ENTRIES * 8];

static void* sample_static_scratch_of_current_device(int* device_out) {
  constexpr int MAX_DEVICES = 64;
  static void* ptrs[MAX_DEVICES] = {};
  static std::mutex lock;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  *device_out = dev;
  std::lock_guard<std::mutex> guard(lock);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_sample_static_scratch);     // once per device, that device current
    if (e != cudaSuccess) {
      me_set_error("me_sample_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

ME_API int me_sample_static(const float* logits, int64_t row_stride, const float* temperature, const int* seeds,
                            const int* positions, int* out, int S, int V, cudaStream_t stream) {
  if (S == 0) return 0;
  ME_REQUIRE(S > 0 && V > 0, "me_sample_static: bad sizes S=%d V=%d", S, V);
  ME_REQUIRE(S <= ME_SAMPLE_STATIC_MAX_ROWS, "me_sample_static: %d rows, the built-in work buffer holds %d; use me_sample()",
             S, ME_SAMPLE_STATIC_MAX_ROWS);
  ME_REQUIRE(V <= ME_SAMPLE_STATIC_MAX_VOCAB, "me_sample_static: vocabulary %d, the built-in work buffer holds %d; use me_sample()",
             V, ME_SAMPLE_STATIC_MAX_VOCAB);
  int dev = -1;
  me_set_error("me_sample_static: no usable CUDA device is current");
  void* scratch = sample_static_scratch_of_current_device(&dev);
  if (scratch == nullptr) return 1;
  const int chunks = me_sample_chunks(V);
  float* part_key = static_cast<float*>(scratch);
  int* part_idx = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + sizeof(float) * SAMPLE_STATIC_ENTRIES);
  me_launch(sample_partial_kernel, dim3(S, chunks), dim3(SAMPLE_THREADS), 0, stream, logits, row_stride, temperature, seeds,
            positions, part_key, part_idx, V, chunks);
  ME_LAUNCH_CHECK("me_sample_static (pass 1)");
  me_launch(sample_final_kernel, dim3(S), dim3(SAMPLE_THREADS), 0, stream, part_key, part_idx, out, chunks);
  ME_LAUNCH_CHECK("me_sample_static (pass 2)");
  return 0;
}
