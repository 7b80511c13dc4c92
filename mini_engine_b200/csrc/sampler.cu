// Greedy and temperature sampling: one block per row of float32 logits.
//
// Reference (layers/sampler.py:5-11): argmax where the temperature is 0, else
// argmax(softmax(logits/T) / E), E ~ Exp(1), which picks the same token as
// argmax(logits/T - log E).  E = -log(u), u = (k + 0.5) / 2^23 with the 23-bit k from a counter-based hash of
// (seed, position, vocabulary index), restated on the host in sampling/sampler.py.  (23 bits, not 24: k + 0.5 must
// be exact in float32, or the largest k would round u to 1 and its entry would win with an infinite key.)
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

// The key of entry v at temperature T > 0: x / T - log(-log(u)), u from the hash of (p, v).
__device__ __forceinline__ float noise_u(uint32_t p, int v) {
  const uint32_t h = mix32((p ^ (uint32_t)v) + 0xC2B2AE35u);
  return ((float)(h >> 9) + 0.5f) * (1.0f / 8388608.0f);      // 23 bits: k + 0.5 is exact in float32 and u stays inside (0, 1)
}
__device__ __forceinline__ float exact_key(float x, float T, uint32_t p, int v) { return x / T - logf(-logf(noise_u(p, v))); }
// The same within 1e-4 (far less for keys of ordinary size) at a quarter of the instructions: the fast logarithm
// (absolute error 2^-21.4 on [0.5, 2], 3 ulp elsewhere) would lose -log(u) for u near 1, where the winners are, so
// there the series of -log(1 - d) stands in, d = 1 - u being exact.
__device__ __forceinline__ float rough_key(float x, float inv_T, uint32_t p, int v) {
  const float u = noise_u(p, v), d = 1.0f - u;
  const float e = d < 0.03125f ? d * (1.0f + d * (0.5f + d * (0.33333334f + d * 0.25f))) : -__logf(u);
  return fmaf(x, inv_T, -__logf(e));
}

// Pass 1: block (row, chunk) finds the best entry of its piece of the vocabulary.  With a temperature every thread
// first takes the rough keys of its entries, then the exact keys of those within a margin of the best rough one
// (one or two as a rule): the entry with the best exact key is always among them, so the draw is the one that exact
// keys for all entries would give.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_partial_kernel(const float* __restrict__ logits, int64_t row_stride, const float* __restrict__ temperature,
                      const int* __restrict__ seeds, const int* __restrict__ positions,
                      float* __restrict__ part_key, int* __restrict__ part_idx, int V, int chunks) {
  constexpr int PER_THREAD = SAMPLE_CHUNK / SAMPLE_THREADS;
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, chunk = blockIdx.y;
  const float* x = logits + (int64_t)row * row_stride;
  const float T = temperature[row];
  const uint32_t s = mix32((uint32_t)seeds[row] + 0x9E3779B9u);
  const uint32_t p = mix32((s ^ (uint32_t)positions[row]) + 0x85EBCA6Bu);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int v0 = chunk * SAMPLE_CHUNK + threadIdx.x;
  float xv[PER_THREAD];
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int v = v0 + i * SAMPLE_THREADS;
    xv[i] = v < V ? x[v] : -INFINITY;
  }
  if (T > 0.f) {
    const float inv_T = 1.0f / T;
    float rough[PER_THREAD], top = -INFINITY;
    int i_top = -1;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
      const int v = v0 + i * SAMPLE_THREADS;
      rough[i] = v < V ? rough_key(xv[i], inv_T, p, v) : -INFINITY;
      if (rough[i] > top) {
        top = rough[i];
        i_top = i;
      }
    }
    // The exact key of the thread's best rough entry, all lanes at once (each for its own entry, read again: an index
    // into registers that is not known at compile time would move them to memory); then, rarely, of the others near it.
    if (i_top >= 0) {
      best_i = v0 + i_top * SAMPLE_THREADS;
      best = exact_key(x[best_i], T, p, best_i);
    }
    const float margin = 1e-3f + 2e-6f * fabsf(top);     // many times the rough keys' error, at any size of key
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
      const int v = v0 + i * SAMPLE_THREADS;
      if (i != i_top && v < V && rough[i] >= top - margin) {
        const float key = exact_key(xv[i], T, p, v);
        if (better(key, v, best, best_i)) {
          best = key;
          best_i = v;
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
      const int v = v0 + i * SAMPLE_THREADS;
      if (v < V && better(xv[i], v, best, best_i)) {
        best = xv[i];
        best_i = v;
      }
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
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    me_set_error("me_sample_static: no usable CUDA device is current");
    return nullptr;
  }
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
