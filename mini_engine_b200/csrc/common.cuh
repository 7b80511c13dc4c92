// Shared helpers of the mini_engine_b200 kernels (sm_100a only).
//
// Every exported function has C linkage, takes raw device pointers, sizes and the stream
// to launch on, returns 0 on success and a non-zero code after storing a message that
// me_last_error() returns.  No function allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <math.h>
#include <utility>

#define ME_API extern "C" __attribute__((visibility("default")))

enum MeDtype { ME_F32 = 0, ME_BF16 = 1 };
typedef __nv_bfloat16 bf16;

void me_set_error(const char* fmt, ...);

#define ME_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      me_set_error(__VA_ARGS__);         \
      return 1;                          \
    }                                    \
  } while (0)

#define ME_LAUNCH_CHECK(what)                                             \
  do {                                                                    \
    cudaError_t e_ = cudaGetLastError();                                  \
    if (e_ != cudaSuccess) {                                              \
      me_set_error("%s: launch failed: %s", what, cudaGetErrorString(e_)); \
      return 2;                                                           \
    }                                                                     \
  } while (0)

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// Sum over a thread block in a fixed order (lanes by butterfly, then warps in index order),
// so that the result does not depend on anything but the data and the block size.
__device__ __forceinline__ float block_sum(float x, float* red /* >= 32 floats of shared memory */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  x = warp_sum(x);
  __syncthreads();
  if (lane == 0) red[warp] = x;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarps; ++w) total += red[w];
  return total;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// Every kernel is launched so that it may start while its predecessor in the stream is still running
// (cudaLaunchAttributeProgrammaticStreamSerialization).  A kernel first fetches what no earlier kernel
// of the step writes (weights, block tables), then calls pdl_wait(), which returns once the predecessor
// has finished and its writes are visible, and only then touches activations or the cache; it writes
// nothing before pdl_wait().  pdl_launch_dependents() lets the successor be scheduled.  In a launch
// without the attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

bool me_pdl_enabled();
int me_sm_count();          // SMs of the current device (asked once)

template <typename... KArgs, typename... Args>
inline cudaError_t me_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = me_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Run `body` with T bound to the C type of a dtype code.
#define ME_DISPATCH_DTYPE(code, T, ...)                                  \
  do {                                                                   \
    if ((code) == ME_F32) { typedef float T; __VA_ARGS__; }              \
    else if ((code) == ME_BF16) { typedef bf16 T; __VA_ARGS__; }         \
    else { me_set_error("unknown dtype code %d", (int)(code)); return 1; } \
  } while (0)
