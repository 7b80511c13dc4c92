/* me_sample_static: the sampling kernels for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference (its sampler, layers/sampler.py:4-11, is
 * eager PyTorch that allocates its temporaries freely); it exists for hosts of this library that
 * are not allowed to call cudaMalloc at the moment they want a token drawn.  Examples: code that
 * runs inside someone else's memory plan (a plugin in a process whose device memory is handed
 * out once at start-up and is then closed), code on a path that must not block (cudaMalloc and
 * cudaFree synchronise the device), and code that simply has no allocator to get the sampler's
 * work buffer from.  me_sample() asks its caller for that work buffer; me_sample_static() keeps
 * one inside the library instead, as a file-scope __device__ array, and so takes only inputs
 * and the output.
 *
 * Limits: at most ME_SAMPLE_STATIC_MAX_ROWS rows and ME_SAMPLE_STATIC_MAX_VOCAB vocabulary
 * entries per call; larger calls are refused with a message (me_last_error()).  The array is
 * 32 KB and every GPU that loads the library holds it until the process exits.
 *
 * The first call on a device looks the array's device address up (cudaGetSymbolAddress) and keeps
 * it; make that first call outside any stream capture.  All calls on a device share the one array:
 * it still holds the last call's partial results, which is harmless because every call writes each
 * entry it later reads (nothing in it has to start at zero), but two calls that overlap on the GPU
 * (different streams, no ordering between them) would overwrite each other's partial results.
 * Order such calls, or use me_sample() with a buffer per stream.  The function calls neither
 * cudaMalloc nor cudaFree nor any routine that allocates.
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define ME_SAMPLE_STATIC_MAX_ROWS 64
#define ME_SAMPLE_STATIC_MAX_VOCAB 262144

#ifdef __cplusplus
extern "C" {
#endif

/* logits [S][row_stride] float32 (V entries used per row), temperature [S] float32 (0 = greedy),
 * seeds and positions [S] int32, out [S] int32; all device pointers.  Returns 0, or non-zero with
 * a message in me_last_error(). */
int me_sample_static(const float* logits, int64_t row_stride, const float* temperature, const int* seeds,
                     const int* positions, int* out, int S, int V, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
