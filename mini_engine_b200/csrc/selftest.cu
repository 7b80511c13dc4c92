// A kernel that exercises the give-up path of the bounded mbarrier waits without any copy in flight.
//
// Every wait of the tensor-map kernels is tma::mbar_wait, a bounded poll that returns false when the barrier
// has not completed in time; the kernel then sets flag 1 of the caller's error word and finishes, and the host
// raises when it next reads the word.  That path cannot be reached with real loads (they always land), so this
// kernel waits on a barrier that nothing ever arrives on: one block, one barrier expecting one arrival, a poll
// limit given by the caller (a few thousand).  Nothing is outstanding when the wait runs out, nothing traps or
// hangs; the kernel reports as the product kernels do and returns.
#include "tma.cuh"

__global__ void wait_expires_kernel(int* err, unsigned limit, int* polls_done) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x == 0) {
    tma::mbar_init(&bar, 1);
    tma::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool landed = tma::mbar_wait(&bar, 0, limit);
    if (!landed) atomicExch(&err[1], 1);
    *polls_done = landed ? 0 : (int)limit;
  }
}

// err: int32[4] on the device (flag 1 is set when the wait ran out); polls_done: int32[1] on the device.
ME_API int me_test_wait_expires(int* err, int limit, int* polls_done, cudaStream_t stream) {
  ME_REQUIRE(err != nullptr && polls_done != nullptr, "me_test_wait_expires: null pointer");
  ME_REQUIRE(limit > 0 && limit <= (1 << 20), "me_test_wait_expires: the poll limit must be in 1..2^20, got %d", limit);
  me_launch(wait_expires_kernel, dim3(1), dim3(32), 0, stream, err, (unsigned)limit, polls_done);
  ME_LAUNCH_CHECK("me_test_wait_expires");
  return 0;
}
