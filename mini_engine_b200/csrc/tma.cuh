// Tensor-map (TMA) loads and mbarriers for sm_100a.
//
// Host: me_tma_encode_2d() fills a CUtensorMap for a row-major 2-D tensor through the driver's
// cuTensorMapEncodeTiled (found with cudaGetDriverEntryPoint, so nothing links against libcuda).
// Device: one thread issues cp.async.bulk.tensor loads that complete on an mbarrier; every wait is a
// bounded poll that returns false instead of spinning for ever.
//
// With the 128-byte swizzle a box row is 128 bytes (64 bfloat16) and the 16-byte piece c of row r lands
// at piece c ^ (r % 8) of that row, provided the tile starts on a 1024-byte boundary of shared memory:
// exactly what ldmatrix needs to read 8 rows without bank conflicts.  The first coordinate of a load
// (the column) times the element size must be a multiple of 16 bytes.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace tma {

constexpr unsigned WAIT_LIMIT = 1u << 22;      // polls of an mbarrier before a wait gives up

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(arrivals));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t phase, unsigned limit = WAIT_LIMIT) {
  const uint32_t a = smem_addr(bar);
  for (unsigned i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(a), "r"(phase) : "memory");
    if (done) return true;
  }
  return false;
}
// Box at (col x, row y) of the tensor into shared memory; completes ``bar`` with the box's bytes.
__device__ __forceinline__ void load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

// A [rows][64] bfloat16 tile written by a 128-byte-swizzled load: element (row, 16-byte piece).
__device__ __forceinline__ bf16* swz128(bf16* tile, int row, int piece) {
  return tile + row * 64 + ((piece ^ (row & 7)) << 3);
}

}  // namespace tma
