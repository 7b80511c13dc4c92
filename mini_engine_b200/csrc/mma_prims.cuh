// Tensor-core and asynchronous-copy primitives shared by the bfloat16 attention kernels:
// cp.async with zero fill, ldmatrix, mma.sync m16n8k16 (bfloat16 in, float32 accumulate), and a
// shared-memory tile layout whose 16-byte pieces are XOR-swizzled against bank conflicts.
#pragma once
#include "common.cuh"

namespace mma_prims {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;     // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A tile of [rows][HD] bfloat16 in shared memory; 16-byte piece c of row r lives at piece c ^ (r & 7).
template <int HD>
__device__ __forceinline__ bf16* tile_ptr(bf16* base, int row, int piece) {
  return base + row * HD + ((piece ^ (row & 7)) << 3);
}

// Where a key's row lives in a paged pool [page][k|v][kv_head][offset][head_dim]: the element offset of
// K's row for key j (V's row is ``v_off`` further), or -1 if the page was given back.  ``page_shift`` is
// log2(page_size) for powers of two (a shift and a mask replace the division), else -1.
struct PageMap {
  const int* bt;
  int page_size, page_shift;
  int64_t page_stride, head_off;     // 2 * nkv * page_size * hd;  kv_head * page_size * hd
  int hd;
  __device__ __forceinline__ int64_t row(int j) const {
    int pi, off;
    if (page_shift >= 0) {
      pi = j >> page_shift;
      off = j & (page_size - 1);
    } else {
      pi = j / page_size;
      off = j - pi * page_size;
    }
    const int page = bt[pi];
    return page < 0 ? -1 : (int64_t)page * page_stride + head_off + (int64_t)off * hd;
  }
};

__device__ __forceinline__ int log2_if_pow2(int x) { return (x & (x - 1)) == 0 ? 31 - __clz(x) : -1; }

}  // namespace mma_prims
