// tcgen05 (5th-generation tensor core) primitives for sm_100a: tensor memory allocation, shared-memory
// and instruction descriptors, MMA issue by one thread, completion through mbarriers, and loads of the
// accumulator from tensor memory.
//
// Operands live in shared memory in the layout that a 128-byte-swizzled TMA load writes: a tile of
// [rows][64 bfloat16] (128 bytes a row), groups of 8 rows 1024 bytes apart, starting on a 1024-byte
// boundary ("K-major, SWIZZLE_128B").  One tcgen05.mma of kind::f16 consumes 16 elements of K (32 bytes
// of every row), so the four K steps inside a 64-element tile advance the descriptor's start address by
// 32 bytes each.  The accumulator D [128 lanes][N columns] of float32 lives in tensor memory; warp w of a
// warpgroup may read lanes 32 (w % 4) .. 32 (w % 4) + 31.
#pragma once
#include "common.cuh"
#include "tma.cuh"

namespace tc5 {

// ---- tensor memory ------------------------------------------------------------------------------------
// One whole warp allocates ``cols`` columns (a power of two >= 32) and the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma::smem_addr(slot_in_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile: start address, stride between groups
// of 8 rows (1024 bytes), descriptor version 1, layout type SWIZZLE_128B (2).
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(const void* tile) {
  const uint64_t addr = tma::smem_addr(tile);
  uint64_t d = 0;
  d |= (addr & 0x3FFFFu) >> 4;                 // bits  0..13: start address / 16
  d |= (uint64_t)0 << 16;                      // bits 16..29: leading byte offset (unused for this layout)
  d |= (uint64_t)(1024 >> 4) << 32;            // bits 32..45: stride byte offset / 16
  d |= (uint64_t)1 << 46;                      // bits 46..47: descriptor version of sm_100
  d |= (uint64_t)2 << 61;                      // bits 61..63: SWIZZLE_128B
  return d;
}
// The same tile read as an MN-major operand (the 64-element direction is M or N, rows are K): groups of 8
// K rows 1024 bytes apart (stride byte offset); successive 64-element blocks of M/N ``lbo_bytes`` apart.
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128(const void* tile, uint32_t lbo_bytes) {
  const uint64_t addr = tma::smem_addr(tile);
  uint64_t d = 0;
  d |= (addr & 0x3FFFFu) >> 4;
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of kind::f16: bfloat16 A and B, float32 D, M x N; A and B each K-major or MN-major.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int M, int N, bool b_mn_major = false, bool a_mn_major = false) {
  return (1u << 4)                      // D format: float32
         | (1u << 7)                    // A format: bfloat16
         | (1u << 10)                   // B format: bfloat16
         | ((a_mn_major ? 1u : 0u) << 15)
         | ((b_mn_major ? 1u : 0u) << 16)
         | ((uint32_t)(N >> 3) << 17)   // N / 8
         | ((uint32_t)(M >> 4) << 24);  // M / 16
}

// ---- issue and completion -----------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]^T, one thread issues.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// The same with A in tensor memory: [128 lanes][K / 2 columns], two consecutive bfloat16 of a row's K in a 32-bit column.
__device__ __forceinline__ void mma_f16_a_in_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has finished.
__device__ __forceinline__ void commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tma::smem_addr(bar)) : "memory");
}

// ---- issue by a whole warp ------------------------------------------------------------------------------------
// The warp that issues the products runs its loop with all 32 lanes, every lane holding the same values, and one
// elected lane issues.  A loop inside ``if (lane == 0)`` is divergent code to the compiler, which then computes
// descriptors and addresses in ordinary registers and moves them over for every product; the issuing thread, not
// the tensor core, set the pace that way (measured on a B200: eight products of 128 x 128 x 16 from shared memory in
// 890 clocks from one lane, 700 from a warp with the descriptors' low words computed and the high words held).
// The warp's index must be known to be the same in all lanes: take it through ``uniform_warp_index()``.
__device__ __forceinline__ int uniform_warp_index() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }
// A shared-memory descriptor as two words: tiles, stages and K steps differ in the low word (start address / 16) only.
struct DescWords { uint32_t lo, hi; };
__device__ __forceinline__ DescWords words_of(uint64_t desc) { return {(uint32_t)desc, (uint32_t)(desc >> 32)}; }
// D[tmem] (+)= A[smem] * B[smem]^T; ``a_off`` and ``b_off`` (units of 16 bytes) are added to the start addresses.
__device__ __forceinline__ void mma_f16_elect(uint32_t d_tmem, DescWords a, uint32_t a_off, DescWords b, uint32_t b_off, uint32_t idesc,
                                              bool accumulate) {
  asm volatile("{\n.reg .pred p, q;\n.reg .b64 da, db;\nmov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\nsetp.ne.b32 p, %6, 0;\n"
               "elect.sync _|q, 0xffffffff;\n@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}\n"
               ::"r"(d_tmem), "r"(a.lo + a_off), "r"(a.hi), "r"(b.lo + b_off), "r"(b.hi), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// The same with A in tensor memory.
__device__ __forceinline__ void mma_f16_a_in_tmem_elect(uint32_t d_tmem, uint32_t a_tmem, DescWords b, uint32_t b_off, uint32_t idesc,
                                                        bool accumulate) {
  asm volatile("{\n.reg .pred p, q;\n.reg .b64 db;\nmov.b64 db, {%2, %3};\nsetp.ne.b32 p, %5, 0;\n"
               "elect.sync _|q, 0xffffffff;\n@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}\n"
               ::"r"(d_tmem), "r"(a_tmem), "r"(b.lo + b_off), "r"(b.hi), "r"(idesc), "r"((uint32_t)accumulate) : "memory");
}
// One arrival when every MMA the warp's elected lane issued so far has finished (the election names the same lane every time).
__device__ __forceinline__ void commit_elect(unsigned long long* bar) {
  asm volatile("{\n.reg .pred q;\nelect.sync _|q, 0xffffffff;\n@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n"
               ::"r"(tma::smem_addr(bar)) : "memory");
}
// A bounded wait of all lanes of a warp on one barrier, with one answer for the warp.
__device__ __forceinline__ bool mbar_wait_warp(unsigned long long* bar, uint32_t phase) {
  return __all_sync(0xffffffffu, tma::mbar_wait(bar, phase));
}

// 32 consecutive float32 columns of this thread's lane.
__device__ __forceinline__ void ld_32cols(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16 consecutive float32 columns of this thread's lane.
__device__ __forceinline__ void ld_16cols(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 64 consecutive float32 columns of this thread's lane in one instruction.
__device__ __forceinline__ void ld_64cols(uint32_t taddr, float (&v)[64]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
               : "r"(taddr)
               : "memory");
}
// Stores of 64 / 32 consecutive float32 columns of this thread's lane, and the wait that makes them complete.
__device__ __forceinline__ void st_64cols(uint32_t taddr, const float (&v)[64]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile("tcgen05.st.sync.aligned.32x32b.x64.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63,%64};\n"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(r[32]), "r"(r[33]), "r"(r[34]), "r"(r[35]), "r"(r[36]), "r"(r[37]), "r"(r[38]), "r"(r[39]), "r"(r[40]), "r"(r[41]), "r"(r[42]), "r"(r[43]), "r"(r[44]), "r"(r[45]), "r"(r[46]), "r"(r[47]), "r"(r[48]), "r"(r[49]), "r"(r[50]), "r"(r[51]), "r"(r[52]), "r"(r[53]), "r"(r[54]), "r"(r[55]), "r"(r[56]), "r"(r[57]), "r"(r[58]), "r"(r[59]), "r"(r[60]), "r"(r[61]), "r"(r[62]), "r"(r[63])
               : "memory");
}
__device__ __forceinline__ void st_32cols(uint32_t taddr, const float (&v)[32]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
__device__ __forceinline__ void st_16cols(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

}  // namespace tc5
