// Host side of the tensor maps: cuTensorMapEncodeTiled through the runtime's driver entry point.
#include "tma.cuh"

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// ``map_out``: 128 bytes, 64-byte aligned.  A row-major [rows][cols] tensor of 2-byte elements whose rows are
// ``row_pitch_bytes`` apart; boxes of [box_rows][box_cols]; swizzle 0 (none) or 128 (bytes).
ME_API int me_tma_encode_2d(void* map_out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_pitch_bytes,
                            uint32_t box_rows, uint32_t box_cols, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  ME_REQUIRE(fn != nullptr, "me_tma_encode_2d: the driver does not offer cuTensorMapEncodeTiled");
  ME_REQUIRE(((uintptr_t)base & 15) == 0 && row_pitch_bytes % 16 == 0, "me_tma_encode_2d: base and row pitch must be 16-byte aligned");
  ME_REQUIRE(box_rows >= 1 && box_rows <= 256 && box_cols >= 1 && box_cols <= 256, "me_tma_encode_2d: box %ux%u", box_rows, box_cols);
  ME_REQUIRE(swizzle == 0 || (swizzle == 128 && box_cols * 2 == 128), "me_tma_encode_2d: the 128-byte swizzle needs boxes of 64 columns");
  ME_REQUIRE(((uintptr_t)map_out & 63) == 0, "me_tma_encode_2d: the map must be 64-byte aligned");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ME_REQUIRE(r == CUDA_SUCCESS, "me_tma_encode_2d: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}
