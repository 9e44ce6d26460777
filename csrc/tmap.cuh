// Host-side construction of TMA tensor maps. The driver entry point is fetched at run
// time through the CUDA runtime so that the library links against cudart only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>
#include <stdio.h>

namespace pnm {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of 16-bit elements with `ld` elements between rows;
// box = [box_rows, box_cols]; 128-byte swizzle when box_cols * 2 == 128, else none.
// Returns 0 on success.
inline int make_tmap_2d_b16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                            uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = (box_cols * 2 == 128)  ? CU_TENSOR_MAP_SWIZZLE_128B
                          : (box_cols * 2 == 64) ? CU_TENSOR_MAP_SWIZZLE_64B
                                                 : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D tensor [Z, Y, X] of 16-bit elements, X contiguous, `ldy` elements between rows and `ldz` between slabs;
// box = [1, box_y, 64] with 128-byte swizzle, i.e. box_y rows of 128 bytes in shared memory.  Returns 0 on success.
inline int make_tmap_3d_b16(CUtensorMap* out, const void* base, uint64_t Z, uint64_t Y, uint64_t X, uint64_t ldy,
                            uint64_t ldz, uint32_t box_y) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ldy * 2) & 15) || ((ldz * 2) & 15) || box_y > 256) return -2;
  cuuint64_t dims[3] = {X, Y, Z};
  cuuint64_t strides[2] = {ldy * 2, ldz * 2};
  cuuint32_t box[3] = {64, box_y, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 4-D channels-last image tensor [N, H, W, C] of 16-bit elements; box = [1, box_h, box_w, 64 channels], 128-byte
// swizzle: in shared memory the box is box_h * box_w rows of 128 bytes (x fastest), i.e. the layout of a 2-D
// [rows, 64] tile, so the GEMM's K-major operand descriptors apply unchanged.  Returns 0 on success.
inline int make_tmap_nhwc_b16(CUtensorMap* out, const void* base, uint64_t N, uint64_t H, uint64_t W, uint64_t C,
                              uint32_t box_h, uint32_t box_w) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((C * 2) & 15) || C < 64) return -2;
  cuuint64_t dims[4] = {C, W, H, N};
  cuuint64_t strides[3] = {C * 2, W * C * 2, H * W * C * 2};
  cuuint32_t box[4] = {64, box_w, box_h, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace pnm
