// 2-D tensor maps over a quantised weight matrix seen as [rows][row bytes / 4] 32-bit words, and the
// copy of one box of such a map into shared memory. Used by the streaming GEMV kernels: one request
// to the copy engine brings 8 rows x one unit instead of one request per row.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ring.cuh"

namespace dyn {

// One box into shared memory (128-byte aligned destination), completing on `bar` with the box's
// full byte count (parts of the box outside the matrix arrive as zeros and count too). x counts
// words along a row and must be a multiple of 4: a tensor copy starts on a 16-byte boundary.
__device__ __forceinline__ void tma_box_g2s(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Map of `rows` rows of `row_bytes` bytes (a multiple of 16, base 16-byte aligned) with boxes of
// box_rows x box_words words, dense in shared memory, zeros outside the matrix. swizzle128 (boxes of
// exactly 32 words = 128 bytes per row, destination 1024-byte aligned): the 16-byte piece c of box row r
// lands at piece c ^ (r & 7), so that lanes reading the same piece of eight rows hit different banks.
inline int make_row_box_map(const uint8_t* data, size_t row_bytes, int64_t rows, int box_words, int box_rows,
                            CUtensorMap* out, bool swizzle128 = false) {
  typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    DYN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    DYN_CHECK(fn != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  DYN_CHECK(row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(data) & 15) == 0 && box_words % 4 == 0 && box_words <= 256,
            "tensor map: rows of %zu bytes / boxes of %d words do not meet the 16-byte rules", row_bytes, box_words);
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 4), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_words, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(data), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DYN_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

}  // namespace dyn
