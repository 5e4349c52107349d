// Host-side construction of TMA tensor maps.  The encoder lives in the driver library; it is looked up
// through the runtime so that this library has no link-time dependency on libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lfm25 {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_entry() {
    static EncodeTiledFn entry = [] {
        void* pointer = nullptr;
        cudaDriverEntryPointQueryResult query = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &query) != cudaSuccess ||
            query != cudaDriverEntryPointSuccess) {
            pointer = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(pointer);
    }();
    return entry;
}

// 2-D row-major tensor [rows, row_bytes / element_size] with 128-byte-swizzled boxes of
// (box_rows x 128 bytes).  `row_bytes` is the pitch and must be a multiple of 16.
inline bool make_swizzled_2d_map(CUtensorMap* map, CUtensorMapDataType type, uint32_t element_size, const void* base,
                                 uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    EncodeTiledFn encode = encode_tiled_entry();
    if (encode == nullptr) {
        return false;
    }
    const cuuint64_t dims[2] = {row_bytes / element_size, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {128 / element_size, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, type, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same for a tensor whose rows are `width` elements wide but `pitch_bytes` apart (a column block of a wider
// buffer); `pitch_bytes` must be a multiple of 16 and `base` 16-byte aligned.
inline bool make_swizzled_2d_map_width(CUtensorMap* map, CUtensorMapDataType type, uint32_t element_size,
                                       const void* base, uint64_t rows, uint64_t width, uint64_t pitch_bytes,
                                       uint32_t box_rows) {
    EncodeTiledFn encode = encode_tiled_entry();
    if (encode == nullptr) {
        return false;
    }
    const cuuint64_t dims[2] = {width, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {128 / element_size, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, type, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace lfm25
