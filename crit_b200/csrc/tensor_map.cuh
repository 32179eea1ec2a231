// Host side of the TMA loads: tensor maps over one page tensor, made per launch (a pure host call, no stream work).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace crit_b200 {

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline encode_tiled_fn encoder() {
    static encode_tiled_fn found = nullptr;
    static bool asked = false;
    if (!asked) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult how;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &how) == cudaSuccess &&
            how == cudaDriverEntryPointSuccess)
            found = (encode_tiled_fn)fn;
        cudaGetLastError();
        asked = true;
    }
    return found;
}

// A 3-D map over one page tensor [slots][kv_heads][dim]; a box is 16 slots of one head, 128 bytes wide.
inline bool page_map(CUtensorMap* map, const void* pages, int pk, int dim, int kv_heads, int64_t slots) {
    encode_tiled_fn encode = encoder();
    if (!encode) return false;
    const int es = pk < 2 ? 2 : 1;
    const CUtensorMapDataType type = pk == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                             : (pk == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
    const cuuint64_t dims[3] = {(cuuint64_t)dim, (cuuint64_t)kv_heads, (cuuint64_t)slots};
    const cuuint64_t strides[2] = {(cuuint64_t)dim * es, (cuuint64_t)dim * es * kv_heads};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / es), 1, 16};
    const cuuint32_t steps[3] = {1, 1, 1};
    return encode(map, type, 3, const_cast<void*>(pages), dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same E4M3 page tensor with the dimensions permuted, [128 bytes][slots][kv_heads]: a box is 16 slots of ALL kv
// heads, one contiguous piece of the tensor (16 x kv_heads x 128 bytes) that lands head-major, row 16 * head + slot.
inline bool page_rows_map(CUtensorMap* map, const void* pages, int dim, int kv_heads, int64_t slots) {
    encode_tiled_fn encode = encoder();
    if (!encode || dim != 128 || kv_heads < 1 || kv_heads > 8) return false;
    const cuuint64_t dims[3] = {128, (cuuint64_t)slots, (cuuint64_t)kv_heads};
    const cuuint64_t strides[2] = {(cuuint64_t)128 * kv_heads, 128};
    const cuuint32_t box[3] = {128, 16, (cuuint32_t)kv_heads};
    const cuuint32_t steps[3] = {1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(pages), dims, strides, box, steps,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace crit_b200
