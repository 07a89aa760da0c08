// Host-side encoding of TMA tensor maps and the device-side tiled load, shared by the prefill and
// decode kernels.  The encoder is a driver entry point fetched through the runtime, so the library
// links no driver stub.
#pragma once

#include <cuda.h>

#include "b2kv_common.cuh"

namespace b2kv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// View of a cache of any layout as (d, token, head, sequence): element (b, t, h, d) at
// b*sb + t*st + h*sh + d (strides in elements).  `tokens` bounds the token coordinate: rows past it
// read as zero and are not written.  `box_tokens` rows of `box_d` elements per copy.
inline bool make_cache_tensor_map(CUtensorMap* map, const void* base, int dtype, int D, int tokens, int H, int B,
                                  int64_t sb, int64_t st, int64_t sh, int box_d, int box_tokens,
                                  CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (fn == nullptr) return false;
    const cuuint64_t es = static_cast<cuuint64_t>(elt_bytes(dtype));
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(H),
                                static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st) * es, static_cast<cuuint64_t>(sh) * es,
                                   static_cast<cuuint64_t>(sb) * es};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(box_d), static_cast<cuuint32_t>(box_tokens), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType type =
        dtype == B2KV_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    return fn(map, type, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Global -> shared tiled load of one box; completion is counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

}  // namespace b2kv
