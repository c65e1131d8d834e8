// Tensor-map (TMA) helpers shared by the kernels that fetch pages of the key/value
// cache as boxes: the host side encodes a map of one layer's cache seen as a matrix
// [pages * kv heads * page size, head size] with boxes of `box_rows` x 64 elements
// and the 128-byte swizzle; the device side issues one tiled copy that reports its
// bytes to an mbarrier.  The innermost coordinate of every copy is a multiple of 64
// elements (128 bytes), as a tiled copy needs a 16-byte aligned start.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace slb_tma {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// bfloat16 matrix [rows, row_elems] (row_elems a multiple of 64), boxes of box_rows x 64
static inline int make_rows_map(CUtensorMap* map, const void* ptr, int row_elems, long long rows,
                                int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return SLB_ERR_BAD_ARG;
    const cuuint64_t dims[2] = {(cuuint64_t)row_elems, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_elems * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : SLB_ERR_BAD_ARG;
}

// The same matrix seen as [panels of 64 elements][rows][64]: a box of
// {64, box_rows, row_elems / 64} brings box_rows whole rows with ONE copy and lands
// as [panel][row][64 elements], each 128-byte line swizzled as in the 2-D form.
static inline int make_paneled_rows_map(CUtensorMap* map, const void* ptr, int row_elems, long long rows,
                                        int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr || row_elems % 64 != 0) return SLB_ERR_BAD_ARG;
    const cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(row_elems / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)row_elems * 2, 128u};
    const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)(row_elems / 64)};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : SLB_ERR_BAD_ARG;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)),
          "r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// the 3-D copy with an L2 eviction policy for the lines it brings (createpolicy)
__device__ __forceinline__ void tma_load_3d_hint(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                                 int c1, int c2, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)),
          "r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)),
          "r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(c0), "r"(c1)
        : "memory");
}

}  // namespace slb_tma
