// Tensor Memory Accelerator helpers: host-side tensor-map construction for (rows, heads, columns)
// tensors and the device-side bulk tensor load (one destination CTA) with mbarrier transaction counting.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llattn {
namespace tma {

constexpr int ERR_TENSOR_MAP = -8;   // LLATTN_ERR_TENSOR_MAP of the public header: the driver refused a tensor map

// A (BT, NH, C) bf16 tensor (C contiguous) seen as a rank-3 map; a box is 64 columns x 1 head x
// `box_rows` rows, 128-byte swizzled: exactly one 64-column panel of a shared-memory operand tile.
inline int make_panel_map(CUtensorMap* out, const void* base, long BT, int NH, int C, int box_rows) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) return ERR_TENSOR_MAP;
        fn = reinterpret_cast<EncodeFn>(ptr);
    }
    const cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)NH, (cuuint64_t)BT};
    const cuuint64_t strides[2] = {(cuuint64_t)C * 2, (cuuint64_t)NH * C * 2};
    const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ERR_TENSOR_MAP;
}

// A (BT, NH, C) fp32 tensor; a box is 32 columns (128 bytes) x 1 head x `box_rows` rows, 128-byte
// swizzled: the unit of the reduce-add stores of gradient tiles.
inline int make_f32_box_map(CUtensorMap* out, const void* base, long BT, int NH, int C, int box_rows) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) return ERR_TENSOR_MAP;
        fn = reinterpret_cast<EncodeFn>(ptr);
    }
    const cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)NH, (cuuint64_t)BT};
    const cuuint64_t strides[2] = {(cuuint64_t)C * 4, (cuuint64_t)NH * C * 4};
    const cuuint32_t box[3] = {32, 1, (cuuint32_t)box_rows};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ERR_TENSOR_MAP;
}

#ifdef __CUDACC__
__device__ __forceinline__ void expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
// one panel: columns [col0, col0+64) of head `head`, rows [row0, row0 + box_rows); col0 * 2 bytes must be a multiple of 16
__device__ __forceinline__ void load_panel(void* smem_dst, const CUtensorMap* map, int col0, int head, int row0, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
        ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(map), "r"(col0), "r"(head), "r"(row0),
          "r"((uint32_t)__cvta_generic_to_shared(bar))
        : "memory");
}
// global[box] += shared[box] (fp32) for one 128 x 32 box; col0 * 4 bytes must be a multiple of 16
__device__ __forceinline__ void reduce_add_box(const CUtensorMap* map, int col0, int head, int row0, const void* smem_src) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3}], [%4];\n"
        ::"l"(map), "r"(col0), "r"(head), "r"(row0), "r"((uint32_t)__cvta_generic_to_shared(smem_src))
        : "memory");
}
// global[box] = shared[box] for one box of a map; col0 * element size must be a multiple of 16 bytes and no coordinate negative
__device__ __forceinline__ void store_box(const CUtensorMap* map, int col0, int head, int row0, const void* smem_src) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];\n"
        ::"l"(map), "r"(col0), "r"(head), "r"(row0), "r"((uint32_t)__cvta_generic_to_shared(smem_src))
        : "memory");
}
__device__ __forceinline__ void commit_group() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// the sources of every committed bulk operation of this thread have been read
__device__ __forceinline__ void wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }
// the sources of every committed bulk operation of this thread but the latest group have been read
__device__ __forceinline__ void wait_group_read1() { asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory"); }
// ... but the latest N groups
template <int N>
__device__ __forceinline__ void wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory"); }
// every committed bulk operation of this thread has completed
__device__ __forceinline__ void wait_group0() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
#endif

}  // namespace tma
}  // namespace llattn
