// Self-test of the tcgen05 building blocks (descriptor encodings, swizzled tile layout, TMEM
// readback): one 128 x N x 128 bf16 product per operand-layout combination, written to global
// memory for comparison on the host side.  Exposed as llattn_selftest_umma.
#include "llattn_common.cuh"
#include "umma.cuh"
#include "../../include/llattn.h"

namespace llattn {

// mode 0: A [128][kred], B [N][kred]      -> D = A B^T   (both K-major)
// mode 1: A [128][kred], B [kred][N]      -> D = A B     (A K-major, B MN-major)
// mode 2: A [kred][128], B [kred][N]      -> D = A^T B   (both MN-major)
__global__ void __launch_bounds__(128, 1) umma_selftest_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B,
                                                               float* __restrict__ D, int N, int kred, int mode,
                                                               int* __restrict__ err) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = smem;                 // up to 128 x 128 bf16 = 32 KB
    unsigned char* sB = smem + 32768;         // up to 128 x 128 bf16
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5;

    const int a_rows = (mode == 2) ? kred : 128, a_cols = (mode == 2) ? 128 : kred;
    const int b_rows = (mode == 0) ? N : kred, b_cols = (mode == 0) ? kred : N;
    for (int e = tid; e < a_rows * a_cols; e += 128) {
        const int r = e / a_cols, c = e % a_cols;
        *reinterpret_cast<bf16*>(sA + umma::tile_offset(r, c, a_rows)) = A[e];
    }
    for (int e = tid; e < b_rows * b_cols; e += 128) {
        const int r = e / b_cols, c = e % b_cols;
        *reinterpret_cast<bf16*>(sB + umma::tile_offset(r, c, b_rows)) = B[e];
    }
    if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);
    if (tid == 0) {
        umma::mbar_init(&bar, 1);
        umma::fence_mbar_init();
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tbase = tmem_slot;
    if (tid == 0) {
        const uint32_t a = umma::smem_addr(sA), b = umma::smem_addr(sB);
        if (mode == 0) umma::gemm_kk(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, false, false), false);
        if (mode == 1) umma::gemm_km(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, false, true), false);
        if (mode == 2) umma::gemm_mm(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, true, true), false);
        umma::commit(&bar);
    }
    const bool ok = umma::mbar_wait(&bar, 0);
    umma::fence_after_sync();
    if (!ok) {
        if (tid == 0) atomicExch(err, 1);
    } else {
        for (int c0 = 0; c0 < N; c0 += 32) {
            float v[32];
            umma::tmem_ld32(umma::tmem_addr(tbase, warp, c0), v);
#pragma unroll
            for (int i = 0; i < 32; ++i) D[(long)tid * N + c0 + i] = v[i];
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tbase, 128);
}

}  // namespace llattn

extern "C" int llattn_selftest_umma(const void* A, const void* B, float* D, int N, int kred, int mode, int* err_flag,
                                    void* stream) {
    if (!A || !B || !D || !err_flag) return LLATTN_ERR_NULL;
    if (!(N == 64 || N == 128) || !(kred == 64 || kred == 128) || mode < 0 || mode > 2) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    const size_t sm = 65536 + 1024;
    cudaError_t e = cudaFuncSetAttribute(llattn::umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    llattn::umma_selftest_kernel<<<1, 128, sm, (cudaStream_t)stream>>>((const llattn::bf16*)A, (const llattn::bf16*)B, D, N, kred,
                                                                        mode, err_flag);
    return (int)cudaGetLastError();
}
