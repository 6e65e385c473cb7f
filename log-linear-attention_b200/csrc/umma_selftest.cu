// Self-test of the tcgen05 building blocks (descriptor encodings, swizzled tile layout, TMEM
// readback): one 128 x N x 128 bf16 product per operand-layout combination, written to global
// memory for comparison on the host side.  Exposed as llattn_selftest_umma.
#include "llattn_common.cuh"
#include "umma.cuh"
#include "../../include/llattn.h"
#include "llattn_testing.h"

namespace llattn {

// mode 0: A [128][kred], B [N][kred]      -> D = A B^T   (both K-major)
// mode 1: A [128][kred], B [kred][N]      -> D = A B     (A K-major, B MN-major)
// mode 2: A [kred][128], B [kred][N]      -> D = A^T B   (both MN-major)
__global__ void __launch_bounds__(128, 1) umma_selftest_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B,
                                                               float* __restrict__ D, int N, int kred, int tmode,
                                                               int* __restrict__ err) {
    const int mode = tmode >= 10 ? tmode - 10 + 100 : tmode;      // 100.. : no run-time shaped issue below
    const int lmode = tmode % 10;                                  // operand layout combination
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // modes 10..12 place the tiles high in shared memory (the address range that the kernels' later tiles use)
    unsigned char* sA = smem + (tmode >= 10 ? 131072 : 0);              // up to 128 x 128 bf16 = 32 KB
    unsigned char* sB = smem + (tmode >= 10 ? 131072 + 49152 : 32768);  // up to 128 x 128 bf16
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5;

    const int a_rows = (lmode == 2) ? kred : 128, a_cols = (lmode == 2) ? 128 : kred;
    const int b_rows = (lmode == 0) ? N : kred, b_cols = (lmode == 0) ? kred : N;
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
        // mode + 10 selects the compile-time shaped issue loops that the kernels use
        if (mode == 0) umma::gemm_kk(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, false, false), false);
        if (mode == 1) umma::gemm_km(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, false, true), false);
        if (mode == 2) umma::gemm_mm(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, true, true), false);
#define LLATTN_ST_CASE(NN, KK)                                                                                              \
        if (N == NN && kred == KK) {                                                                                        \
            if (tmode == 10) umma::gemm_kk<128, NN, KK>(tbase, a, b, umma::idesc_bf16(128, NN, false, false), false);       \
            if (tmode == 11) umma::gemm_km<128, KK, KK>(tbase, a, b, umma::idesc_bf16(128, NN, false, true), false);        \
            if (tmode == 12) umma::gemm_mm<KK, KK, KK>(tbase, a, b, umma::idesc_bf16(128, NN, true, true), false);          \
        }
        LLATTN_ST_CASE(64, 64)
        LLATTN_ST_CASE(64, 128)
        LLATTN_ST_CASE(128, 64)
        LLATTN_ST_CASE(128, 128)
#undef LLATTN_ST_CASE
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

// Issue-to-completion time of `reps` back-to-back products of one layout combination (operands already in
// shared memory, accumulators in tensor memory): the per-instruction cost that the kernel designs assume.
// issuers = 2: warps 0 and 1 each issue `reps` products into their own accumulator at the same time.
// Dynamic shared memory: 64 KB of operands (modes 0..2) or 128 KB (modes 3, 4, whose B tile has 256-row panels:
// the chain reads up to byte 32768 + 32768 + 128 * 128 of it).
__global__ void __launch_bounds__(128, 1) umma_cycles_kernel(int N, int kred, int mode, int reps, int issuers, int smem_bytes,
                                                             long long* __restrict__ cycles, int* __restrict__ err) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = smem;
    unsigned char* sB = smem + 32768;
    __shared__ uint64_t bar[2];
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int e = tid; e < smem_bytes / 4; e += 128) reinterpret_cast<uint32_t*>(smem)[e] = 0x3c003c00u;     // small finite bf16 pairs
    if (warp == 0) umma::tmem_alloc(&tmem_slot, 256);
    if (tid == 0) {
        umma::mbar_init(&bar[0], 1);
        umma::mbar_init(&bar[1], 1);
        umma::fence_mbar_init();
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tbase = tmem_slot + (warp == 1 ? 128 : 0);
    const long long t0 = clock64();
    if (lane == 0 && warp < (issuers % 10)) {
        const uint32_t a = umma::smem_addr(sA), b = umma::smem_addr(sB);
        const int a_rows = (mode == 2) ? kred : 128, b_rows = (mode == 0) ? N : kred;
        // the compile-time shaped issue loops of the kernels where one exists for the combination
        if (mode == 2 && N == 64 && kred == 64) {
            // the second batch of the reverse-order backward pass: seven chains of different layouts and widths
            // into different accumulators (36 instructions per repetition)
            const uint32_t t = tmem_slot;
            for (int r = 0; r < reps; ++r) {
                umma::gemm_mm<128, 128, 128>(t + 0, a, b, umma::idesc_bf16(128, 64, true, true), false);
                umma::gemm_km<128, 128, 128>(t + 64, b, a + 16384, umma::idesc_bf16(128, 64, false, true), false);
                umma::gemm_kk<128, 128, 64>(t + 128, a, b, umma::idesc_bf16(128, 128, false, false), false);
                umma::gemm_mm<128, 128, 64>(t + 0, b, a, umma::idesc_bf16(128, 64, true, true), false);
                umma::gemm_mm<128, 128, 64>(t + 64, b + 8192, a + 8192, umma::idesc_bf16(128, 64, true, true), false);
                umma::gemm_mm<128, 128, 128>(t + 128, a, b + 16384, umma::idesc_bf16(128, 64, true, true), false);
            }
        } else if (mode == 3) {
            // the chains of the Gated DeltaNet scans: narrow accumulators (N = 32 per level, adjacent levels in one chain)
            // from a 256-row K-major B tile, and the MN-major A form with a 64-token reduction
            for (int r = 0; r < reps; ++r) umma::gemm_kk<128, 256, 128>(tbase, a, b, umma::idesc_bf16(128, N, false, false), r > 0);
        } else if (mode == 4) {
            for (int r = 0; r < reps; ++r) umma::gemm_mk<64, 256, 64>(tbase, a, b, umma::idesc_bf16(128, N, true, false), r > 0);
        } else if (mode == 0 && N == 128 && kred == 128) {
            for (int r = 0; r < reps; ++r) umma::gemm_kk<128, 128, 128>(tbase, a, b, umma::idesc_bf16(128, 128, false, false), r > 0);
        } else if (mode == 0 && N == 128 && kred == 64) {
            for (int r = 0; r < reps; ++r) umma::gemm_kk<128, 128, 64>(tbase, a, b, umma::idesc_bf16(128, 128, false, false), r > 0);
        } else if (mode == 1 && N == 64 && kred == 128) {
            for (int r = 0; r < reps; ++r) umma::gemm_km<128, 128, 128>(tbase, a, b, umma::idesc_bf16(128, 64, false, true), r > 0);
        } else if (mode == 2 && N == 64 && kred == 128) {
            for (int r = 0; r < reps; ++r) umma::gemm_mm<128, 128, 128>(tbase, a, b, umma::idesc_bf16(128, 64, true, true), r > 0);
        } else if (mode == 2 && N == 128 && kred == 128) {
            for (int r = 0; r < reps; ++r) umma::gemm_mm<128, 128, 128>(tbase, a, b, umma::idesc_bf16(128, 128, true, true), r > 0);
        } else {
            for (int r = 0; r < reps; ++r) {
                if (mode == 0) umma::gemm_kk(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, false, false), r > 0);
                if (mode == 1) umma::gemm_km(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, false, true), r > 0);
                if (mode == 2) umma::gemm_mm(tbase, a, a_rows, b, b_rows, kred, umma::idesc_bf16(128, N, true, true), r > 0);
            }
        }
        umma::commit(&bar[warp]);
    }
    // issuers >= 10: every thread of the CTA waits on the completion barrier while the products run
    // (what the element-wise warps of the kernels do), instead of thread 0 alone
    if (tid == 0 || issuers >= 10) {
        bool ok = umma::mbar_wait(&bar[0], 0);
        if ((issuers % 10) > 1) ok = umma::mbar_wait(&bar[1], 0) && ok;
        const long long t1 = clock64();
        if (tid == 0) *cycles = t1 - t0;
        if (!ok) atomicExch(err, 1);
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem_slot, 256);
}

}  // namespace llattn

namespace llattn {
// waits on a barrier that never completes; gives up after `limit` polls and reports like the production kernels
__global__ void wait_timeout_kernel(uint32_t limit, int* status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        umma::mbar_init(&bar, 1);
        umma::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !umma::mbar_wait(&bar, 0, limit)) atomicExch(status, 1);
}
}  // namespace llattn

extern "C" int llattn_selftest_umma_cycles(int N, int kred, int mode, int reps, int issuers, long long* cycles, int* err_flag,
                                           void* stream) {
    if (!cycles || !err_flag) return LLATTN_ERR_NULL;
    if (!(kred == 64 || kred == 128) || mode < 0 || mode > 4 || reps < 1 || reps > 4096 ||
        !(issuers == 1 || issuers == 2 || issuers == 11 || issuers == 12))
        return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (mode <= 2 ? !(N == 64 || N == 128) : !(N >= 32 && N <= 128 && N % 32 == 0)) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    const int operand_bytes = mode >= 3 ? 131072 : 65536;
    const size_t sm = (size_t)operand_bytes + 1024;
    cudaError_t e = cudaFuncSetAttribute(llattn::umma_cycles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    llattn::umma_cycles_kernel<<<1, 128, sm, (cudaStream_t)stream>>>(N, kred, mode, reps, issuers, operand_bytes, cycles, err_flag); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

extern "C" int llattn_selftest_umma(const void* A, const void* B, float* D, int N, int kred, int mode, int* err_flag,
                                    void* stream) {
    if (!A || !B || !D || !err_flag) return LLATTN_ERR_NULL;
    if (!(N == 64 || N == 128) || !(kred == 64 || kred == 128) || !((mode >= 0 && mode <= 2) || (mode >= 10 && mode <= 12)))
        return LLATTN_ERR_UNSUPPORTED_SHAPE;
    const size_t sm = (mode >= 10 ? 131072 + 49152 + 32768 : 65536) + 1024;
    cudaError_t e = cudaFuncSetAttribute(llattn::umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    llattn::umma_selftest_kernel<<<1, 128, sm, (cudaStream_t)stream>>>((const llattn::bf16*)A, (const llattn::bf16*)B, D, N, kred,
                                                                        mode, err_flag); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

extern "C" int llattn_selftest_wait_timeout(int spin_limit, int* status_dev, void* stream) {
    if (!status_dev) return LLATTN_ERR_NULL;
    const unsigned limit = spin_limit < 1 ? 1u : (spin_limit > (1 << 20) ? (1u << 20) : (unsigned)spin_limit);
    llattn::wait_timeout_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit, status_dev); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

// ---- element-wise phase micro-benchmark: the fp32 block product of the triangular inverses (256 threads, each one row x
// eight columns of a 32 x 32 x 32 product from shared memory), timed with clock64() around `reps` executions of COPIES copies
// of its code.  (The operand pointers are chosen at run time between a static and a dynamic allocation, so the compiler cannot
// drop the stores of the results as dead, which it does when they go to a static array nothing reads.)  `env` adds features of the production kernels' environment one at a time:
//   bit 0: the operands sit in a 160 KB dynamic shared-memory allocation (200 KB with the static arrays)
//   bit 1: the CTA holds all 512 tensor-memory columns meanwhile
//   bit 2: one thread of warp 8 polls an mbarrier with try_wait (as the MMA-issuing thread does) instead of a plain flag
//   `spin_warps` (0..4) warps beyond the eight working ones poll while the loop runs.
namespace llattn {
template <int COPIES>
__global__ void __launch_bounds__(384, 1) ew_product_cycles_kernel(int reps, int spin_warps, int env, long long* __restrict__ cycles,
                                                                   float* __restrict__ sink) {
    constexpr int LDA = 68, BS = 32;
    extern __shared__ unsigned char dyn_raw[];
    __shared__ float stA[64 * LDA], stX[64 * LDA], stT[32 * 32];
    __shared__ volatile int flag;
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float *sA = stA, *sX = stX, *sT = stT;
    if (env & 1) {
        unsigned char* dyn = umma::align_1024(dyn_raw);
        sA = reinterpret_cast<float*>(dyn + 65536);
        sX = reinterpret_cast<float*>(dyn + 102400);
        sT = reinterpret_cast<float*>(dyn + 102400 + 128 * LDA * 4);
    }
    for (int e = tid; e < 64 * LDA; e += 384) {
        sA[e] = 0.001f * (e % 97);
        sX[e] = 0.002f * (e % 89);
    }
    if (tid == 0) {
        flag = 0;
        umma::mbar_init(&bar, 1);
        umma::fence_mbar_init();
    }
    if ((env & 2) && warp == 8) umma::tmem_alloc(&tmem_slot, 512);
    __syncthreads();
    if (warp >= 8) {
        if (warp - 8 < spin_warps) {
            if ((env & 4) && warp == 8) {
                if (lane == 0) umma::mbar_wait(&bar, 0);                     // bounded; completed when the timed loop ends
            } else {
                for (unsigned it = 0; it < (1u << 24) && flag == 0; ++it) {  // bounded: the flag is set when the timed loop ends
                }
            }
        }
        if ((env & 2) && warp == 8) {
            for (unsigned it = 0; it < (1u << 24) && flag == 0; ++it) {
            }
            __syncwarp();
            umma::tmem_dealloc(tmem_slot, 512);
        }
        return;
    }
    float total = 0.f;
    asm volatile("bar.sync 2, 256;\n" ::: "memory");
    const long long t0 = clock64();
    for (int rep = 0; rep < reps; ++rep) {
#pragma unroll
        for (int copy = 0; copy < COPIES; ++copy) {
            const int cq = (tid + copy) & 3, r = (tid >> 2) & 31, m = tid >> 7;
            const float* Mrow = sA + (m * BS + r) * LDA;
            const float* Xc = sX + cq * 8;
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
            for (int k4 = 0; k4 < BS; k4 += 4) {
                const float4 mm = *reinterpret_cast<const float4*>(Mrow + k4);
                const float mv[4] = {mm.x, mm.y, mm.z, mm.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float4 x0 = *reinterpret_cast<const float4*>(Xc + (k4 + e) * LDA);
                    const float4 x1 = *reinterpret_cast<const float4*>(Xc + (k4 + e) * LDA + 4);
                    acc[0] += mv[e] * x0.x; acc[1] += mv[e] * x0.y; acc[2] += mv[e] * x0.z; acc[3] += mv[e] * x0.w;
                    acc[4] += mv[e] * x1.x; acc[5] += mv[e] * x1.y; acc[6] += mv[e] * x1.z; acc[7] += mv[e] * x1.w;
                }
            }
            float* T = sT + (r * BS + cq * 8) % (32 * 32 - 8);
            *reinterpret_cast<float4*>(T) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4*>(T + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            total += acc[0] + acc[7];
            asm volatile("bar.sync 2, 256;\n" ::: "memory");
        }
    }
    const long long t1 = clock64();
    if (tid == 0) {
        cycles[0] = t1 - t0;
        flag = 1;
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(&bar)) : "memory");
    }
    sink[tid] = total;
}
}  // namespace llattn

extern "C" int llattn_selftest_ew_cycles(int reps, int spin_warps, int copies, int env, long long* cycles, float* sink, void* stream) {
    if (!cycles || !sink || reps < 1 || reps > 4096 || spin_warps < 0 || spin_warps > 4 || env < 0 || env > 7) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if ((env & 4) && spin_warps < 1) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sm = (env & 1) ? 160 * 1024 + 1024 : 0;
    cudaError_t e;
#define LLATTN_EW_CASE(C)                                                                                                     \
    if (copies == C) {                                                                                                        \
        if ((e = cudaFuncSetAttribute(llattn::ew_product_cycles_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                      160 * 1024 + 1024)) != cudaSuccess)                                                     \
            return (int)e;                                                                                                    \
        llattn::ew_product_cycles_kernel<C><<<1, 384, sm, st>>>(reps, spin_warps, env, cycles, sink);                         \
        LLATTN_LAUNCHED();                                                                                                    \
        return (int)cudaGetLastError();                                                                                       \
    }
    LLATTN_EW_CASE(1)
    LLATTN_EW_CASE(64)
#undef LLATTN_EW_CASE
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}
