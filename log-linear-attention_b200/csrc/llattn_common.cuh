// Shared device helpers for the log-linear attention kernels (sm_100a).
//
// Conventions used by every kernel in this directory
//   * tensors are contiguous, "sequence first": q,k (B,T,G,K) bf16; v,o,do (B,T,H,V) bf16;
//     g (B,T,H) fp32; lambda (B,T,H,L) bf16; head h reads q/k group h / (H/G).
//   * a chunk is CH = 64 tokens; a segment is 2^MLOW consecutive chunks.  Fenwick levels whose
//     period fits inside a segment ("low" levels) are kept on chip by the chunk kernels; the
//     remaining ("high") levels are handled at segment granularity by the seg_* kernels.
//   * shared-memory tiles are row major with 8 elements (16 bytes) of padding per row so that
//     ldmatrix is bank-conflict free.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch_count.h"

namespace llattn {

constexpr int CH = 64;        // chunk length (the reference fixes 64, hattention/kernel.py:355-356)
constexpr int PAD = 8;        // bf16 elements of row padding in shared memory
constexpr int INTRA_LEVELS = 7;   // levels 0..6 live inside a 64-token chunk (bit_length(i^j), i,j<64)
constexpr int MAX_L = 32;

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- async copies (16 bytes)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem_dst)), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// copy a ROWS x COLS bf16 tile (COLS multiple of 8) from global (row stride g_stride elements)
// into padded shared memory (row stride COLS + PAD)
template <int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void load_tile_async(bf16* s, const bf16* g, long g_stride, int tid) {
    constexpr int CPR = COLS / 8;
    constexpr int TOTAL = ROWS * CPR;
#pragma unroll
    for (int i = tid; i < TOTAL; i += NTHREADS) {
        int r = i / CPR, c = (i % CPR) * 8;
        cp_async16(s + r * (COLS + PAD) + c, g + (long)r * g_stride + c);
    }
}

// ---------------------------------------------------------------- warp-level MMA (bf16, fp32 acc)
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const bf16* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const bf16* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc[(16*MT) x (16*NP)] += A[(16*MT) x kred] * B[kred x (16*NP)]   for one warp.
//   A_T == false : A stored [m][k] (k contiguous), row stride lda, tile origin (row a0, k 0)
//   A_T == true  : A stored [k][m] (m contiguous), row stride lda, tile origin (k 0, col a0)
//   B_T == false : B stored [n][k] (k contiguous), row stride ldb, tile origin (row b0, k 0)
//   B_T == true  : B stored [k][n] (n contiguous), row stride ldb, tile origin (k 0, col b0)
// acc[mt][nt][e] follows the m16n8 accumulator fragment: rows mt*16 + lane/4 (+8 for e>=2),
// cols nt*8 + 2*(lane%4) + (e&1).
template <int MT, int NP, bool A_T, bool B_T>
__device__ __forceinline__ void warp_gemm(float (&acc)[MT][2 * NP][4], const bf16* A, int lda, int a0,
                                          const bf16* B, int ldb, int b0, int kred, int lane) {
    const int l8 = lane & 7, lq = (lane >> 3) & 1, lh = lane >> 4;
    for (int kk = 0; kk < kred; kk += 16) {
        uint32_t af[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            if (!A_T) {
                ldsm_x4(af[mt], A + (a0 + mt * 16 + l8 + lq * 8) * lda + kk + lh * 8);
            } else {
                ldsm_x4_t(af[mt], A + (kk + l8 + lh * 8) * lda + a0 + mt * 16 + lq * 8);
            }
        }
#pragma unroll
        for (int np = 0; np < NP; ++np) {
            uint32_t bfr[4];
            if (!B_T) {
                ldsm_x4(bfr, B + (b0 + np * 16 + l8 + lh * 8) * ldb + kk + lq * 8);
            } else {
                ldsm_x4_t(bfr, B + (kk + l8 + lq * 8) * ldb + b0 + np * 16 + lh * 8);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma16816(acc[mt][2 * np], af[mt], bfr[0], bfr[1]);
                mma16816(acc[mt][2 * np + 1], af[mt], bfr[2], bfr[3]);
            }
        }
    }
}

template <int MT, int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[MT][NT][4]) {
#pragma unroll
    for (int a = 0; a < MT; ++a)
#pragma unroll
        for (int b = 0; b < NT; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[a][b][e] = 0.f;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// exp(x) for x <= 0 (and 0 for x > 0 never arises in causal positions; callers mask)
__device__ __forceinline__ float fexp(float x) { return __expf(x); }

// Fenwick bucket of (target i, source j), j <= i: bit_length(i ^ j).  Equals the reference's
// recursive get_level_index_weak (hattention/base.py:41-46) and its T x T lookup table.
__device__ __forceinline__ int level_of(int i, int j) { return 32 - __clz(i ^ j); }

// inclusive scan of 64 floats held two per lane (elements 2*lane, 2*lane+1) by one warp
__device__ __forceinline__ void warp_cumsum64(float& x0, float& x1, int lane) {
    x1 += x0;
    float s = x1;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        float t = __shfl_up_sync(0xffffffffu, s, d);
        if (lane >= d) s += t;
    }
    float prev = s - x1;
    x0 += prev;
    x1 = s;
}

__device__ __forceinline__ void red_add_f32(float* addr, float v) {
    asm volatile("red.global.add.f32 [%0], %1;\n" ::"l"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add_f32x2(float* addr, float a, float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};\n" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

}  // namespace llattn
