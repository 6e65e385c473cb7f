// Blackwell (sm_100a) 5th-generation tensor core helpers: tcgen05.mma with shared-memory operand
// descriptors, tensor memory (TMEM) allocation and readback, mbarrier completion tracking.
//
// Shared-memory operand tiles use ONE physical layout everywhere: a tile of R rows x C bf16
// columns is stored as C/64 "panels"; a panel is R rows of 128 bytes (64 bf16) and is 128-byte
// swizzled (16-byte chunk index XOR (row & 7)); panels are 1024-byte aligned.  This is what a TMA
// box of 64 columns with SWIZZLE_128B produces, and the same bytes serve as
//   * a K-major operand  (MMA's M/N index = row, reduction index = column), and
//   * an MN-major operand (MMA's M/N index = column, reduction index = row).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace llattn {
namespace umma {

constexpr int PANEL_COLS = 64;          // bf16 elements per 128-byte row
constexpr int ROW_BYTES = 128;
constexpr uint32_t SPIN_LIMIT = 1u << 20;   // bounded waits: give up and flag instead of hanging

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// First 1024-byte boundary inside a dynamic shared-memory array, formed by pointer arithmetic on the array itself.
__device__ __forceinline__ unsigned char* align_1024(unsigned char* shared_array) {
    return shared_array + ((1024u - (smem_addr(shared_array) & 1023u)) & 1023u);
}

// byte offset of element (row, col) inside a tile of `rows` rows stored as 64-column panels
__device__ __forceinline__ uint32_t tile_offset(int row, int col, int rows) {
    const int panel = col >> 6, c = col & 63;
    const int chunk = (c >> 3) ^ (row & 7);
    return (uint32_t)(panel * rows * ROW_BYTES + row * ROW_BYTES + chunk * 16 + (c & 7) * 2);
}

// ---- shared memory matrix descriptors (SWIZZLE_128B, sm_100 version field = 1)
// The upper 32 bits are the same for every operand of these kernels: stride offset 1024 bytes (8-row groups),
// descriptor version 1 (bit 46), swizzle mode 128 B (bits 61..63 = 2).  Only the lower word differs: start
// address >> 4 in bits 0..13 and the leading offset >> 4 in bits 16..29.  The issue loops therefore carry one
// 32-bit register per operand and add compile-time offsets to it; the 64-bit descriptor is assembled inside
// the instruction's asm block (fewer live registers in the issuing warp, one add per operand and step).
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
// K-major: 8-row groups are 1024 bytes apart; the leading-dimension field is unused with swizzle
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1u << 16); }
// MN-major: consecutive 64-element blocks of the M/N index are `panel_bytes` apart (leading
// offset), consecutive 8-row groups of the reduction index are 1024 bytes apart (stride offset)
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t saddr, uint32_t panel_bytes) {
    return ((saddr >> 4) & 0x3FFFu) | (((panel_bytes >> 4) & 0x3FFFu) << 16);
}

// ---- instruction descriptor: bf16 x bf16 -> fp32, dense
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) |
           (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_desc_lo, uint32_t b_desc_lo, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_desc_lo), "r"(b_desc_lo), "r"(idesc), "r"((uint32_t)accumulate), "r"(DESC_HI)
        : "memory");
}
// A operand from tensor memory (bf16 pairs packed in 32-bit columns), B from shared memory
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_desc_lo, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %4, 0;\n\tmov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_desc_lo), "r"(idesc), "r"((uint32_t)accumulate), "r"(DESC_HI)
        : "memory");
}

// The three operand-layout combinations.  Tile row counts and the reduction length are template
// parameters so that every descriptor is "base + constant"; the start-address field occupies the
// low 14 bits (16-byte units) and shared memory addresses stay below 256 KB, so adding a byte
// offset >> 4 to the 64-bit descriptor never carries into another field.
//
// D[128 x N] (+)= A[128 x KRED] * B[N x KRED]^T : both operands K-major tiles (rows = M / N index)
template <int A_ROWS, int B_ROWS, int KRED>
__device__ __forceinline__ void gemm_kk(uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr, uint32_t idesc, bool accumulate) {
    const uint32_t da = desc_lo_kmajor(a_saddr), db = desc_lo_kmajor(b_saddr);
#pragma unroll
    for (int kk = 0; kk < KRED; kk += 16) {
        const uint32_t ka = (kk >> 6) * A_ROWS * ROW_BYTES + (kk & 63) * 2;
        const uint32_t kb = (kk >> 6) * B_ROWS * ROW_BYTES + (kk & 63) * 2;
        mma_ss(d_tmem, da + (ka >> 4), db + (kb >> 4), idesc, accumulate || kk > 0);
    }
}
// A K-major tile (rows = M index), B stored [KRED rows][N cols] (MN-major)
template <int A_ROWS, int B_ROWS, int KRED>
__device__ __forceinline__ void gemm_km(uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr, uint32_t idesc, bool accumulate) {
    const uint32_t da = desc_lo_kmajor(a_saddr), db = desc_lo_mnmajor(b_saddr, B_ROWS * ROW_BYTES);
#pragma unroll
    for (int kk = 0; kk < KRED; kk += 16) {
        const uint32_t ka = (kk >> 6) * A_ROWS * ROW_BYTES + (kk & 63) * 2;
        mma_ss(d_tmem, da + (ka >> 4), db + ((kk * ROW_BYTES) >> 4), idesc, accumulate || kk > 0);
    }
}
// A stored [KRED rows][M cols], B stored [KRED rows][N cols] (both MN-major): D = A^T B
template <int A_ROWS, int B_ROWS, int KRED>
__device__ __forceinline__ void gemm_mm(uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr, uint32_t idesc, bool accumulate) {
    const uint32_t da = desc_lo_mnmajor(a_saddr, A_ROWS * ROW_BYTES), db = desc_lo_mnmajor(b_saddr, B_ROWS * ROW_BYTES);
#pragma unroll
    for (int kk = 0; kk < KRED; kk += 16) {
        mma_ss(d_tmem, da + ((kk * ROW_BYTES) >> 4), db + ((kk * ROW_BYTES) >> 4), idesc, accumulate || kk > 0);
    }
}
// A stored [KRED rows][M cols] (MN-major), B a K-major tile (rows = N index): D = A^T B^T
template <int A_ROWS, int B_ROWS, int KRED>
__device__ __forceinline__ void gemm_mk(uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr, uint32_t idesc, bool accumulate) {
    const uint32_t da = desc_lo_mnmajor(a_saddr, A_ROWS * ROW_BYTES), db = desc_lo_kmajor(b_saddr);
#pragma unroll
    for (int kk = 0; kk < KRED; kk += 16) {
        const uint32_t kb = (kk >> 6) * B_ROWS * ROW_BYTES + (kk & 63) * 2;
        mma_ss(d_tmem, da + ((kk * ROW_BYTES) >> 4), db + (kb >> 4), idesc, accumulate || kk > 0);
    }
}
// run-time sized variants (self-test)
__device__ __forceinline__ void gemm_kk(uint32_t d_tmem, uint32_t a_saddr, int a_rows, uint32_t b_saddr, int b_rows,
                                        int kred, uint32_t idesc, bool accumulate) {
    for (int kk = 0; kk < kred; kk += 16) {
        const uint32_t ka = (kk >> 6) * a_rows * ROW_BYTES + (kk & 63) * 2;
        const uint32_t kb = (kk >> 6) * b_rows * ROW_BYTES + (kk & 63) * 2;
        mma_ss(d_tmem, desc_lo_kmajor(a_saddr + ka), desc_lo_kmajor(b_saddr + kb), idesc, accumulate || kk > 0);
    }
}
__device__ __forceinline__ void gemm_km(uint32_t d_tmem, uint32_t a_saddr, int a_rows, uint32_t b_saddr, int b_rows,
                                        int kred, uint32_t idesc, bool accumulate) {
    for (int kk = 0; kk < kred; kk += 16) {
        const uint32_t ka = (kk >> 6) * a_rows * ROW_BYTES + (kk & 63) * 2;
        mma_ss(d_tmem, desc_lo_kmajor(a_saddr + ka), desc_lo_mnmajor(b_saddr + kk * ROW_BYTES, b_rows * ROW_BYTES), idesc,
               accumulate || kk > 0);
    }
}
__device__ __forceinline__ void gemm_mm(uint32_t d_tmem, uint32_t a_saddr, int a_rows, uint32_t b_saddr, int b_rows,
                                        int kred, uint32_t idesc, bool accumulate) {
    for (int kk = 0; kk < kred; kk += 16) {
        mma_ss(d_tmem, desc_lo_mnmajor(a_saddr + kk * ROW_BYTES, a_rows * ROW_BYTES),
               desc_lo_mnmajor(b_saddr + kk * ROW_BYTES, b_rows * ROW_BYTES), idesc, accumulate || kk > 0);
    }
}

// ---- completion tracking
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
// arrive on `bar` when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
// bounded wait; returns false if the phase did not complete within the spin limit, or at once if
// another thread of the CTA has already given up (*abort != 0); sets *abort on giving up
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
    const uint32_t a = smem_addr(bar);
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return true;
        if ((it & 255) == 255 && *abort) return false;
    }
    *abort = 1;
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = SPIN_LIMIT) {
    const uint32_t a = smem_addr(bar);
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// bounded wait for warps that have nothing else to do until the phase completes: sleeps between polls so that the
// polling does not compete with the tensor core's operand fetch from shared memory
__device__ __forceinline__ bool mbar_wait_backoff(uint64_t* bar, uint32_t parity, volatile int* abort, unsigned ns) {
    const uint32_t a = smem_addr(bar);
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(a), "r"(parity)
            : "memory");
        if (done) return true;
        if ((it & 255) == 255 && *abort) return false;
        __nanosleep(ns);
    }
    *abort = 1;
    return false;
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// make generic-proxy shared memory writes (st.shared, cp.async) visible to the tensor core's async proxy
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- tensor memory
// one full warp allocates `ncols` (power of two >= 32) columns and publishes the base address
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(slot_in_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
// 32 consecutive fp32 columns of this thread's lane (lane = 32 * (warp % 4) + laneid)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 16 consecutive fp32 columns of this thread's lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 16 consecutive fp32 columns, issue only: the destination registers are valid after tmem_ld_wait4 has named them
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// one wait for four 16-column loads in flight; every destination register is an operand so that no use of them can
// be scheduled above the wait
__device__ __forceinline__ void tmem_ld_wait4(uint32_t (&a)[16], uint32_t (&b)[16], uint32_t (&c)[16], uint32_t (&d)[16]) {
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;\n"
        : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]),
          "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]),
          "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]),
          "+r"(b[9]), "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]),
          "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]), "+r"(c[4]), "+r"(c[5]), "+r"(c[6]), "+r"(c[7]), "+r"(c[8]),
          "+r"(c[9]), "+r"(c[10]), "+r"(c[11]), "+r"(c[12]), "+r"(c[13]), "+r"(c[14]), "+r"(c[15]),
          "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]), "+r"(d[4]), "+r"(d[5]), "+r"(d[6]), "+r"(d[7]), "+r"(d[8]),
          "+r"(d[9]), "+r"(d[10]), "+r"(d[11]), "+r"(d[12]), "+r"(d[13]), "+r"(d[14]), "+r"(d[15])
        :
        : "memory");
}
// compiler-level completion point for one more 16-column load (after a wait that has already covered it in hardware,
// or on its own)
__device__ __forceinline__ void tmem_ld_wait1(uint32_t (&a)[16]) {
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;\n"
        : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]),
          "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15])
        :
        : "memory");
}
// 4 consecutive fp32 columns of this thread's lane
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float (&v)[4]) {
    uint32_t r[4];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]) : : "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
// two 16-column loads (e.g. the same columns of two accumulators) in flight together, one wait
__device__ __forceinline__ void tmem_ld16x2(uint32_t taddr_a, float (&a)[16], uint32_t taddr_b, float (&b)[16]) {
    uint32_t r[16], q[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr_a)
        : "memory");
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]), "=r"(q[8]),
          "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15])
        : "r"(taddr_b)
        : "memory");
    // the wait names every destination register as an operand so that no use of them can be scheduled above it
    asm volatile(
        "tcgen05.wait::ld.sync.aligned;\n"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
          "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(q[0]), "+r"(q[1]), "+r"(q[2]), "+r"(q[3]), "+r"(q[4]), "+r"(q[5]), "+r"(q[6]), "+r"(q[7]), "+r"(q[8]),
          "+r"(q[9]), "+r"(q[10]), "+r"(q[11]), "+r"(q[12]), "+r"(q[13]), "+r"(q[14]), "+r"(q[15])
        :
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = __uint_as_float(r[i]);
        b[i] = __uint_as_float(q[i]);
    }
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// 16 consecutive fp32 columns of this thread's lane (complete after tmem_wait_st)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// address of (lane quarter of this warp, column) relative to an allocation base
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int warp, int col) {
    return base + (uint32_t((warp & 3) * 32) << 16) + (uint32_t)col;
}

}  // namespace umma
}  // namespace llattn
