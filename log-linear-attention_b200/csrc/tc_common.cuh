// Pieces shared by the tcgen05 kernels of the log-linear Mamba-2 path: tile geometry, warp roles,
// CTA barriers, optional phase timing.
#pragma once
#include "llattn_common.cuh"
#include "llattn_mamba2.h"
#include "tma.cuh"
#include "umma.cuh"

namespace llattn {

// Optional phase timing for tuning (build with -DLLATTN_STAMPS): three threads of one CTA record
// clock64() at fixed points of one pair; llattn_debug_read_stamps copies the table to the host.
#ifdef LLATTN_STAMPS
static __device__ long long g_stamps[3][32];
#define STAMP()                                                             \
    do {                                                                    \
        if (stamp_slot >= 0 && nstamp < 32) g_stamps[stamp_slot][nstamp++] = clock64(); \
    } while (0)
#define STAMPR()                                                            \
    do {                                                                    \
        if (stamp_slot >= 0 && nstamp < 16) g_stamps[stamp_slot][16 + nstamp++] = clock64(); \
    } while (0)
#else
#define STAMP() do { } while (0)
#define STAMPR() do { } while (0)
#endif

namespace tc {
constexpr int KD = 128, VD = 64, PT = 128;          // pair of chunks = 128 tokens
constexpr uint32_t Q_BYTES = PT * KD * 2;            // 32 KB
constexpr uint32_t V_BYTES = PT * VD * 2;            // 16 KB
constexpr uint32_t H_BYTES = KD * VD * 2;            // 16 KB
// tensor memory columns
constexpr int TM_S = 0, TM_O = 128, TM_T0 = 192, TM_T1 = 256, TM_KV = 320, TM_COLS = 512;
// warps 0..7 do the element-wise work (two per tensor-memory lane quarter), warp 8 issues the MMAs;
// the CTA is launched with three warpgroups so that registers can be moved from the third to the
// first two (setmaxnreg); warps 9..11 exit at once
constexpr int NTHREADS = 384, MMA_WARP = 8;
constexpr int MAX_L_TC = 20;        // lambda levels supported by this kernel (T up to 64 * 2^13)
constexpr int LAM_LD = MAX_L + 2;   // row stride of the staged lambda tile: odd number of 32-bit words, no bank conflicts
}  // namespace tc


// CTA-wide barrier over the 8 element-wise warps and the MMA warp (the spare warps of the third
// warpgroup exit at once and never take part)
// Register hand-over between the third warpgroup (TMA producer, MMA issuer, two idle warps) and the two
// element-wise warpgroups.  The kernel is launched with 168 registers per thread (384 threads); what the third
// group gives up must cover what the other two take, otherwise setmaxnreg.inc waits for registers that never
// become free.  The check is on the values themselves, so an unbalanced pair does not compile.
template <int DEC, int INC>
struct RegisterSplit {
    static_assert(DEC % 8 == 0 && INC % 8 == 0 && DEC >= 24 && INC <= 256, "setmaxnreg takes multiples of 8 in [24, 256]");
    static_assert(128 * (168 - DEC) >= 256 * (INC - 168), "the register pool does not cover this split");
    __device__ static __forceinline__ void release() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(DEC)); }
    __device__ static __forceinline__ void acquire() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(INC)); }
};

// Hands a TMA-filled tile back to the producer from a thread that has read it with ld.shared.  The arrive must
// not be performed before those loads have returned (the producer would refill the tile under them), and
// nothing orders a plain arrive after earlier loads whose results are not used yet.  So the release is preceded,
// in program order and in the same asm block, by a shared-memory store whose VALUE is computed from every loaded
// word: the store cannot issue before the loads have delivered their data, and the arrive issues after it.
// `sink` is any 4-byte shared-memory word that nothing reads (one per thread or shared by all).
__device__ __forceinline__ void release_tile_after_loads(uint64_t* bar, uint32_t* sink, uint32_t digest_of_loaded_words) {
    asm volatile(
        "st.shared.u32 [%0], %1;\n\tmbarrier.arrive.shared::cta.b64 _, [%2];\n"
        ::"r"(umma::smem_addr(sink)), "r"(digest_of_loaded_words), "r"(umma::smem_addr(bar))
        : "memory");
}

__device__ __forceinline__ void bar_work() { asm volatile("bar.sync 1, 288;\n" ::: "memory"); }

// one 32-byte global store (a full sector per lane; two 16-byte stores of a thread that owns a row would touch every sector twice)
__device__ __forceinline__ void st_global_32B(void* dst, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                 ::"l"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

// barrier over the 8 element-wise warps only
__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 2, 256;\n" ::: "memory"); }

// g_stamps lives in one translation unit only
}  // namespace llattn
