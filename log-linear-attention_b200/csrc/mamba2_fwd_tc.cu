// Log-linear Mamba-2 chunk kernel on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory), K = 128, V = 64.  Same mathematics and same segment organisation as
// m2_chunk_fwd_kernel (mamba2_fwd.cu); the differences are the tile shapes:
//   * the CTA walks its segment in PAIRS of chunks (128 tokens) so that every product has M = 128:
//       S  = q k^T              128 x 128 x 128   (the 128 x 128 masked tile covers levels 0..7, i.e.
//                                                  the two intra-chunk blocks and chunk-level 0 between them)
//       O  = P v                128 x  64 x 128
//       T  = q H_level          128 x  64 x 128   per pair-level whose bit is set (chunk level >= 1)
//       KV = k^T (v * decay)    128 x  64 x 128   summary of the pair
//   * operands sit in 128-byte-swizzled shared memory tiles read directly by the tensor core;
//     the masks / decays / lambda weights are applied on the way from tensor memory to the bf16
//     P tile; level-state masters stay in registers in the tensor-memory readout layout (one
//     state row per thread), their bf16 copies are written once as MN-major operands.
#include "llattn_common.cuh"
#include "llattn_mamba2.h"
#include "umma.cuh"

namespace llattn {

namespace tc {
constexpr int KD = 128, VD = 64, PT = 128;          // pair of chunks = 128 tokens
constexpr uint32_t Q_BYTES = PT * KD * 2;            // 32 KB
constexpr uint32_t V_BYTES = PT * VD * 2;            // 16 KB
constexpr uint32_t H_BYTES = KD * VD * 2;            // 16 KB
// tensor memory columns
constexpr int TM_S = 0, TM_O = 128, TM_T0 = 192, TM_T1 = 256, TM_KV = 320, TM_COLS = 512;
}  // namespace tc

template <int MLOW>
struct FwdTcSmem {
    static constexpr int MP = MLOW - 1;              // pair levels kept on chip
    static constexpr uint32_t q_off = 0;                               // [2]
    static constexpr uint32_t v_off = q_off + 2 * tc::Q_BYTES;         // [2]
    static constexpr uint32_t k_off = v_off + 2 * tc::V_BYTES;
    static constexpr uint32_t p_off = k_off + tc::Q_BYTES;
    static constexpr uint32_t vs_off = p_off + tc::PT * tc::PT * 2;
    static constexpr uint32_t h_off = vs_off + tc::V_BYTES;
    static constexpr uint32_t gp_off = h_off + (MP > 0 ? MP : 1) * tc::H_BYTES;   // float [128]
    static constexpr uint32_t bar_off = gp_off + 128 * 4;              // 4 mbarriers + tmem slot + abort flag
    static constexpr uint32_t total = bar_off + 64 + 1024;             // + slack for 1024-byte alignment
};

// 128 x COLS bf16 tile from global (row stride g_stride elements) into the swizzled panel layout
template <int COLS>
__device__ __forceinline__ void load_tile_swz(unsigned char* s, const bf16* g, long g_stride, int tid) {
    constexpr int CPR = COLS / 8;
#pragma unroll
    for (int i = tid; i < tc::PT * CPR; i += 256) {
        const int r = i / CPR, c = (i % CPR) * 8;
        cp_async16(s + umma::tile_offset(r, c, tc::PT), g + (long)r * g_stride + c);
    }
}

template <int MLOW>
__global__ void __launch_bounds__(256, 1) m2_chunk_fwd_tc_kernel(const Mamba2Params p) {
    using SM = FwdTcSmem<MLOW>;
    constexpr int MP = SM::MP;
    constexpr int SEGP = 1 << MP;                    // pairs per segment
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = smem + SM::q_off;
    unsigned char* sV = smem + SM::v_off;
    unsigned char* sK = smem + SM::k_off;
    unsigned char* sP = smem + SM::p_off;
    unsigned char* sVs = smem + SM::vs_off;
    unsigned char* sH = smem + SM::h_off;
    float* sGp = reinterpret_cast<float*>(smem + SM::gp_off);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);     // S, T, O, KV
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 40);
    static_assert(MP <= 2, "two tensor-memory slots for level reads");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % p.NS;
    const int b = blockIdx.x / (p.H * p.NS);
    const int grp = h / (p.H / p.G);
    const int L = p.L;
    const int npairs = min(SEGP, p.NT / 2 - r * SEGP);
    const bool hi_init = (p.o_has_high != 0) && (r != 0);
    const int row = (warp & 3) * 32 + lane;          // tensor-memory lane of this thread
    const int ch = warp >> 2;                        // which half of the columns this thread handles

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) umma::mbar_init(&bars[i], 1);
        umma::fence_mbar_init();
        *abort_flag = *p.err;                        // an earlier CTA gave up: do not pile on
    }
    __syncthreads();
    if (*abort_flag) return;                         // uniform: every thread reads the same shared word
    if (warp == 0) umma::tmem_alloc(tmem_slot, tc::TM_COLS);
    auto issue_qv = [&](int pl, int st) {
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        load_tile_swz<tc::KD>(sQ + st * tc::Q_BYTES, p.q + (((long)b * p.T + t0) * p.G + grp) * tc::KD, (long)p.G * tc::KD, tid);
        load_tile_swz<tc::VD>(sV + st * tc::V_BYTES, p.v + (((long)b * p.T + t0) * p.H + h) * tc::VD, (long)p.H * tc::VD, tid);
        cp_async_commit();
    };
    auto issue_k = [&](int pl) {
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        load_tile_swz<tc::KD>(sK, p.k + (((long)b * p.T + t0) * p.G + grp) * tc::KD, (long)p.G * tc::KD, tid);
        cp_async_commit();
    };
    issue_qv(0, 0);
    issue_k(0);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;

    float M[MP > 0 ? MP : 1][32];     // masters: row `row` of each low pair-level state, 32 columns
    float dsum[MP > 0 ? MP : 1];
#pragma unroll
    for (int i = 0; i < (MP > 0 ? MP : 1); ++i) dsum[i] = 0.f;
    uint32_t phS = 0, phT = 0, phO = 0, phKV = 0;
    bool ok = true;

    constexpr uint32_t ID_S = umma::idesc_bf16(128, 128, false, false);
    constexpr uint32_t ID_KM = umma::idesc_bf16(128, 64, false, true);
    constexpr uint32_t ID_MM = umma::idesc_bf16(128, 64, true, true);

    for (int pl = 0; pl < npairs; ++pl) {
        const int st = pl & 1;
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        // lambda of this thread's row: levels 0..7 (inside the pair) and the low pair levels
        float lam[8 + (MP > 0 ? MP : 1)];
        {
            const bf16* lp = p.l + (((long)b * p.T + t0 + row) * p.H + h) * L;
#pragma unroll
            for (int i = 0; i < 8 + MP; ++i) lam[i] = (i < L) ? __bfloat162float(lp[i]) : 0.f;
        }
        cp_async_wait<0>();
        if (pl + 1 < npairs) issue_qv(pl + 1, st ^ 1);
        // in-chunk cumulative sums of g (output) and the pair-wide cumulative sum
        if (warp < 2) {
            const float* gp = p.g + ((long)b * p.T + t0 + warp * CH) * p.H + h;
            float x0 = gp[(long)(2 * lane) * p.H], x1 = gp[(long)(2 * lane + 1) * p.H];
            warp_cumsum64(x0, x1, lane);
            float* gc = p.g_cum + ((long)b * p.T + t0 + warp * CH) * p.H + h;
            gc[(long)(2 * lane) * p.H] = x0;
            gc[(long)(2 * lane + 1) * p.H] = x1;
            sGp[warp * CH + 2 * lane] = x0;
            sGp[warp * CH + 2 * lane + 1] = x1;
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        __syncthreads();
        umma::fence_after_sync();
        const uint32_t aQ = umma::smem_addr(sQ + st * tc::Q_BYTES), aK = umma::smem_addr(sK);
        const uint32_t aV = umma::smem_addr(sV + st * tc::V_BYTES);
        int nread = 0;
#pragma unroll
        for (int lv = 0; lv < MP; ++lv) nread += (pl >> lv) & 1;
        if (tid == 0) {
            umma::gemm_kk(tbase + tc::TM_S, aQ, tc::PT, aK, tc::PT, tc::KD, ID_S, false);
            umma::commit(&bars[0]);
            if (nread > 0) {
                int slot = 0;
#pragma unroll
                for (int lv = 0; lv < MP; ++lv)
                    if ((pl >> lv) & 1) {
                        umma::gemm_km(tbase + (slot == 0 ? tc::TM_T0 : tc::TM_T1), aQ, tc::PT,
                                      umma::smem_addr(sH + lv * tc::H_BYTES), tc::KD, tc::KD, ID_KM, false);
                        ++slot;
                    }
                umma::commit(&bars[1]);
            }
        }
        // pair-wide cumulative decay: second chunk continues from the end of the first
        const float gla = sGp[CH - 1];
        const float Gi = sGp[row] + (row >= CH ? gla : 0.f);
        const float glp = gla + sGp[2 * CH - 1];

        // ---- Vs = v * exp(glp - Gp_j)   (same swizzled offsets as v)
        {
            const unsigned char* cV = sV + st * tc::V_BYTES;
#pragma unroll
            for (int i = tid; i < tc::PT * (tc::VD / 8); i += 256) {
                const int j = i / (tc::VD / 8), c = (i % (tc::VD / 8)) * 8;
                const float sc = fexp(glp - (sGp[j] + (j >= CH ? gla : 0.f)));
                const uint32_t off = umma::tile_offset(j, c, tc::PT);
                uint4 x = *reinterpret_cast<const uint4*>(cV + off);
                uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v2 = *reinterpret_cast<__nv_bfloat162*>(&xw[e]);
                    xw[e] = pack_bf16(__bfloat162float(v2.x) * sc, __bfloat162float(v2.y) * sc);
                }
                *reinterpret_cast<uint4*>(sVs + off) = x;
            }
        }
        // ---- S -> P (bf16, K-major A operand of P v).  This thread: row `row`, 32-column blocks ch and ch+2
        ok = umma::mbar_wait(&bars[0], phS, abort_flag);
        phS ^= 1;
        umma::fence_after_sync();
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const int j0 = (ch + 2 * blk) * 32;
            uint32_t packed[16];
            if (j0 > row) {
#pragma unroll
                for (int e = 0; e < 16; ++e) packed[e] = 0u;
            } else {
                float s[32];
                umma::tmem_ld32(umma::tmem_addr(tbase + tc::TM_S, warp, j0), s);
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float pv[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int j = j0 + e + u;
                        float val = 0.f;
                        if (j <= row) {
                            const float Gj = sGp[j] + (j >= CH ? gla : 0.f);
                            const int lev = level_of(row, j);
                            float lm = lam[0];
#pragma unroll
                            for (int q = 1; q < 8; ++q) lm = (lev == q) ? lam[q] : lm;
                            val = s[e + u] * fexp(Gi - Gj) * lm;
                        }
                        pv[u] = val;
                    }
                    packed[e >> 1] = pack_bf16(pv[0], pv[1]);
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(sP + umma::tile_offset(row, j0 + c * 8, tc::PT)) =
                    make_uint4(packed[c * 4], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        __syncthreads();
        umma::fence_after_sync();
        if (tid == 0) {
            umma::gemm_km(tbase + tc::TM_O, umma::smem_addr(sP), tc::PT, aV, tc::PT, tc::PT, ID_KM, false);
            umma::commit(&bars[2]);
            umma::gemm_mm(tbase + tc::TM_KV, aK, tc::PT, umma::smem_addr(sVs), tc::PT, tc::PT, ID_MM, false);
            umma::commit(&bars[3]);
        }

        // ---- output row of this thread: columns ch*32 .. +31
        float o[32];
        bf16* go = p.o + (((long)b * p.T + t0 + row) * p.H + h) * tc::VD + ch * 32;
        if (hi_init) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 x = *reinterpret_cast<const uint4*>(go + c * 8);
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[e]);
                    o[c * 8 + e * 2] = __bfloat162float(v2.x);
                    o[c * 8 + e * 2 + 1] = __bfloat162float(v2.y);
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0.f;
        }
        if (nread > 0 && ok) {
            ok = umma::mbar_wait(&bars[1], phT, abort_flag);
            phT ^= 1;
            umma::fence_after_sync();
            int slot = 0;
#pragma unroll
            for (int lv = 0; lv < MP; ++lv)
                if ((pl >> lv) & 1) {
                    float t[32];
                    umma::tmem_ld32(umma::tmem_addr(tbase + (slot == 0 ? tc::TM_T0 : tc::TM_T1), warp, ch * 32), t);
                    const float rs = lam[8 + lv] * fexp(Gi + dsum[lv]);
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] += rs * t[e];
                    ++slot;
                }
        }
        if (ok) {
            ok = umma::mbar_wait(&bars[2], phO, abort_flag);
            phO ^= 1;
            umma::fence_after_sync();
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tc::TM_O, warp, ch * 32), t);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 x;
                uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) xw[e] = pack_bf16(o[c * 8 + e * 2] + t[c * 8 + e * 2], o[c * 8 + e * 2 + 1] + t[c * 8 + e * 2 + 1]);
                *reinterpret_cast<uint4*>(go + c * 8) = x;
            }
        }
        // ---- pair summary and the Fenwick carry over pair levels (thread = state row `row`)
        if (ok) {
            ok = umma::mbar_wait(&bars[3], phKV, abort_flag);
            phKV ^= 1;
            umma::fence_after_sync();
        }
        if (pl + 1 < npairs) issue_k(pl + 1);        // k tile is free once S and KV are done
        if (MP > 0 && pl + 1 < npairs && ok) {
            const int j = __ffs(~pl) - 1;
            if (j < MP) {
                float kv[32];
                umma::tmem_ld32(umma::tmem_addr(tbase + tc::TM_KV, warp, ch * 32), kv);
#pragma unroll
                for (int lv = 0; lv < MP; ++lv)
                    if (lv < j) {
                        const float dec = fexp(dsum[lv] + glp);
#pragma unroll
                        for (int e = 0; e < 32; ++e) kv[e] += dec * M[lv][e];
                    }
#pragma unroll
                for (int lv = 0; lv < MP; ++lv) {
                    if (lv == j) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) M[lv][e] = kv[e];
                        unsigned char* dst = sH + lv * tc::H_BYTES;
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            *reinterpret_cast<uint4*>(dst + umma::tile_offset(row, ch * 32 + c * 8, tc::KD)) =
                                make_uint4(pack_bf16(kv[c * 8], kv[c * 8 + 1]), pack_bf16(kv[c * 8 + 2], kv[c * 8 + 3]),
                                           pack_bf16(kv[c * 8 + 4], kv[c * 8 + 5]), pack_bf16(kv[c * 8 + 6], kv[c * 8 + 7]));
                        dsum[lv] = 0.f;
                    } else {
                        dsum[lv] += glp;
                    }
                }
            } else {
#pragma unroll
                for (int lv = 0; lv < MP; ++lv) dsum[lv] += glp;
            }
        }
        umma::fence_before_sync();
        __syncthreads();
        umma::fence_after_sync();
        if (*abort_flag) break;                      // uniform: read after the barrier
    }
    if (*abort_flag && tid == 0) atomicExch(p.err, 1);
    cp_async_wait<0>();
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tbase, tc::TM_COLS);
}

int mamba2_fwd_tc_launch(const Mamba2Params& p, cudaStream_t stream) {
    auto kern = m2_chunk_fwd_tc_kernel<M2_MLOW>;
    const size_t sm = FwdTcSmem<M2_MLOW>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    kern<<<p.B * p.H * p.NS, 256, sm, stream>>>(p);
    return (int)cudaGetLastError();
}

}  // namespace llattn
