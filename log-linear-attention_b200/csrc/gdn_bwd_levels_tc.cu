// Log-linear Gated DeltaNet backward: the chunk-parallel gradients that pair forward level states with their
// adjoints, on tcgen05 / TMEM / TMA (K = 128, V a multiple of 64).  Same mathematics as gdn_bwd_levels_kernel
// (gdn_bwd.cu); reference being replaced: hattention/chunkwise_hgdn.py:799-1010 (per level chunk_bwd_dqkwg and the
// state-dependent part of chunk_gated_delta_rule_bwd_dhu).
//
// For a chunk c, every level lv whose bit is set in c, H = the state the chunk reads and E = the adjoint of the
// state that H flows into (level lv above the carry jc, else the carry level), per 64-column half of V:
//     R = qd H,  Z = wd H,  KE = kd E                         (first batch: [qd; wd] H is one M = 128 product)
//     d lambda[i, lv] += sum_v do[i,v] R[i,v]
//     d_qd += (lambda_lv * do) H^T,  d_wd -= KE H^T            (second batch: [lambda do; KE] H^T is one M = 128 product)
//     d_kd -= Z E^T,  d_dec += <E, H>
// and once per half  d_kd += u E_jc^T,  d_u = kd E_jc.
// Persistent CTAs walk the (batch, chunk, head) items with a stride of the grid; inside an item the steps
// (half of V, level) are software pipelined: the tensor core works on the first batch of step s + 1 while the
// element-wise warps turn the results of step s into the operands of its second batch.  The three 64 x K results
// of an item accumulate in tensor memory across all its steps.
#include "tc_common.cuh"
#include "llattn_gdn.h"

namespace llattn {

namespace glt {
constexpr int KD = 128, NTHREADS = 384, MMA_WARP = 8;
constexpr uint32_t QW_BYTES = 128 * KD * 2;          // [qd; wd]: two panels of 128 rows
constexpr uint32_t KD_BYTES = CH * KD * 2;           // kd: two panels of 64 rows
constexpr uint32_t UV_BYTES = CH * 128 * 2;          // u or do of a chunk: up to two 64-column panels of 64 rows
constexpr uint32_t HE_BYTES = KD * 128;              // one [K][64] state tile (one panel of 128 rows)
constexpr uint32_t OP_BYTES = 128 * 128;             // [lambda do; KE]: one panel of 128 rows
constexpr uint32_t NZ_BYTES = CH * 128;              // -Z: one panel of 64 rows
// tensor memory columns
constexpr int TM_RZ = 0, TM_KE = 128, TM_QW = 256, TM_K = 384, TM_COLS = 512;   // RZ / KE double buffered (64 columns each)
constexpr int LSTRIDE = GDN_MAXLEV + 1;              // row stride of the staged lambda / d lambda tables (floats)
}  // namespace glt

struct LevTcSmem {
    static constexpr int NSTAGE = 3;                                            // state tiles in flight: the loads' latency exceeds a step
    static constexpr uint32_t qw_off = 0;
    static constexpr uint32_t kd_off = qw_off + glt::QW_BYTES;                  // the M = 128 read of kd runs into do (never used)
    static constexpr uint32_t do_off = kd_off + glt::KD_BYTES;
    static constexpr uint32_t he_off = do_off + glt::UV_BYTES;                  // [NSTAGE] x (H or u half | E)
    static constexpr uint32_t nz_off = he_off + NSTAGE * 2 * glt::HE_BYTES;     // [2]; the M = 128 read of the second one runs into op
    static constexpr uint32_t op_off = nz_off + 2 * glt::NZ_BYTES;              // [2]
    static constexpr uint32_t lam_off = op_off + 2 * glt::OP_BYTES;             // float [64][LSTRIDE]
    static constexpr uint32_t dl_off = lam_off + CH * glt::LSTRIDE * 4;         // float [2][64][LSTRIDE]
    static constexpr uint32_t red_off = dl_off + 2 * CH * glt::LSTRIDE * 4;     // float [16]
    static constexpr uint32_t rowt_off = red_off + 64;                          // float [4][64]: row terms of the decay gradient
    static constexpr uint32_t bar_off = (rowt_off + 4 * CH * 4 + 7) & ~7u;
    static constexpr uint32_t total = bar_off + 256 + 1024;
};
static_assert(LevTcSmem::total <= 232448, "shared memory of one CTA");

// One (half of V, level) step of an item.  level < 0 is the step of the chunk's own writes (u E_jc^T, d_u).
struct LevStep {
    int level, vh;
};

__device__ __forceinline__ LevStep lev_step(int s, int c, int per_half, bool trans, uint32_t live) {
    LevStep st;
    st.vh = s / per_half;
    int r = s - st.vh * per_half;
    st.level = -1;
    if (trans) {
        if (r == 0) return st;
        --r;
    }
    uint32_t m = live;
    for (int i = 0; i < r; ++i) m &= m - 1;
    st.level = __ffs(m) - 1;
    return st;
}

__global__ void __launch_bounds__(glt::NTHREADS, 1) gdn_bwd_levels_tc_kernel(const __grid_constant__ GdnParams p) {
    using SM = LevTcSmem;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQW = smem + SM::qw_off;
    unsigned char* sKd = smem + SM::kd_off;
    unsigned char* sDO = smem + SM::do_off;
    unsigned char* sHE = smem + SM::he_off;
    unsigned char* sOP = smem + SM::op_off;
    unsigned char* sNZ = smem + SM::nz_off;
    float* sLam = reinterpret_cast<float*>(smem + SM::lam_off);
    float* sDl = reinterpret_cast<float*>(smem + SM::dl_off);
    float* sRed = reinterpret_cast<float*>(smem + SM::red_off);
    float* sRowT = reinterpret_cast<float*>(smem + SM::rowt_off);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* fullC = bars + 0;      // chunk tiles (qd, wd, kd, u, do) landed
    uint64_t* emptyC = bars + 1;     // every product of the item is complete and the element-wise warps are done with do (256 arrivals)
    uint64_t* full = bars + 2;       // [3] state tiles of a step landed
    uint64_t* empty = bars + 5;      // [3] second batch of the step that used the stage complete
    uint64_t* barA = bars + 8;       // [2] first batch of a step complete
    uint64_t* barOp = bars + 10;     // [2] operands of the second batch written / first batch results consumed (256 arrivals)
    uint64_t* barB = bars + 12;      // [2] second batch of a step complete
    uint64_t* accFree = bars + 14;   // the item's results have left tensor memory (256 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 136);
    constexpr int NSTAGE = SM::NSTAGE;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nlev = p.NLEV, NT = p.NT, NVH = p.V / 64;
    const uint32_t lev_mask = (1u << nlev) - 1u;
    const int nitems = p.B * NT * p.H;
    const int npair = p.V / 64;                      // level-state tiles are stored per pair of 32-column slices

    if (tid == 0) {
        umma::mbar_init(fullC, 1);
        umma::mbar_init(emptyC, 256);
#pragma unroll
        for (int i = 2; i < 10; ++i) umma::mbar_init(&bars[i], 1);
        umma::mbar_init(&barOp[0], 256);
        umma::mbar_init(&barOp[1], 256);
        umma::mbar_init(&barB[0], 1);
        umma::mbar_init(&barB[1], 1);
        umma::mbar_init(accFree, 256);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    // row index (in units of K rows) of the [K][64] tile of (b, h, pair vp, chunk c, level lv) inside hs / dhs
    auto tile_row0 = [&](int b, int h, int vp, int c, int lv) -> int {
        return (int)((((((long)b * p.H + h) * npair + vp) * NT + c) * nlev + lv) * glt::KD);
    };

    if (warp >= glt::MMA_WARP) {
        if (warp == glt::MMA_WARP + 1) {
            // ---------------- TMA producer
            if (lane == 0) {
                uint32_t g = 0, nchunk = 0;
                for (int item = blockIdx.x; item < nitems; item += gridDim.x, ++nchunk) {
                    const int h = item % p.H, c = (item / p.H) % NT, b = item / (p.H * NT);
                    const bool trans = (c + 1 < NT);
                    const uint32_t live = (uint32_t)c & lev_mask;
                    const int jc = __ffs(~c) - 1;
                    const int per_half = __popc(live) + (trans ? 1 : 0);
                    const int nsteps = per_half * NVH;
                    if (nsteps == 0) continue;
                    if (nchunk > 0 && !umma::mbar_wait(emptyC, (nchunk - 1) & 1, abort_flag)) break;
                    const int row0 = b * p.T + c * CH;
                    tma::expect_tx(fullC, glt::QW_BYTES + glt::KD_BYTES + (uint32_t)NVH * CH * 128);
                    tma::load_panel(sQW, &p.tm_qd, 0, h, row0, fullC);
                    tma::load_panel(sQW + 128 * 128, &p.tm_qd, 64, h, row0, fullC);
                    tma::load_panel(sQW + 64 * 128, &p.tm_wd, 0, h, row0, fullC);
                    tma::load_panel(sQW + 128 * 128 + 64 * 128, &p.tm_wd, 64, h, row0, fullC);
                    tma::load_panel(sKd, &p.tm_kd, 0, h, row0, fullC);
                    tma::load_panel(sKd + CH * 128, &p.tm_kd, 64, h, row0, fullC);
                    for (int vh = 0; vh < NVH; ++vh) tma::load_panel(sDO + vh * CH * 128, &p.tm_do, vh * 64, h, row0, fullC);
                    bool ok = true;
                    for (int s = 0; s < nsteps && ok; ++s, ++g) {
                        const int st = g % NSTAGE;
                        if (g >= NSTAGE) ok = umma::mbar_wait(&empty[st], ((g / NSTAGE) - 1) & 1, abort_flag);
                        if (!ok) break;
                        const LevStep ls = lev_step(s, c, per_half, trans, live);
                        unsigned char* hT = sHE + st * 2 * glt::HE_BYTES;
                        unsigned char* eT = hT + glt::HE_BYTES;
                        tma::expect_tx(&full[st], (ls.level >= 0 ? glt::HE_BYTES : (uint32_t)CH * 128) + (trans ? glt::HE_BYTES : 0u));
                        if (ls.level >= 0) tma::load_panel(hT, &p.tm_hs, 0, 0, tile_row0(b, h, ls.vh, c, ls.level), &full[st]);
                        else tma::load_panel(hT, &p.tm_u, ls.vh * 64, h, row0, &full[st]);       // the chunk's own writes: this half of u takes the H slot
                        if (trans) {
                            const int le = (ls.level > jc) ? ls.level : jc;
                            tma::load_panel(eT, &p.tm_dhs, 0, 0, tile_row0(b, h, ls.vh, c, le), &full[st]);
                        }
                    }
                    if (!ok) break;
                }
            }
            return;
        }
        if (warp > glt::MMA_WARP) return;
        // ---------------- MMA issuer
        umma::tmem_alloc(tmem_slot, glt::TM_COLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        const uint32_t aQW = umma::smem_addr(sQW), aKd = umma::smem_addr(sKd);
        constexpr uint32_t ID_KM64 = umma::idesc_bf16(128, 64, false, true);
        constexpr uint32_t ID_KK128 = umma::idesc_bf16(128, 128, false, false);
        uint32_t g = 0, nchunk = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, ++nchunk) {
            const int c = (item / p.H) % NT;
            const bool trans = (c + 1 < NT);
            const uint32_t live = (uint32_t)c & lev_mask;
            const int per_half = __popc(live) + (trans ? 1 : 0);
            const int nsteps = per_half * NVH;
            if (nsteps == 0) continue;
            if (lane == 0) {
                ok = umma::mbar_wait(fullC, nchunk & 1, abort_flag);
                bool first_qw = true, first_k = true;
                // first batch of a step: [qd; wd] H and kd E into the step's result slots
                auto issue_first = [&](int s, uint32_t gs) -> bool {
                    const int st = gs % NSTAGE, tb = gs & 1;
                    if (!umma::mbar_wait(&full[st], (gs / NSTAGE) & 1, abort_flag)) return false;
                    umma::fence_after_sync();
                    const LevStep ls = lev_step(s, c, per_half, trans, live);
                    const uint32_t aH = umma::smem_addr(sHE + st * 2 * glt::HE_BYTES), aE = aH + glt::HE_BYTES;
                    if (ls.level >= 0) umma::gemm_km<128, glt::KD, glt::KD>(tbase + glt::TM_RZ + tb * 64, aQW, aH, ID_KM64, false);
                    if (trans) umma::gemm_km<CH, glt::KD, glt::KD>(tbase + glt::TM_KE + tb * 64, aKd, aE, ID_KM64, false);
                    umma::commit(&barA[tb]);
                    return true;
                };
#ifdef LLATTN_STAMPS
                int nstamp = 0;
                const int stamp_slot = (blockIdx.x == 5 && nchunk == 8) ? 2 : -1;
#endif
                if (ok) ok = issue_first(0, g);
                for (int s = 0; s < nsteps && ok; ++s, ++g) {
                    const int st = g % NSTAGE, tb = g & 1;
                    STAMP();                                 // m0 top of the step
                    if (s + 1 < nsteps) ok = issue_first(s + 1, g + 1);
                    STAMP();                                 // m1 first batch of the next step issued
                    if (ok) ok = umma::mbar_wait(&barOp[tb], (g >> 1) & 1, abort_flag);
                    if (!ok) break;
                    STAMP();                                 // m2 operands of this step ready
                    // the first second batch of an item overwrites the previous item's results
                    if (s == 0 && nchunk > 0 && !umma::mbar_wait(accFree, (nchunk - 1) & 1, abort_flag)) { ok = false; break; }
                    umma::fence_after_sync();
                    const LevStep ls = lev_step(s, c, per_half, trans, live);
                    const uint32_t aH = umma::smem_addr(sHE + st * 2 * glt::HE_BYTES), aE = aH + glt::HE_BYTES;
                    if (ls.level >= 0) {
                        // [lambda do; KE] H^T -> d_qd (rows 0..63), -d_wd (rows 64..127);  (-Z) E^T -> d_kd
                        umma::gemm_kk<128, glt::KD, CH>(tbase + glt::TM_QW, umma::smem_addr(sOP + tb * glt::OP_BYTES), aH, ID_KK128, !first_qw);
                        first_qw = false;
                        if (trans) {
                            umma::gemm_kk<CH, glt::KD, CH>(tbase + glt::TM_K, umma::smem_addr(sNZ + tb * glt::NZ_BYTES), aE, ID_KK128, !first_k);
                            first_k = false;
                        }
                    } else {
                        // u E_jc^T -> d_kd (this half of u sits in the stage's H slot)
                        umma::gemm_kk<CH, glt::KD, CH>(tbase + glt::TM_K, aH, aE, ID_KK128, !first_k);
                        first_k = false;
                    }
                    umma::commit(&barB[tb]);
                    umma::commit(&empty[st]);
                    STAMP();                                 // m3 second batch issued
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            g = __shfl_sync(0xffffffffu, g, 0);
        }
        if (lane == 0 && ok && g > 0) umma::mbar_wait(&barB[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag);
        __syncwarp();
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();
        umma::tmem_dealloc(tbase, glt::TM_COLS);
        return;
    }

    // ================= warps 0..7: element-wise =================
    const int rb = warp & 3, ch = warp >> 2;
    const int row = rb * 32 + lane;            // tensor-memory lane
    const bool qrow = rb < 2;                  // lanes 0..63: R / KE / d_qd / d_kd rows; lanes 64..127: Z / d_wd rows
    const int i = row & 63;                    // token of the chunk
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;
    uint32_t g = 0, nchunk = 0;
    bool alive = true;
    const bool fuse_rows = p.dqd_neg != nullptr && p.d_grow != nullptr;

    // lambda of an item's inter-chunk levels is requested one item ahead (a few values per thread) so that the loads'
    // latency is covered by the previous item's steps
    constexpr int LAMQ = (CH * glt::LSTRIDE + 255) / 256;
    __nv_bfloat16 lam_next[LAMQ];
    auto fetch_lambda = [&](int item) {
        const int h = item % p.H, c = (item / p.H) % NT, b = item / (p.H * NT);
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
#pragma unroll
        for (int q = 0; q < LAMQ; ++q) {
            const int e = tid + q * 256;
            const int r = e / glt::LSTRIDE, lv = e - r * glt::LSTRIDE;
            lam_next[q] = (e < CH * glt::LSTRIDE && lv < nlev) ? p.l[(rowbase + (long)r * p.H) * p.L + INTRA_LEVELS + lv] : __float2bfloat16(0.f);
        }
    };
    if ((int)blockIdx.x < nitems) fetch_lambda(blockIdx.x);

    for (int item = blockIdx.x; item < nitems && alive; item += gridDim.x) {
        const int h = item % p.H, c = (item / p.H) % NT, b = item / (p.H * NT);
        const bool trans = (c + 1 < NT);
        const uint32_t live = (uint32_t)c & lev_mask;
        const int per_half = __popc(live) + (trans ? 1 : 0);
        const int nsteps = per_half * NVH;
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
        float* gq = p.d_qd + (rowbase + (long)i * p.H) * glt::KD + ch * 64;
        float* gw = p.d_wd + (rowbase + (long)i * p.H) * glt::KD + ch * 64;
        float* gk = p.d_kd + (rowbase + (long)i * p.H) * glt::KD + ch * 64;
        if (nsteps == 0) {
            // a one-chunk sequence: no level states at all
#pragma unroll
            for (int e = 0; e < 64; e += 4) {
                if (qrow) {
                    *reinterpret_cast<float4*>(gq + e) = make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4*>(gk + e) = make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
                    *reinterpret_cast<float4*>(gw + e) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            for (int e = tid; e < CH * (p.V / 8); e += 256) {
                const int r = e / (p.V / 8), c8 = (e % (p.V / 8)) * 8;
                *reinterpret_cast<uint4*>(p.d_u + (rowbase + (long)r * p.H) * p.V + c8) = make_uint4(0u, 0u, 0u, 0u);
            }
            if (tid == 0) p.d_gl[((long)b * NT + c) * p.H + h] = 0.f;
            if (fuse_rows) {
                if (tid < CH) p.d_grow[rowbase + (long)tid * p.H] = 0.f;
                if (qrow) {
#pragma unroll
                    for (int e = 0; e < 64; e += 8)
                        *reinterpret_cast<uint4*>(p.dqd_neg + (rowbase + (long)i * p.H) * glt::KD + ch * 64 + e) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            continue;
        }
#ifdef LLATTN_STAMPS
        int nstamp = 0;
        const int stamp_slot = (blockIdx.x == 5 && nchunk == 8) ? (tid == 0 ? 0 : (tid == 64 ? 1 : -1)) : -1;
#endif
        STAMP();                                             // item top
        // lambda of the inter-chunk levels and the d lambda accumulators of this item
#pragma unroll
        for (int q = 0; q < LAMQ; ++q) {
            const int e = tid + q * 256;
            if (e < CH * glt::LSTRIDE) {
                sLam[e] = __bfloat162float(lam_next[q]);
                sDl[e] = 0.f;
                sDl[CH * glt::LSTRIDE + e] = 0.f;
            }
        }
        if (item + (int)gridDim.x < nitems) fetch_lambda(item + gridDim.x);
        // cumulative gates used by the item's results: requested now, used after the last step
        float g_row = 0.f, g_last = 0.f;
        if (fuse_rows && qrow) g_row = __ldg(p.g_cum + rowbase + (long)i * p.H);
        if (tid == 0) g_last = __ldg(p.g_cum + rowbase + (long)(CH - 1) * p.H);
        if (tid == 0) tma::wait_group_read0();           // the previous item's staged results have been read
        bar_compute();
        float ddec = 0.f;
        bool any_level = false;

        for (int s = 0; s < nsteps; ++s, ++g) {
            const int st = g & 1;                    // result slots / operand tiles alternate; the state tiles rotate over NSTAGE
            const unsigned char* stage = sHE + (g % NSTAGE) * 2 * glt::HE_BYTES;
            const LevStep ls = lev_step(s, c, per_half, trans, live);
            const int lv = ls.level, vh = ls.vh;
            STAMP();                                         // e0 top of the step
            bool ok = umma::mbar_wait(&barA[st], (g >> 1) & 1, abort_flag);
            // the operand tiles of this parity were last read by the second batch of step g - 2
            if (ok && g >= 2) ok = umma::mbar_wait(&barB[st], ((g >> 1) - 1) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            umma::fence_after_sync();
            STAMP();                                         // e1 first batch complete
            unsigned char* op = sOP + st * glt::OP_BYTES;
            if (lv >= 0) {
                any_level = true;
                float t[32];
                umma::tmem_ld32(umma::tmem_addr(tbase + glt::TM_RZ + st * 64, warp, ch * 32), t);
                if (qrow) {
                    // d lambda and the lambda-scaled copy of do (rows 0..63 of the stacked operand)
                    const float lm = sLam[i * glt::LSTRIDE + lv];
                    float dot = 0.f;
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const uint4 dx = *reinterpret_cast<const uint4*>(sDO + vh * CH * 128 + umma::tile_offset(i, ch * 32 + cc * 8, CH));
                        const uint32_t* xw = reinterpret_cast<const uint32_t*>(&dx);
                        uint32_t ow[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[e]);
                            const float a0 = __bfloat162float(v2.x), a1 = __bfloat162float(v2.y);
                            dot += a0 * t[cc * 8 + e * 2] + a1 * t[cc * 8 + e * 2 + 1];
                            ow[e] = pack_bf16(lm * a0, lm * a1);
                        }
                        *reinterpret_cast<uint4*>(op + umma::tile_offset(i, ch * 32 + cc * 8, 128)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                    sDl[(ch * CH + i) * glt::LSTRIDE + lv] += dot;
                } else if (trans) {
                    // -Z
                    unsigned char* nz = sNZ + st * glt::NZ_BYTES;
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                        *reinterpret_cast<uint4*>(nz + umma::tile_offset(i, ch * 32 + cc * 8, CH)) =
                            make_uint4(pack_bf16(-t[cc * 8], -t[cc * 8 + 1]), pack_bf16(-t[cc * 8 + 2], -t[cc * 8 + 3]),
                                       pack_bf16(-t[cc * 8 + 4], -t[cc * 8 + 5]), pack_bf16(-t[cc * 8 + 6], -t[cc * 8 + 7]));
                }
            }
            if (trans) {
                if (qrow) {
                    float ke[32];
                    umma::tmem_ld32(umma::tmem_addr(tbase + glt::TM_KE + st * 64, warp, ch * 32), ke);
                    if (lv >= 0) {
                        // KE: rows 64..127 of the stacked operand
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc)
                            *reinterpret_cast<uint4*>(op + umma::tile_offset(64 + i, ch * 32 + cc * 8, 128)) =
                                make_uint4(pack_bf16(ke[cc * 8], ke[cc * 8 + 1]), pack_bf16(ke[cc * 8 + 2], ke[cc * 8 + 3]),
                                           pack_bf16(ke[cc * 8 + 4], ke[cc * 8 + 5]), pack_bf16(ke[cc * 8 + 6], ke[cc * 8 + 7]));
                    } else {
                        // d_u = kd E_jc, 32 columns of this half of V
                        bf16* du = p.d_u + (rowbase + (long)i * p.H) * p.V + vh * 64 + ch * 32;
#pragma unroll
                        for (int c2 = 0; c2 < 2; ++c2) {
                            uint32_t w[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) w[e] = pack_bf16(ke[c2 * 16 + 2 * e], ke[c2 * 16 + 2 * e + 1]);
                            st_global_32B(du + c2 * 16, w);
                        }
                    }
                } else if (lv >= 0) {
                    // <E, H>: the two tiles have the same layout, so equal offsets are equal elements
                    const unsigned char* hT = stage;
                    const unsigned char* eT = hT + glt::HE_BYTES;
                    const int t128 = (rb - 2) * 32 + lane + ch * 64;       // 0..127
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const uint32_t off = (uint32_t)(q * 128 + t128) * 16;
                        const uint4 hx = *reinterpret_cast<const uint4*>(hT + off);
                        const uint4 ex = *reinterpret_cast<const uint4*>(eT + off);
                        const uint32_t* hw = reinterpret_cast<const uint32_t*>(&hx);
                        const uint32_t* ew = reinterpret_cast<const uint32_t*>(&ex);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&hw[e]);
                            const __nv_bfloat162 bb = *reinterpret_cast<const __nv_bfloat162*>(&ew[e]);
                            ddec += __bfloat162float(a.x) * __bfloat162float(bb.x) + __bfloat162float(a.y) * __bfloat162float(bb.y);
                        }
                    }
                }
            }
            umma::fence_async_smem();
            umma::fence_before_sync();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(&barOp[st])) : "memory");
            STAMP();                                         // e2 operands written
        }
        if (!alive) break;
        // ---- results of the item
        {
            const uint32_t gl = g - 1;               // last step
            const bool ok = umma::mbar_wait(&barB[gl & 1], (gl >> 1) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            umma::fence_after_sync();
        }
        // row terms for the chunk-local gradients (when requested), while the chunk's own qd / wd / kd tiles are still in shared
        // memory: d_qd . qd + d_wd . wd - d_kd . kd per token, the chunk total of d_kd . kd, and -(d_qd exp(G)) in bf16
        float rterm = 0.f, kdot = 0.f;
        const bool zero_qw = !any_level || (!qrow && !trans);   // without a transition wd has no gradient and its rows were never computed
        // d_qd, -d_wd, d_kd leave through shared memory: each thread writes its row's 32 floats of a 64 x 32 box (128-byte
        // swizzled), one thread stores the six boxes of a half with bulk tensor stores.  Both halves are staged in the
        // operand tiles of the steps, idle until the next item's first step.  The chunk's own tiles are released (emptyC)
        // once the row terms have been taken from them.
        {
            const int row0 = b * p.T + c * CH;
            auto stage_half = [&](const int hb) {
                unsigned char* stg = sNZ;
                STAMP();                                     // r0 / r3 half begins
                float t[32];
                if (!zero_qw) {
                    umma::tmem_ld32(umma::tmem_addr(tbase + glt::TM_QW, warp, ch * 64 + hb * 32), t);
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) t[e] = 0.f;
                }
                if (hb == 1) {
                    // the first half's boxes must have been read before the staging area is rewritten
                    if (tid == 0) tma::wait_group_read0();
                    bar_compute();
                }
                STAMP();                                     // r1 / r4 staging free
                const float sg = qrow ? 1.f : -1.f;
                unsigned char* box = stg + ((qrow ? 0 : 2) + ch) * 8192 + i * 128;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    *reinterpret_cast<float4*>(box + ((j ^ (i & 7)) << 4)) = make_float4(sg * t[4 * j], sg * t[4 * j + 1], sg * t[4 * j + 2], sg * t[4 * j + 3]);
                if (qrow) {
                    if (trans) {
                        umma::tmem_ld32(umma::tmem_addr(tbase + glt::TM_K, warp, ch * 64 + hb * 32), t);
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) t[e] = 0.f;
                    }
                    box = stg + (4 + ch) * 8192 + i * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(box + ((j ^ (i & 7)) << 4)) = make_float4(t[4 * j], t[4 * j + 1], t[4 * j + 2], t[4 * j + 3]);
                }
                STAMP();                                     // r2 / r5 rows staged
                umma::fence_async_smem();
                if (hb == 1) {
                    umma::fence_before_sync();
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(accFree)) : "memory");
                }
                bar_compute();
                if (tid == 0) {
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
                        tma::store_box(&p.tm_dqd, c2 * 64 + hb * 32, h, row0, stg + c2 * 8192);
                        tma::store_box(&p.tm_dwd, c2 * 64 + hb * 32, h, row0, stg + (2 + c2) * 8192);
                        tma::store_box(&p.tm_dkd, c2 * 64 + hb * 32, h, row0, stg + (4 + c2) * 8192);
                    }
                    tma::commit_group();
                }
            };
            // the row terms are computed while the first half's boxes are being read
            stage_half(0);
            if (fuse_rows) {
                const float sg = qrow ? 1.f : -1.f;
                const float eg = -fexp(g_row);
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    float t[32];
                    if (!zero_qw) {
                        umma::tmem_ld32(umma::tmem_addr(tbase + glt::TM_QW, warp, ch * 64 + hb * 32), t);
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) t[e] = 0.f;
                    }
                    const unsigned char* orow = sQW + ch * (128 * 128) + row * 128;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 x = *reinterpret_cast<const uint4*>(orow + (((hb * 4 + j) ^ (row & 7)) << 4));
                        const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xs[e]));
                            rterm += sg * (t[8 * j + 2 * e] * f.x + t[8 * j + 2 * e + 1] * f.y);
                        }
                    }
                    if (qrow) {
                        __nv_bfloat16* dst = p.dqd_neg + (rowbase + (long)i * p.H) * glt::KD + ch * 64 + hb * 32;
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            uint32_t w[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) w[e] = pack_bf16(t[16 * j + 2 * e] * eg, t[16 * j + 2 * e + 1] * eg);
                            st_global_32B(dst + 16 * j, w);
                        }
                        if (trans) {
                            umma::tmem_ld32(umma::tmem_addr(tbase + glt::TM_K, warp, ch * 64 + hb * 32), t);
                            const unsigned char* krow = sKd + ch * (CH * 128) + i * 128;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint4 x = *reinterpret_cast<const uint4*>(krow + (((hb * 4 + j) ^ (i & 7)) << 4));
                                const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xs[e]));
                                    kdot += t[8 * j + 2 * e] * f.x + t[8 * j + 2 * e + 1] * f.y;
                                }
                            }
                        }
                    }
                }
                sRowT[((rb >> 1) * 2 + ch) * CH + i] = rterm - kdot;   // four partial sums per token: (q | w rows) x column half
            }
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(emptyC)) : "memory");
            stage_half(1);
        }
        STAMP();                                             // r6 stores issued
        if (!trans) {
            // the last chunk's writes reach no later chunk
            for (int e = tid; e < CH * (p.V / 8); e += 256) {
                const int r = e / (p.V / 8), c8 = (e % (p.V / 8)) * 8;
                *reinterpret_cast<uint4*>(p.d_u + (rowbase + (long)r * p.H) * p.V + c8) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            ddec += __shfl_xor_sync(0xffffffffu, ddec, d);
            kdot += __shfl_xor_sync(0xffffffffu, kdot, d);
        }
        if (lane == 0) {
            sRed[warp] = ddec;
            sRed[8 + warp] = kdot;
        }
        bar_compute();
        if (tid == 0) {
            float t = 0.f, tk = 0.f;
            for (int w = 0; w < 8; ++w) {
                t += sRed[w];
                tk += sRed[8 + w];
            }
            p.d_gl[((long)b * NT + c) * p.H + h] = t * fexp(g_last) + tk;
        }
        if (fuse_rows && tid < CH)
            p.d_grow[rowbase + (long)tid * p.H] = (sRowT[tid] + sRowT[CH + tid]) + (sRowT[2 * CH + tid] + sRowT[3 * CH + tid]);
        for (int e = tid; e < CH * glt::LSTRIDE; e += 256) {
            const int r = e / glt::LSTRIDE, lv = e - r * glt::LSTRIDE;
            if (lv < nlev) p.dl[(rowbase + (long)r * p.H) * p.L + INTRA_LEVELS + lv] = sDl[e] + sDl[CH * glt::LSTRIDE + e];
        }
        bar_compute();                               // the tables are rewritten for the next item
        STAMP();                                             // item end
        ++nchunk;
    }
    if (tid == 0) tma::wait_group0();
    umma::fence_before_sync();
    bar_work();
}

int gdn_bwd_levels_tc_dispatch(const GdnParams& p0, cudaStream_t stream) {
    if (p0.K != glt::KD || p0.V % 64 != 0 || p0.V > 128 || p0.NLEV > GDN_MAXLEV) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    GdnParams p = p0;
    const long BT = (long)p.B * p.T;
    int rc;
    if ((rc = tma::make_panel_map(&p.tm_qd, p.qd, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_wd, p.wd, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_kd, p.kd, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_u, p.u, BT, p.H, p.V, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_do, p.d_o, BT, p.H, p.V, CH)) != 0) return rc;
    if ((rc = tma::make_f32_box_map(&p.tm_dqd, p.d_qd, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_f32_box_map(&p.tm_dwd, p.d_wd, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_f32_box_map(&p.tm_dkd, p.d_kd, BT, p.H, p.K, CH)) != 0) return rc;
    const long tiles = (long)p.B * p.H * (p.V / 64) * p.NT * (p.NLEV > 0 ? p.NLEV : 1);
    if ((rc = tma::make_panel_map(&p.tm_hs, p.hs, tiles * glt::KD, 1, 64, glt::KD)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_dhs, p.dhs, tiles * glt::KD, 1, 64, glt::KD)) != 0) return rc;
    int dev = 0, sms = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    const int nitems = p.B * p.NT * p.H;
    const int grid = nitems < sms ? nitems : sms;
    auto kern = gdn_bwd_levels_tc_kernel;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LevTcSmem::total)) != cudaSuccess) return (int)e;
    kern<<<grid, glt::NTHREADS, LevTcSmem::total, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

}  // namespace llattn

#ifdef LLATTN_STAMPS
extern "C" int llattn_debug_read_stamps_gdn_levels(long long* host_dst) {
    return (int)cudaMemcpyFromSymbol(host_dst, llattn::g_stamps, sizeof(llattn::g_stamps));
}
#endif
