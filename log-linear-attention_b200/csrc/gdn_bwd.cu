// Log-linear Gated DeltaNet chunkwise backward for sm_100a: the two kernels that deal with the
// inter-chunk level states.
//
// Reference being replaced: hattention/chunkwise_hgdn.py:799-1010 (per level: chunk_bwd_dqkwg,
// chunk_gated_delta_rule_bwd_dhu, chunk_bwd_dv_local and the torch glue between them).
//
// Forward recurrence per level state H (K x V), chunk c, with dec = exp(gl), and the chunk's
// matrices kd, wd, qd (64 x K), u (64 x V):
//     readers:     o_i += lambda[i, level] (qd_i . H)            for every level whose bit is set in c
//     transition:  H_jc' = dec Msum + kd^T (u - wd Msum),  Msum = sum of the states below the carry jc
//                  H_lv' = dec H_lv - kd^T (wd H_lv)              for a set bit above the carry
// The adjoint states obey a recurrence that does not involve the forward states at all:
//     E (adjoint of a state after chunk c)  ->  dec E - wd^T (kd E)  (+ qd^T (lambda_lv * do) for readers)
// so the sequential kernel (gdn_scan_bwd_kernel) mirrors the forward scan and only carries adjoints;
// it writes them out per chunk.  Everything that needs forward states AND adjoints (d_qd, d_wd, d_kd,
// the decay gradient, d lambda of the inter-chunk levels) is chunk-parallel: gdn_bwd_levels_kernel.
#include "llattn_common.cuh"
#include "llattn_gdn.h"
#include "llattn_mamba2.h"

namespace llattn {

// acc += A^T B with B's rows (the contraction index) scaled by sc[] (bf16): the product with
// lambda_lv * do without materialising that tile.  A is stored [kred][M], B is stored [kred][N].
template <int MT, int NP>
__device__ __forceinline__ void warp_gemm_tt_bscale(float (&acc)[MT][2 * NP][4], const bf16* A, int lda, int a0,
                                                    const bf16* B, int ldb, int b0, int kred, int lane, const bf16* sc) {
    const int l8 = lane & 7, lq = (lane >> 3) & 1, lh = lane >> 4;
    for (int kk = 0; kk < kred; kk += 16) {
        uint32_t af[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) ldsm_x4_t(af[mt], A + (kk + l8 + lh * 8) * lda + a0 + mt * 16 + lq * 8);
        const __nv_bfloat162 s0 = *reinterpret_cast<const __nv_bfloat162*>(sc + kk + 2 * (lane & 3));
        const __nv_bfloat162 s1 = *reinterpret_cast<const __nv_bfloat162*>(sc + kk + 8 + 2 * (lane & 3));
#pragma unroll
        for (int np = 0; np < NP; ++np) {
            uint32_t bfr[4];
            ldsm_x4_t(bfr, B + (kk + l8 + lq * 8) * ldb + b0 + np * 16 + lh * 8);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&bfr[r]);
                x = __hmul2(x, (r & 1) ? s1 : s0);
                bfr[r] = *reinterpret_cast<uint32_t*>(&x);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma16816(acc[mt][2 * np], af[mt], bfr[0], bfr[1]);
                mma16816(acc[mt][2 * np + 1], af[mt], bfr[2], bfr[3]);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// sequential reverse scan: adjoints of the level states
// ------------------------------------------------------------------------------------------
template <int KD>
struct ScanBwdSmem {
    static constexpr int LDK = KD + PAD, LDS = GDN_VS + PAD;
    static constexpr size_t qw_off = 0;                                          // bf16 [2][128][LDK]: rows 0..63 qd, 64..127 wd
    static constexpr size_t kd_off = qw_off + 2ull * 128 * LDK * 2;              // bf16 [64][LDK]
    static constexpr size_t do_off = kd_off + 1ull * CH * LDK * 2;               // bf16 [2][64][LDS]
    static constexpr size_t e_off = do_off + 2ull * CH * LDS * 2;                // bf16 [MAXLEV][KD][LDS] adjoint copies
    static constexpr size_t ke_off = e_off + (size_t)GDN_MAXLEV * KD * LDS * 2;  // bf16 [MAXLEV][64][LDS]  -(kd E)
    static constexpr size_t lam_off = ke_off + (size_t)GDN_MAXLEV * CH * LDS * 2;   // bf16 [2][MAXLEV][64]
    static constexpr size_t gl_off = lam_off + 2ull * GDN_MAXLEV * CH * 2;       // float [2]
    static constexpr size_t total = gl_off + 16;
};

template <int KD>
__global__ void __launch_bounds__(256, 1) gdn_scan_bwd_kernel(const GdnParams p) {
    using SM = ScanBwdSmem<KD>;
    constexpr int LDK = SM::LDK, LDS = SM::LDS;
    static_assert(KD == 128, "one 16-row state tile per warp");
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQWb = reinterpret_cast<bf16*>(smem + SM::qw_off);
    bf16* sKd = reinterpret_cast<bf16*>(smem + SM::kd_off);
    bf16* sDo = reinterpret_cast<bf16*>(smem + SM::do_off);
    bf16* sE = reinterpret_cast<bf16*>(smem + SM::e_off);
    bf16* sKE = reinterpret_cast<bf16*>(smem + SM::ke_off);
    bf16* sLam = reinterpret_cast<bf16*>(smem + SM::lam_off);
    float* sGl = reinterpret_cast<float*>(smem + SM::gl_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nvs = p.V / GDN_VS;
    const int vs = blockIdx.x % nvs;
    const int h = (blockIdx.x / nvs) % p.H;
    const int b = blockIdx.x / (nvs * p.H);
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
    const int nlev = p.NLEV;
    const int NT = p.NT;

    // one commit group per chunk: kd (single buffer, consumed in the first half of a chunk), do and the
    // stacked qd / wd tile (double buffered)
    auto issue_tiles = [&](int c, int st) {
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
        load_tile_async<CH, KD, 256>(sKd, p.kd + rowbase * KD, (long)p.H * KD, tid);
        load_tile_async<CH, GDN_VS, 256>(sDo + st * CH * LDS, p.d_o + rowbase * p.V + vs * GDN_VS, (long)p.H * p.V, tid);
        load_tile_async<CH, KD, 256>(sQWb + st * 128 * LDK, p.qd + rowbase * KD, (long)p.H * KD, tid);
        load_tile_async<CH, KD, 256>(sQWb + st * 128 * LDK + 64 * LDK, p.wd + rowbase * KD, (long)p.H * KD, tid);
        cp_async_commit();
    };
    bf16 lam_reg[(CH * GDN_MAXLEV + 255) / 256];
    float gl_reg = 0.f;
    auto fetch_small = [&](int c) {
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
#pragma unroll
        for (int i = 0; i < (CH * GDN_MAXLEV + 255) / 256; ++i) {
            const int e = tid + i * 256;
            const int row = e / GDN_MAXLEV, lv = e % GDN_MAXLEV;
            lam_reg[i] = (row < CH && lv < nlev) ? p.l[(rowbase + (long)row * p.H) * p.L + INTRA_LEVELS + lv] : __float2bfloat16(0.f);
        }
        if (tid == 0) gl_reg = p.g_cum[rowbase + (long)(CH - 1) * p.H];
    };
    auto store_small = [&](int st) {
#pragma unroll
        for (int i = 0; i < (CH * GDN_MAXLEV + 255) / 256; ++i) {
            const int e = tid + i * 256;
            const int row = e / GDN_MAXLEV, lv = e % GDN_MAXLEV;
            if (row < CH) sLam[(st * GDN_MAXLEV + lv) * CH + row] = lam_reg[i];
        }
        if (tid == 0) sGl[st] = gl_reg;
    };

    // fp32 masters of the adjoints: this warp holds rows [warp*16, +16) x 32 columns of every level
    float dM[GDN_MAXLEV][1][4][4];
#pragma unroll
    for (int lv = 0; lv < GDN_MAXLEV; ++lv) zero_acc(dM[lv]);

    issue_tiles(NT - 1, (NT - 1) & 1);
    fetch_small(NT - 1);
    store_small((NT - 1) & 1);

    for (int c = NT - 1; c >= 0; --c) {
        const int st = c & 1;
        const bf16* sQW = sQWb + st * 128 * LDK;
        cp_async_wait<0>();                    // the tiles of this chunk
        __syncthreads();
        const bool trans = (c + 1 < NT);       // the chunk's transition feeds later chunks
        const int cn = c + 1;                  // levels that hold a state after this chunk: the set bits of c + 1
        const int jc = __ffs(~c) - 1;
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
        const bf16* cDo = sDo + st * CH * LDS;
        const bf16* cLam = sLam + st * GDN_MAXLEV * CH;
        const float dec = fexp(sGl[st]);

        if (trans) {
            // adjoints of the states written by this chunk, for the chunk-parallel gradient kernel
            bf16* dst = p.dhs + ((size_t)blockIdx.x * NT + c) * nlev * (KD * GDN_VS);
            for (int lv = 0; lv < nlev; ++lv) {
                if (!((cn >> lv) & 1)) continue;
                for (int e = tid; e < KD * (GDN_VS / 8); e += 256) {
                    const int r = e / (GDN_VS / 8), c8 = (e % (GDN_VS / 8)) * 8;
                    *reinterpret_cast<uint4*>(dst + (size_t)lv * KD * GDN_VS + r * GDN_VS + c8) =
                        *reinterpret_cast<const uint4*>(sE + lv * KD * LDS + r * LDS + c8);
                }
            }
        }
        // ---- kd E for every state written by this chunk; the carry level's product is d_u
        {
            const int i0 = (warp & 3) * 16, j0 = (warp >> 2) * 16;
#pragma unroll
            for (int lv = 0; lv < GDN_MAXLEV; ++lv) {
                if (trans && lv < nlev && ((cn >> lv) & 1)) {
                    float acc[1][2][4];
                    zero_acc(acc);
                    warp_gemm<1, 1, false, true>(acc, sKd, LDK, i0, sE + lv * KD * LDS, LDS, j0, KD, lane);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int i = i0 + lr + hh * 8, j = j0 + nt * 8 + lc2;
                            *reinterpret_cast<uint32_t*>(sKE + (lv * CH + i) * LDS + j) = pack_bf16(-acc[0][nt][hh * 2], -acc[0][nt][hh * 2 + 1]);
                            if (lv == jc)
                                *reinterpret_cast<uint32_t*>(p.d_u + (rowbase + (long)i * p.H) * p.V + vs * GDN_VS + j) =
                                    pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
                        }
                }
            }
            if (!trans) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = i0 + lr + hh * 8, j = j0 + nt * 8 + lc2;
                        *reinterpret_cast<uint32_t*>(p.d_u + (rowbase + (long)i * p.H) * p.V + vs * GDN_VS + j) = 0u;
                    }
            }
        }
        __syncthreads();                       // kd has been consumed, the -(kd E) tiles are written
        if (c > 0) {
            issue_tiles(c - 1, st ^ 1);
            fetch_small(c - 1);
        }

        // ---- adjoints of the states that this chunk reads
        float accg[1][4][4];
        zero_acc(accg);
        if (trans) {
            // below the carry every level receives the same transition term  dec E_jc - wd^T (kd E_jc)
            warp_gemm<1, 2, true, true>(accg, sQW + 64 * LDK, LDK, warp * 16, sKE + jc * CH * LDS, LDS, 0, CH, lane);
#pragma unroll
            for (int lv = 0; lv < GDN_MAXLEV; ++lv)
                if (lv == jc) {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) accg[0][nt][e] += dec * dM[lv][0][nt][e];
                }
        }
#pragma unroll
        for (int lv = 0; lv < GDN_MAXLEV; ++lv) {
            if (lv < nlev && ((c >> lv) & 1)) {
                float acc[1][4][4];
                zero_acc(acc);
                warp_gemm_tt_bscale<1, 2>(acc, sQW, LDK, warp * 16, cDo, LDS, 0, CH, lane, cLam + lv * CH);
                if (trans && lv > jc) {
                    warp_gemm<1, 2, true, true>(acc, sQW + 64 * LDK, LDK, warp * 16, sKE + lv * CH * LDS, LDS, 0, CH, lane);
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) dM[lv][0][nt][e] = dec * dM[lv][0][nt][e] + acc[0][nt][e];
                } else {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) dM[lv][0][nt][e] = accg[0][nt][e] + acc[0][nt][e];
                }
                bf16* dst = sE + lv * KD * LDS;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
                        *reinterpret_cast<uint32_t*>(dst + (warp * 16 + lr + hh * 8) * LDS + nt * 8 + lc2) =
                            pack_bf16(dM[lv][0][nt][hh * 2], dM[lv][0][nt][hh * 2 + 1]);
            } else {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) dM[lv][0][nt][e] = 0.f;
            }
        }
        if (c > 0) store_small(st ^ 1);        // the barrier at the top of the next chunk publishes it
    }
}

// ------------------------------------------------------------------------------------------
// chunk-parallel: gradients that pair forward states with adjoints
// ------------------------------------------------------------------------------------------
// One CTA per (batch, head, chunk).  For every level lv whose bit is set in c, with H = the state the
// chunk reads and E = the adjoint of the state that H flows into (level lv above the carry, else the
// carry level jc):
//     R = qd H,  Z = wd H,  kdE = kd E
//     d lambda[i, lv] = sum_v do[i,v] R[i,v]          d_qd += (lambda_lv * do) H^T
//     d_wd -= kdE H^T                                  d_kd -= Z E^T          d_dec += <E, H>
// and once per chunk  d_kd += u E_jc^T.  V is processed in halves of 64 columns; the three 64 x K
// results stay in registers across all (level, half) steps.
template <int KD, int VD>
struct LevSmem {
    static constexpr int LDK = KD + PAD, LDV = VD + PAD, LDH = 64 + PAD;
    static constexpr size_t qw_off = 0;                                       // bf16 [128][LDK]: qd, wd
    static constexpr size_t kd_off = qw_off + 1ull * 128 * LDK * 2;           // bf16 [64][LDK]
    static constexpr size_t u_off = kd_off + 1ull * CH * LDK * 2;             // bf16 [64][LDV]
    static constexpr size_t do_off = u_off + 1ull * CH * LDV * 2;             // bf16 [64][LDV]
    static constexpr size_t h_off = do_off + 1ull * CH * LDV * 2;             // bf16 [2][KD][LDH]
    static constexpr size_t e_off = h_off + 2ull * KD * LDH * 2;              // bf16 [2][KD][LDH]
    static constexpr size_t dol_off = e_off + 2ull * KD * LDH * 2;            // bf16 [64][LDH]  lambda_lv * do
    static constexpr size_t nz_off = dol_off + 1ull * CH * LDH * 2;           // bf16 [64][LDH]  -Z
    static constexpr size_t ke_off = nz_off + 1ull * CH * LDH * 2;            // bf16 [64][LDH]  kd E
    static constexpr size_t lam_off = ke_off + 1ull * CH * LDH * 2;           // float [64][MAXLEV]
    static constexpr size_t dl_off = lam_off + 1ull * CH * GDN_MAXLEV * 4;    // float [64][MAXLEV]
    static constexpr size_t red_off = dl_off + 1ull * CH * GDN_MAXLEV * 4;    // float [8]
    static constexpr size_t total = red_off + 64;
};

template <int KD, int VD>
__global__ void __launch_bounds__(256, 1) gdn_bwd_levels_kernel(const GdnParams p) {
    using SM = LevSmem<KD, VD>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, LDH = SM::LDH;
    constexpr int NVH = VD / 64;
    static_assert(KD == 128, "column split of the 64 x K results assumes K = 128");
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQW = reinterpret_cast<bf16*>(smem + SM::qw_off);
    bf16* sKd = reinterpret_cast<bf16*>(smem + SM::kd_off);
    bf16* sU = reinterpret_cast<bf16*>(smem + SM::u_off);
    bf16* sDo = reinterpret_cast<bf16*>(smem + SM::do_off);
    bf16* sH = reinterpret_cast<bf16*>(smem + SM::h_off);
    bf16* sE = reinterpret_cast<bf16*>(smem + SM::e_off);
    bf16* sDOl = reinterpret_cast<bf16*>(smem + SM::dol_off);
    bf16* sNZ = reinterpret_cast<bf16*>(smem + SM::nz_off);
    bf16* sKE = reinterpret_cast<bf16*>(smem + SM::ke_off);
    float* sLam = reinterpret_cast<float*>(smem + SM::lam_off);
    float* sDl = reinterpret_cast<float*>(smem + SM::dl_off);
    float* sRed = reinterpret_cast<float*>(smem + SM::red_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int c = (blockIdx.x / p.H) % p.NT;
    const int b = blockIdx.x / (p.H * p.NT);
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
    const int nlev = p.NLEV, NT = p.NT;
    const int nvs = p.V / GDN_VS;
    const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
    const bool trans = (c + 1 < NT);
    const int jc = __ffs(~c) - 1;

    // steps: per half of V, an optional step -1 (u E_jc^T) and one step per set bit of c
    const int nlive = __popc((unsigned)c & ((1u << nlev) - 1u));
    const int per_half = nlive + (trans ? 1 : 0);
    const int nsteps = per_half * NVH;
    auto step_level = [&](int s) -> int {      // -1 for the u E_jc^T step
        int r = s % per_half;
        if (trans) {
            if (r == 0) return -1;
            --r;
        }
        int m = c;
        for (int i = 0; i < r; ++i) m &= m - 1;
        return __ffs(m) - 1;
    };
    auto tile_src = [&](const bf16* base, int lv, int vsl) -> const bf16* {
        return base + ((((size_t)(b * p.H + h) * nvs + vsl) * NT + c) * nlev + lv) * (size_t)(KD * GDN_VS);
    };
    auto issue_step = [&](int s, int buf) {
        const int lv = step_level(s), vh = s / per_half;
        for (int e = tid; e < 2 * KD * (GDN_VS / 8); e += 256) {
            const int sl = e / (KD * (GDN_VS / 8)), r = (e / (GDN_VS / 8)) % KD, c8 = (e % (GDN_VS / 8)) * 8;
            if (lv >= 0) cp_async16(sH + (buf * KD + r) * LDH + sl * GDN_VS + c8, tile_src(p.hs, lv, vh * 2 + sl) + r * GDN_VS + c8);
            if (trans) {
                const int le = (lv > jc) ? lv : jc;
                cp_async16(sE + (buf * KD + r) * LDH + sl * GDN_VS + c8, tile_src(p.dhs, le, vh * 2 + sl) + r * GDN_VS + c8);
            }
        }
        cp_async_commit();
    };

    load_tile_async<CH, KD, 256>(sQW, p.qd + rowbase * KD, (long)p.H * KD, tid);
    load_tile_async<CH, KD, 256>(sQW + 64 * LDK, p.wd + rowbase * KD, (long)p.H * KD, tid);
    load_tile_async<CH, KD, 256>(sKd, p.kd + rowbase * KD, (long)p.H * KD, tid);
    load_tile_async<CH, VD, 256>(sU, p.u + rowbase * VD, (long)p.H * VD, tid);
    load_tile_async<CH, VD, 256>(sDo, p.d_o + rowbase * VD, (long)p.H * VD, tid);
    cp_async_commit();
    for (int e = tid; e < CH * GDN_MAXLEV; e += 256) {
        const int i = e / GDN_MAXLEV, lv = e % GDN_MAXLEV;
        sLam[e] = (lv < nlev) ? __bfloat162float(p.l[(rowbase + (long)i * p.H) * p.L + INTRA_LEVELS + lv]) : 0.f;
        sDl[e] = 0.f;
    }
    if (nsteps > 0) issue_step(0, 0);

    float dqd[1][8][4], dwd[1][8][4], dkd[1][8][4];
    zero_acc(dqd);
    zero_acc(dwd);
    zero_acc(dkd);
    float ddec = 0.f;
    const int i0 = (warp & 3) * 16;            // rows of the 64-row products
    const int ch = warp >> 2;                  // column half

    for (int s = 0; s < nsteps; ++s) {
        const int buf = s & 1;
        const int lv = step_level(s), vh = s / per_half;
        cp_async_wait<0>();
        __syncthreads();                       // tiles of step s landed; everyone is done with step s-1
        if (s + 1 < nsteps) issue_step(s + 1, buf ^ 1);
        const bf16* cH = sH + buf * KD * LDH;
        const bf16* cE = sE + buf * KD * LDH;
        if (lv >= 0) {
            // ---- [qd; wd] H : warps 0..3 get R rows, warps 4..7 get Z rows (64 columns)
            float acc[1][8][4];
            zero_acc(acc);
            warp_gemm<1, 4, false, true>(acc, sQW, LDK, warp * 16, cH, LDH, 0, KD, lane);
            if (warp < 4) {
                float part[2] = {0.f, 0.f};
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = warp * 16 + lr + hh * 8;
                        const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(sDo + i * LDV + vh * 64 + nt * 8 + lc2);
                        part[hh] += __bfloat162float(d.x) * acc[0][nt][hh * 2] + __bfloat162float(d.y) * acc[0][nt][hh * 2 + 1];
                    }
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    part[hh] += __shfl_xor_sync(0xffffffffu, part[hh], 1);
                    part[hh] += __shfl_xor_sync(0xffffffffu, part[hh], 2);
                    if ((lane & 3) == 0) sDl[(warp * 16 + lr + hh * 8) * GDN_MAXLEV + lv] += part[hh];
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
                        *reinterpret_cast<uint32_t*>(sNZ + ((warp - 4) * 16 + lr + hh * 8) * LDH + nt * 8 + lc2) =
                            pack_bf16(-acc[0][nt][hh * 2], -acc[0][nt][hh * 2 + 1]);
            }
            // lambda_lv * do
            for (int e = tid; e < CH * 32; e += 256) {
                const int i = e >> 5, j2 = (e & 31) * 2;
                const float lm = sLam[i * GDN_MAXLEV + lv];
                const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(sDo + i * LDV + vh * 64 + j2);
                *reinterpret_cast<uint32_t*>(sDOl + i * LDH + j2) = pack_bf16(lm * __bfloat162float(d.x), lm * __bfloat162float(d.y));
            }
            if (trans) {
                // kd E and <E, H>
                float ke[1][4][4];
                zero_acc(ke);
                warp_gemm<1, 2, false, true>(ke, sKd, LDK, i0, cE, LDH, ch * 32, KD, lane);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
                        *reinterpret_cast<uint32_t*>(sKE + (i0 + lr + hh * 8) * LDH + ch * 32 + nt * 8 + lc2) =
                            pack_bf16(ke[0][nt][hh * 2], ke[0][nt][hh * 2 + 1]);
                for (int e = tid; e < KD * 32; e += 256) {
                    const int r = e >> 5, j2 = (e & 31) * 2;
                    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(cE + r * LDH + j2);
                    const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(cH + r * LDH + j2);
                    ddec += __bfloat162float(x.x) * __bfloat162float(y.x) + __bfloat162float(x.y) * __bfloat162float(y.y);
                }
            }
            __syncthreads();
            warp_gemm<1, 4, false, false>(dqd, sDOl, LDH, i0, cH, LDH, ch * 64, 64, lane);
            if (trans) {
                warp_gemm<1, 4, false, false>(dwd, sKE, LDH, i0, cH, LDH, ch * 64, 64, lane);
                warp_gemm<1, 4, false, false>(dkd, sNZ, LDH, i0, cE, LDH, ch * 64, 64, lane);
            }
        } else {
            // u E_jc^T
            warp_gemm<1, 4, false, false>(dkd, sU + vh * 64, LDV, i0, cE, LDH, ch * 64, 64, lane);
            // d_u = kd E_jc (gradient of the chunk's own writes), 64 columns of this half of V
            float ke[1][4][4];
            zero_acc(ke);
            warp_gemm<1, 2, false, true>(ke, sKd, LDK, i0, cE, LDH, ch * 32, KD, lane);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    *reinterpret_cast<uint32_t*>(p.d_u + (rowbase + (long)(i0 + lr + hh * 8) * p.H) * VD + vh * 64 + ch * 32 + nt * 8 + lc2) =
                        pack_bf16(ke[0][nt][hh * 2], ke[0][nt][hh * 2 + 1]);
        }
    }
    if (nsteps == 0) {
        cp_async_wait<0>();
    }
    if (!trans) {
        // the last chunk's writes reach no later chunk
        for (int e = tid; e < CH * (VD / 8); e += 256) {
            const int i = e / (VD / 8), c8 = (e % (VD / 8)) * 8;
            *reinterpret_cast<uint4*>(p.d_u + (rowbase + (long)i * p.H) * VD + c8) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // ---- results
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int i = i0 + lr + hh * 8, j = ch * 64 + nt * 8 + lc2;
            const long off = (rowbase + (long)i * p.H) * KD + j;
            *reinterpret_cast<float2*>(p.d_qd + off) = make_float2(dqd[0][nt][hh * 2], dqd[0][nt][hh * 2 + 1]);
            *reinterpret_cast<float2*>(p.d_wd + off) = make_float2(-dwd[0][nt][hh * 2], -dwd[0][nt][hh * 2 + 1]);
            *reinterpret_cast<float2*>(p.d_kd + off) = make_float2(dkd[0][nt][hh * 2], dkd[0][nt][hh * 2 + 1]);
        }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ddec += __shfl_xor_sync(0xffffffffu, ddec, d);
    if (lane == 0) sRed[warp] = ddec;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += sRed[w];
        const float gl = p.g_cum[rowbase + (long)(CH - 1) * p.H];
        p.d_gl[((long)b * NT + c) * p.H + h] = t * fexp(gl);
    }
    for (int e = tid; e < CH * GDN_MAXLEV; e += 256) {
        const int i = e / GDN_MAXLEV, lv = e % GDN_MAXLEV;
        if (lv < nlev) p.dl[(rowbase + (long)i * p.H) * p.L + INTRA_LEVELS + lv] = sDl[e];
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
int gdn_bwd_scan_dispatch(const GdnParams& p, cudaStream_t stream) {
    if (p.K != 128) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (g_use_tensor_core_path.load()) return gdn_scan_bwd_tc_dispatch(p, stream);
    auto kern = gdn_scan_bwd_kernel<128>;
    const size_t sm = ScanBwdSmem<128>::total;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
    kern<<<p.B * p.H * (p.V / GDN_VS), 256, sm, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

template <int KD, int VD>
static int launch_levels(const GdnParams& p, cudaStream_t stream) {
    auto kern = gdn_bwd_levels_kernel<KD, VD>;
    const size_t sm = LevSmem<KD, VD>::total;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
    kern<<<p.B * p.NT * p.H, 256, sm, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

// true when the kernel gdn_bwd_levels_dispatch selects also writes dqd_neg / d_grow and folds sum d_kd.kd into d_gl
bool gdn_bwd_levels_writes_row_terms(const GdnParams& p) {
    return p.K == 128 && g_use_tensor_core_path.load() && p.V % 64 == 0 && p.V <= 128;
}

int gdn_bwd_levels_dispatch(const GdnParams& p, cudaStream_t stream) {
    if (p.K == 128 && g_use_tensor_core_path.load()) return gdn_bwd_levels_tc_dispatch(p, stream);
    if (p.K == 128 && p.V == 128) return launch_levels<128, 128>(p, stream);
    if (p.K == 128 && p.V == 64) return launch_levels<128, 64>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace llattn
