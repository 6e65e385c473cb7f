// Log-linear Gated DeltaNet: the chunk-parallel preparation of the forward on tcgen05 / TMEM / TMA (K = 128).
// Same mathematics as gdn_chunk_prep_kernel<.., false> (gdn_fwd.cu); reference being replaced:
// fla_future/chunk_scaled_dot_kkt.py, solve_tril.py, wy_fast.py and chunk_fwd_kernel_o_intra of
// hattention/chunkwise_hgdn.py:566-700.  Per chunk (G = in-chunk cumulative log decay, gl = G at the chunk end):
//   batch 1   [q; k] k^T                      -> tril(q k^T) (bf16 operand), A = stril(beta_i k_i.k_j), A * Gamma (fp32)
//   CUDA cores: (I + A)^-1, (I + A Gamma)^-1   (blocked forward substitution in fp32)
//   batch 2   [Aw; Au] (beta k), [Aw; Au] (beta v)   -> w (rows 0..63), u (rows 64..127)
//   batch 3   tril(q k^T) w, tril(q k^T) Aw, kd^T wd  -> qd, X, Wd = (e^gl - 1) I - kd^T wd
//   batch 4   P v  with  P = X * Gamma * beta_j * lambda[i, bit_length(i ^ j)]   -> intra-chunk output
// Persistent CTAs (one per SM) walk the (batch, chunk, head) items; the q / k tile of the next item is loaded by TMA
// while the current one is worked on.  Products whose M is 64 are issued with M = 128 (the upper 64 result rows are
// not used); stacked operands ([q; k], [Aw; Au]) make both halves useful where two products share their B operand.
#include "tc_common.cuh"
#include "llattn_gdn.h"

namespace llattn {

namespace gpt {
constexpr int KD = 128, NTHREADS = 384, MMA_WARP = 8;
constexpr int LDA = CH + 4;                            // row stride of the fp32 matrices of the triangular solves
constexpr uint32_t QK_BYTES = 128 * KD * 2;            // [q; k]: two panels of 128 rows
constexpr uint32_t T64_BYTES = CH * 128 * 2;           // a 64-row tile with 128 columns: two panels of 64 rows
// tensor memory columns
constexpr int TM_D1 = 0, TM_W = 64, TM_U = 192, TM_QW = 320, TM_X = 448, TM_WD = 64, TM_O = 192, TM_COLS = 512;
}  // namespace gpt

struct PrepTcSmem {
    static constexpr uint32_t in_off = 0;                                          // [2] [q; k]
    static constexpr uint32_t v_off = in_off + 2 * gpt::QK_BYTES;                  // v (64 rows)
    static constexpr uint32_t awu_off = v_off + gpt::T64_BYTES;                    // [Aw; Au]: one panel of 128 rows
    static constexpr uint32_t qkt_off = awu_off + 128 * 128;                       // tril(q k^T), later P: 64 rows (+ 64 never used)
    static constexpr uint32_t r1_off = qkt_off + 128 * 128;                        // A, A*Gamma (fp32) -> beta k, beta v -> w, wd
    static constexpr uint32_t r2_off = r1_off + 36864;                             // inverses (fp32) + block products -> kd
    static constexpr uint32_t t_off = r2_off + 128 * gpt::LDA * 4;                 // float [2][32][32]
    static constexpr uint32_t f_off = r2_off + 43008;                              // G[64] beta[64] lam[64][8]
    static constexpr uint32_t bar_off = f_off + (2 * CH + CH * 8) * 4;
    static constexpr uint32_t total = bar_off + 256 + 1024;
};
static_assert(2 * CH * gpt::LDA * 4 <= 36864 && 128 * gpt::LDA * 4 + 2 * 32 * 32 * 4 <= 43008, "fp32 scratch fits its regions");
static_assert(PrepTcSmem::total <= 232448, "shared memory of one CTA");

template <int VD>
__global__ void __launch_bounds__(gpt::NTHREADS, 1) gdn_chunk_prep_tc_kernel(const __grid_constant__ GdnParams p) {
    using SM = PrepTcSmem;
    constexpr int LDA = gpt::LDA;
    constexpr uint32_t V_BYTES = CH * VD * 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sIn = smem + SM::in_off;
    unsigned char* sV = smem + SM::v_off;
    unsigned char* sAWU = smem + SM::awu_off;
    unsigned char* sQKT = smem + SM::qkt_off;
    unsigned char* sR1 = smem + SM::r1_off;
    unsigned char* sR2 = smem + SM::r2_off;
    float* sA = reinterpret_cast<float*>(sR1);
    float* sAg = sA + CH * LDA;
    float* sX = reinterpret_cast<float*>(sR2);
    float* sT = reinterpret_cast<float*>(smem + SM::t_off);
    float* sGc = reinterpret_cast<float*>(smem + SM::f_off);
    float* sBe = sGc + CH;
    float* sLam = sBe + CH;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* fullQK = bars + 0;     // [2]
    uint64_t* emptyQK = bars + 2;    // [2] (256 arrivals: the element-wise warps read q and k rows with generic loads)
    uint64_t* fullV = bars + 4;
    uint64_t* emptyV = bars + 5;     // the product P v of the item is complete
    uint64_t* bD = bars + 6;         // [4] batch 1..4 complete
    uint64_t* bOp = bars + 10;       // [3] operands of batch 2..4 written (256 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 112);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 120);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NT = p.NT;
    const int nitems = p.B * NT * p.H;

    if (tid == 0) {
        umma::mbar_init(&fullQK[0], 1);
        umma::mbar_init(&fullQK[1], 1);
        umma::mbar_init(&emptyQK[0], 256);
        umma::mbar_init(&emptyQK[1], 256);
        umma::mbar_init(fullV, 1);
        umma::mbar_init(emptyV, 1);
#pragma unroll
        for (int i = 0; i < 4; ++i) umma::mbar_init(&bD[i], 1);
#pragma unroll
        for (int i = 0; i < 3; ++i) umma::mbar_init(&bOp[i], 256);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    if (warp >= gpt::MMA_WARP) {
        if (warp == gpt::MMA_WARP + 1) {
            // ---------------- TMA producer
            if (lane == 0) {
                uint32_t n = 0;
                for (int item = blockIdx.x; item < nitems; item += gridDim.x, ++n) {
                    const int h = item % p.H, c = (item / p.H) % NT, b = item / (p.H * NT);
                    const int st = n & 1, row0 = b * p.T + c * CH;
                    if (n >= 2 && !umma::mbar_wait(&emptyQK[st], ((n >> 1) - 1) & 1, abort_flag)) break;
                    unsigned char* qk = sIn + st * gpt::QK_BYTES;
                    tma::expect_tx(&fullQK[st], gpt::QK_BYTES);
                    tma::load_panel(qk, &p.tm_q, 0, h, row0, &fullQK[st]);                       // q: rows 0..63 of both panels
                    tma::load_panel(qk + 128 * 128, &p.tm_q, 64, h, row0, &fullQK[st]);
                    tma::load_panel(qk + 64 * 128, &p.tm_k, 0, h, row0, &fullQK[st]);            // k: rows 64..127
                    tma::load_panel(qk + 128 * 128 + 64 * 128, &p.tm_k, 64, h, row0, &fullQK[st]);
                    if (n >= 1 && !umma::mbar_wait(emptyV, (n - 1) & 1, abort_flag)) break;
                    tma::expect_tx(fullV, V_BYTES);
                    for (int vp = 0; vp < VD / 64; ++vp) tma::load_panel(sV + vp * CH * 128, &p.tm_v, vp * 64, h, row0, fullV);
                }
            }
            return;
        }
        if (warp > gpt::MMA_WARP) return;
        // ---------------- MMA issuer
        umma::tmem_alloc(tmem_slot, gpt::TM_COLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        const uint32_t aAWU = umma::smem_addr(sAWU), aQKT = umma::smem_addr(sQKT), aR1 = umma::smem_addr(sR1), aKD = umma::smem_addr(sR2),
                       aV = umma::smem_addr(sV);
        constexpr uint32_t ID_KK64 = umma::idesc_bf16(128, 64, false, false);
        constexpr uint32_t ID_KM128 = umma::idesc_bf16(128, 128, false, true);
        constexpr uint32_t ID_KM64 = umma::idesc_bf16(128, 64, false, true);
        constexpr uint32_t ID_KMV = umma::idesc_bf16(128, VD, false, true);
        constexpr uint32_t ID_MM128 = umma::idesc_bf16(128, 128, true, true);
        uint32_t n = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, ++n) {
            const int st = n & 1;
            const uint32_t ph = n & 1;
            const uint32_t aQK = umma::smem_addr(sIn + st * gpt::QK_BYTES);
            if (lane == 0) {
                ok = umma::mbar_wait(&fullQK[st], (n >> 1) & 1, abort_flag);
                if (ok) {
                    umma::fence_after_sync();
                    // batch 1: [q; k] k^T (the k rows of the stacked tile are the B operand)
                    umma::gemm_kk<128, 128, gpt::KD>(tbase + gpt::TM_D1, aQK, aQK + 64 * 128, ID_KK64, false);
                    umma::commit(&bD[0]);
                    ok = umma::mbar_wait(&bOp[0], ph, abort_flag);
                }
                if (ok) {
                    umma::fence_after_sync();
                    // batch 2: [Aw; Au] (beta k) -> w in rows 0..63;  [Aw; Au] (beta v) -> u in rows 64..127
                    umma::gemm_km<128, CH, CH>(tbase + gpt::TM_W, aAWU, aR1, ID_KM128, false);
                    umma::gemm_km<128, CH, CH>(tbase + gpt::TM_U, aAWU, aR1 + gpt::T64_BYTES, ID_KMV, false);
                    umma::commit(&bD[1]);
                    ok = umma::mbar_wait(&bOp[1], ph, abort_flag);
                }
                if (ok) {
                    umma::fence_after_sync();
                    // batch 3: tril(q k^T) w,  tril(q k^T) Aw,  kd^T wd
                    umma::gemm_km<CH, CH, CH>(tbase + gpt::TM_QW, aQKT, aR1, ID_KM128, false);
                    umma::gemm_km<CH, 128, CH>(tbase + gpt::TM_X, aQKT, aAWU, ID_KM64, false);
                    umma::gemm_mm<CH, CH, CH>(tbase + gpt::TM_WD, aKD, aR1 + gpt::T64_BYTES, ID_MM128, false);
                    umma::commit(&bD[2]);
                    ok = umma::mbar_wait(&bOp[2], ph, abort_flag);
                }
                if (ok) {
                    umma::fence_after_sync();
                    // batch 4: P v
                    umma::gemm_km<CH, CH, CH>(tbase + gpt::TM_O, aQKT, aV, ID_KMV, false);
                    umma::commit(&bD[3]);
                    umma::commit(emptyV);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (lane == 0 && ok && n > 0) umma::mbar_wait(&bD[3], (n - 1) & 1, abort_flag);
        __syncwarp();
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();
        umma::tmem_dealloc(tbase, gpt::TM_COLS);
        return;
    }

    // ================= warps 0..7: element-wise =================
    const int rb = warp & 3, ch = warp >> 2;
    const int row = rb * 32 + lane;            // tensor-memory lane
    const bool qrow = rb < 2;                  // lanes 0..63
    const int i = row & 63;                    // token of the chunk
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;
    uint32_t n = 0;
    float pre_g[2] = {0.f, 0.f};
    bf16 pre_b = __float2bfloat16(0.f), pre_l[2] = {__float2bfloat16(0.f), __float2bfloat16(0.f)};
    auto fetch_small = [&](int item) {
        const int h = item % p.H, c = (item / p.H) % NT, b = item / (p.H * NT);
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
        if (warp == 0) {
            pre_g[0] = p.g[rowbase + (long)(2 * lane) * p.H];
            pre_g[1] = p.g[rowbase + (long)(2 * lane + 1) * p.H];
        }
        if (tid >= 64 && tid < 128) pre_b = p.beta[rowbase + (long)(tid - 64) * p.H];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int e = tid + q * 256, r = e >> 3, lv = e & 7;
            if (lv < INTRA_LEVELS) pre_l[q] = p.l[(rowbase + (long)r * p.H) * p.L + lv];
        }
    };
    if ((int)blockIdx.x < nitems) fetch_small(blockIdx.x);

    for (int item = blockIdx.x; item < nitems; item += gridDim.x, ++n) {
        const int h = item % p.H, c = (item / p.H) % NT, b = item / (p.H * NT);
        const int st = n & 1;
        const uint32_t ph = n & 1;
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
        unsigned char* qk = sIn + st * gpt::QK_BYTES;
#ifdef LLATTN_STAMPS
        int nstamp = 0;
        const int stamp_slot = (blockIdx.x == 5 && n == 3) ? (tid == 0 ? 0 : (tid == 64 ? 1 : -1)) : -1;
#endif
        STAMP();                                         // 0 top

        // ---- small per-token inputs: requested one item ahead (registers), staged here
        if (warp == 0) {
            float x0 = pre_g[0], x1 = pre_g[1];
            warp_cumsum64(x0, x1, lane);
            sGc[2 * lane] = x0;
            sGc[2 * lane + 1] = x1;
            p.g_cum[rowbase + (long)(2 * lane) * p.H] = x0;
            p.g_cum[rowbase + (long)(2 * lane + 1) * p.H] = x1;
        }
        if (tid >= 64 && tid < 128) sBe[tid - 64] = __bfloat162float(pre_b);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int e = tid + q * 256, lv = e & 7;
            sLam[e] = (lv < INTRA_LEVELS) ? __bfloat162float(pre_l[q]) : 0.f;
        }
        if (item + (int)gridDim.x < nitems) fetch_small(item + gridDim.x);
        bar_compute();
        STAMP();                                         // 1 small inputs staged
        const float gi = sGc[i], glast = sGc[CH - 1];

        // ---- batch 1 results: tril(q k^T) as a bf16 operand; A and A * Gamma in fp32
        if (!__all_sync(0xffffffffu, umma::mbar_wait(&bD[0], ph, abort_flag))) break;
        umma::fence_after_sync();
        STAMP();                                         // 2 batch 1 complete
        {
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + gpt::TM_D1, warp, ch * 32), t);
            if (qrow) {
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = ch * 32 + cc * 8 + e * 2;
                        w[e] = pack_bf16(j <= i ? t[cc * 8 + e * 2] : 0.f, j + 1 <= i ? t[cc * 8 + e * 2 + 1] : 0.f);
                    }
                    // rows 64..127 of the operand repeat rows 0..63: the products with M = 128 then deliver every result row
                    // twice, and the two lane halves share the element-wise work on it
                    const uint4 v4 = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(sQKT + umma::tile_offset(i, ch * 32 + cc * 8, 128)) = v4;
                    *reinterpret_cast<uint4*>(sQKT + umma::tile_offset(64 + i, ch * 32 + cc * 8, 128)) = v4;
                }
            } else {
                const float bi = sBe[i];
#pragma unroll
                for (int e = 0; e < 32; e += 4) {
                    float a[4], ag[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int j = ch * 32 + e + u;
                        a[u] = (j < i) ? bi * t[e + u] : 0.f;
                        ag[u] = (j < i) ? a[u] * fexp(gi - sGc[j]) : 0.f;
                    }
                    *reinterpret_cast<float4*>(sA + i * LDA + ch * 32 + e) = make_float4(a[0], a[1], a[2], a[3]);
                    *reinterpret_cast<float4*>(sAg + i * LDA + ch * 32 + e) = make_float4(ag[0], ag[1], ag[2], ag[3]);
                }
            }
        }
        umma::fence_before_sync();
        bar_compute();
        STAMP();                                         // 3 A, A Gamma, tril(q k^T) written

        // ---- (I + A)^-1 and (I + A Gamma)^-1 (unit lower triangular, fp32), as 2 x 2 blocks of 32 x 32: the diagonal blocks by
        //      forward substitution (one column per thread, 32 rows in registers), then the block below the diagonal
        //      X_10 = -X_11 (A_10 X_00) as two fp32 products.  (With 16 x 16 blocks the seven barrier-separated stages, each
        //      with little work per thread, took three times as long.)
        {
            constexpr int BS = 32;
            if (tid < 128) {
                const int m = tid >> 6, col = tid & 63, bi = col / BS, cc = col % BS;
                const float* M = (m ? sAg : sA) + (bi * BS) * LDA + bi * BS;
                float x[BS];
#pragma unroll
                for (int r = 0; r < BS; ++r) {
                    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                    for (int j4 = 0; j4 < r; j4 += 4) {
                        const float4 mm = *reinterpret_cast<const float4*>(M + r * LDA + j4);
                        a0 += mm.x * x[j4];
                        if (j4 + 1 < r) a1 += mm.y * x[j4 + 1];
                        if (j4 + 2 < r) a2 += mm.z * x[j4 + 2];
                        if (j4 + 3 < r) a3 += mm.w * x[j4 + 3];
                    }
                    x[r] = ((r == cc) ? 1.f : 0.f) - ((a0 + a1) + (a2 + a3));
                }
                float* X = sX + (m * CH + bi * BS) * LDA + col;
#pragma unroll
                for (int r = 0; r < BS; ++r) X[r * LDA] = x[r];
            }
            bar_compute();
            STAMPR();                                    // r0 diagonal blocks
            // The two products run on 128 threads with a 4 x 4 register tile each (eight 16-byte loads per 64 FMAs): these
            // phases are bound by shared-memory transactions, and one row x eight columns per thread on all 256 threads
            // needed nine loads per 32 FMAs.  The order of summation over k is unchanged.
            if (tid < 128) {
                // T = A_10 X_00
                const int m = tid >> 6, tr = (tid >> 3) & 7, tcq = tid & 7;
                const float* Mrow = (m ? sAg : sA) + (BS + 4 * tr) * LDA;
                const float* Xc = sX + (m * CH) * LDA + 4 * tcq;
                float acc[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll
                for (int k4 = 0; k4 < BS; k4 += 4) {
                    float4 av[4], bv[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) av[i] = *reinterpret_cast<const float4*>(Mrow + i * LDA + k4);
#pragma unroll
                    for (int e = 0; e < 4; ++e) bv[e] = *reinterpret_cast<const float4*>(Xc + (k4 + e) * LDA);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float ae[4] = {av[i].x, av[i].y, av[i].z, av[i].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            acc[i][0] += ae[e] * bv[e].x; acc[i][1] += ae[e] * bv[e].y; acc[i][2] += ae[e] * bv[e].z; acc[i][3] += ae[e] * bv[e].w;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<float4*>(sT + (m * BS + 4 * tr + i) * BS + 4 * tcq) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            }
            bar_compute();
            STAMPR();                                    // r1 first product
            if (tid < 128) {
                // X_10 = -X_11 T
                const int m = tid >> 6, tr = (tid >> 3) & 7, tcq = tid & 7;
                const float* Xii = sX + (m * CH + BS + 4 * tr) * LDA + BS;
                const float* T = sT + (m * BS) * BS + 4 * tcq;
                float acc[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll
                for (int k4 = 0; k4 < BS; k4 += 4) {
                    float4 av[4], bv[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) av[i] = *reinterpret_cast<const float4*>(Xii + i * LDA + k4);
#pragma unroll
                    for (int e = 0; e < 4; ++e) bv[e] = *reinterpret_cast<const float4*>(T + (k4 + e) * BS);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float ae[4] = {av[i].x, av[i].y, av[i].z, av[i].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            acc[i][0] -= ae[e] * bv[e].x; acc[i][1] -= ae[e] * bv[e].y; acc[i][2] -= ae[e] * bv[e].z; acc[i][3] -= ae[e] * bv[e].w;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<float4*>(sX + (m * CH + BS + 4 * tr + i) * LDA + 4 * tcq) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            }
            bar_compute();
            STAMPR();                                    // r2 second product
            // bf16 copies: the stacked operand [Aw; Au] and, as whole rows (16-byte stores), the tensors kept for the backward
            for (int e = tid; e < 2 * CH * (CH / 8); e += 256) {
                const int which = e / (CH * (CH / 8)), r = (e / (CH / 8)) % CH, c8 = (e % (CH / 8)) * 8;
                const float* X = sX + (which * CH + r) * LDA + c8;
                const bool z = (c8 / BS) > (r / BS);                 // blocks above the block diagonal were never written: zero
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) w[q] = z ? 0u : pack_bf16(X[2 * q], X[2 * q + 1]);
                const uint4 v4 = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(sAWU + umma::tile_offset(which * CH + r, c8, 128)) = v4;
                *reinterpret_cast<uint4*>((which ? p.Au : p.Aw) + (rowbase + (long)r * p.H) * CH + c8) = v4;
            }
            bar_compute();                                           // A, A Gamma and the fp32 inverses are dead from here on
        }
        STAMP();                                         // 4 inverses done

        // ---- operands of batch 2: beta k, beta v (in place of A, A Gamma); kd = k exp(gl - G) (in place of the inverses)
        if (!__all_sync(0xffffffffu, umma::mbar_wait(fullV, ph, abort_flag))) break;
        for (int e = tid; e < CH * (gpt::KD / 8); e += 256) {
            const int r = e / (gpt::KD / 8), c8 = (e % (gpt::KD / 8)) * 8;
            const float bi = sBe[r], sc = fexp(glast - sGc[r]);
            const uint4 kx = *reinterpret_cast<const uint4*>(qk + umma::tile_offset(64 + r, c8, 128));
            const uint32_t* xw = reinterpret_cast<const uint32_t*>(&kx);
            uint32_t wb[4], wk[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[q]);
                const float a0 = __bfloat162float(v2.x), a1 = __bfloat162float(v2.y);
                wb[q] = pack_bf16(a0 * bi, a1 * bi);
                wk[q] = pack_bf16(a0 * sc, a1 * sc);
            }
            const uint32_t off = umma::tile_offset(r, c8, CH);
            *reinterpret_cast<uint4*>(sR1 + off) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
            const uint4 kd4 = make_uint4(wk[0], wk[1], wk[2], wk[3]);
            *reinterpret_cast<uint4*>(sR2 + off) = kd4;
            *reinterpret_cast<uint4*>(p.kd + (rowbase + (long)r * p.H) * gpt::KD + c8) = kd4;
        }
        for (int e = tid; e < CH * (VD / 8); e += 256) {
            const int r = e / (VD / 8), c8 = (e % (VD / 8)) * 8;
            const float bi = sBe[r];
            const uint32_t off = umma::tile_offset(r, c8, CH);
            const uint4 vx = *reinterpret_cast<const uint4*>(sV + off);
            const uint32_t* xw = reinterpret_cast<const uint32_t*>(&vx);
            uint32_t wb[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[q]);
                wb[q] = pack_bf16(__bfloat162float(v2.x) * bi, __bfloat162float(v2.y) * bi);
            }
            *reinterpret_cast<uint4*>(sR1 + gpt::T64_BYTES + off) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
        }
        umma::fence_async_smem();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(&bOp[0])) : "memory");
        STAMP();                                         // 5 operands of batch 2 written

        // ---- batch 2 results: w (-> operand tile, wd = w exp(G) -> operand tile and global), u (-> global)
        if (!__all_sync(0xffffffffu, umma::mbar_wait(&bD[1], ph, abort_flag))) break;
        umma::fence_after_sync();
        STAMP();                                         // 6 batch 2 complete
        if (qrow) {
            const float eg = fexp(gi);
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                float t[32];
                umma::tmem_ld32(umma::tmem_addr(tbase + gpt::TM_W, warp, ch * 64 + hb * 32), t);
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    uint32_t wd8[8];
#pragma unroll
                    for (int cq = 0; cq < 2; ++cq) {
                        const int cc = c2 * 2 + cq;
                        const int col = ch * 64 + hb * 32 + cc * 8;
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            w[e] = pack_bf16(t[cc * 8 + e * 2], t[cc * 8 + e * 2 + 1]);
                            wd8[cq * 4 + e] = pack_bf16(t[cc * 8 + e * 2] * eg, t[cc * 8 + e * 2 + 1] * eg);
                        }
                        const uint32_t off = umma::tile_offset(i, col, CH);
                        // beta k is consumed (batch 2 is complete): w takes its place, wd the place of beta v
                        *reinterpret_cast<uint4*>(sR1 + off) = make_uint4(w[0], w[1], w[2], w[3]);
                        *reinterpret_cast<uint4*>(sR1 + gpt::T64_BYTES + off) = make_uint4(wd8[cq * 4], wd8[cq * 4 + 1], wd8[cq * 4 + 2], wd8[cq * 4 + 3]);
                    }
                    st_global_32B(p.wd + (rowbase + (long)i * p.H) * gpt::KD + ch * 64 + hb * 32 + c2 * 16, wd8);
                }
            }
        } else {
#pragma unroll
            for (int hb = 0; hb < VD / 64; ++hb) {
                float t[32];
                umma::tmem_ld32(umma::tmem_addr(tbase + gpt::TM_U, warp, ch * (VD / 2) + hb * 32), t);
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    uint32_t w[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) w[e] = pack_bf16(t[c2 * 16 + e * 2], t[c2 * 16 + e * 2 + 1]);
                    st_global_32B(p.u + (rowbase + (long)i * p.H) * VD + ch * (VD / 2) + hb * 32 + c2 * 16, w);
                }
            }
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(&bOp[1])) : "memory");
        STAMP();                                         // 7 operands of batch 3 written

        // ---- batch 3 results: qd = exp(G) (q - tril(q k^T) w) -> global;  P -> operand tile;  Wd -> global
        if (!__all_sync(0xffffffffu, umma::mbar_wait(&bD[2], ph, abort_flag))) break;
        umma::fence_after_sync();
        STAMP();                                         // 8 batch 3 complete
        {
            // every result row of these products exists twice (lanes i and 64 + i): each lane half takes half of the columns
            const int half = qrow ? 0 : 1;
            const float eg = fexp(gi);
            {
                float t[32];
                const int col0 = ch * 64 + half * 32;
                umma::tmem_ld32(umma::tmem_addr(tbase + gpt::TM_QW, warp, col0), t);
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    uint32_t w[8];
#pragma unroll
                    for (int cq = 0; cq < 2; ++cq) {
                        const int cc = c2 * 2 + cq;
                        const uint4 qx = *reinterpret_cast<const uint4*>(qk + umma::tile_offset(i, col0 + cc * 8, 128));
                        const uint32_t* xw = reinterpret_cast<const uint32_t*>(&qx);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[e]);
                            w[cq * 4 + e] = pack_bf16((__bfloat162float(v2.x) - t[cc * 8 + e * 2]) * eg, (__bfloat162float(v2.y) - t[cc * 8 + e * 2 + 1]) * eg);
                        }
                    }
                    st_global_32B(p.qd + (rowbase + (long)i * p.H) * gpt::KD + col0 + c2 * 16, w);
                }
            }
            float x[16];
            const int j0 = ch * 32 + half * 16;
            umma::tmem_ld16(umma::tmem_addr(tbase + gpt::TM_X, warp, j0), x);
            // The Fenwick level of (i, j) is the position of the highest bit in which they differ.  The low four bits of j are
            // compile-time constants here and its upper two are the same for the whole warp, so "bit k differs" is one of the
            // row's own bits or its complement: lambda is picked from registers with six selects, and the decay and beta of
            // the sixteen columns come in eight 16-byte loads.
            float lamr[8];
            {
                const float4 l0 = *reinterpret_cast<const float4*>(sLam + i * 8), l1 = *reinterpret_cast<const float4*>(sLam + i * 8 + 4);
                lamr[0] = l0.x; lamr[1] = l0.y; lamr[2] = l0.z; lamr[3] = l0.w; lamr[4] = l1.x; lamr[5] = l1.y; lamr[6] = l1.z; lamr[7] = l1.w;
            }
            const bool B0 = i & 1, B1 = i & 2, B2 = i & 4, B3 = i & 8;
            const bool q4 = bool(i & 16) != bool(j0 & 16), q5 = bool(i & 32) != bool(j0 & 32);
            float gcv[16], bev[16];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const float4 g4 = *reinterpret_cast<const float4*>(sGc + j0 + c4 * 4), b4 = *reinterpret_cast<const float4*>(sBe + j0 + c4 * 4);
                gcv[c4 * 4] = g4.x; gcv[c4 * 4 + 1] = g4.y; gcv[c4 * 4 + 2] = g4.z; gcv[c4 * 4 + 3] = g4.w;
                bev[c4 * 4] = b4.x; bev[c4 * 4 + 1] = b4.y; bev[c4 * 4 + 2] = b4.z; bev[c4 * 4 + 3] = b4.w;
            }
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float pv[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int jl = cc * 8 + e * 2 + u;           // low four bits of the column
                        const int j = j0 + jl;
                        const bool q0 = (jl & 1) ? !B0 : B0, q1 = (jl & 2) ? !B1 : B1, q2 = (jl & 4) ? !B2 : B2, q3 = (jl & 8) ? !B3 : B3;
                        float lm = q0 ? lamr[1] : lamr[0];
                        lm = q1 ? lamr[2] : lm;
                        lm = q2 ? lamr[3] : lm;
                        lm = q3 ? lamr[4] : lm;
                        lm = q4 ? lamr[5] : lm;
                        lm = q5 ? lamr[6] : lm;
                        pv[u] = (j <= i) ? x[jl] * fexp(gi - gcv[jl]) * bev[jl] * lm : 0.f;
                    }
                    w[e] = pack_bf16(pv[0], pv[1]);
                }
                // tril(q k^T) is consumed (batch 3 is complete): P takes its place, again with every row twice
                const uint4 v4 = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(sQKT + umma::tile_offset(i, j0 + cc * 8, 128)) = v4;
                *reinterpret_cast<uint4*>(sQKT + umma::tile_offset(64 + i, j0 + cc * 8, 128)) = v4;
            }
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(&emptyQK[st])) : "memory");
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(&bOp[2])) : "memory");

        // Wd leaves while the last product runs (its slots are not touched by that product)
        if (p.wk != nullptr) {
            const float decm1 = fexp(glast) - 1.f;
            bf16* dst = p.wk + ((((long)b * NT + c) * gpt::KD + row) * p.H + h) * gpt::KD + ch * 64;
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                float t[32];
                umma::tmem_ld32(umma::tmem_addr(tbase + gpt::TM_WD, warp, ch * 64 + hb * 32), t);
                // the diagonal of the 128 x 128 matrix crosses this warp's rows in one 32-column block only (the same for the
                // whole warp), at column `lane` of it; everything else is a negation, done on the packed words
                if (ch * 2 + hb == (row >> 5)) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) t[e] = (e == lane) ? t[e] - decm1 : t[e];
                }
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    uint32_t w[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) w[e] = pack_bf16(t[c2 * 16 + e * 2], t[c2 * 16 + e * 2 + 1]) ^ 0x80008000u;
                    st_global_32B(dst + hb * 32 + c2 * 16, w);
                }
            }
        }
        STAMP();                                         // 9 operands of batch 4 written, Wd stored

        // ---- batch 4 result: intra-chunk output rows
        if (!__all_sync(0xffffffffu, umma::mbar_wait(&bD[3], ph, abort_flag))) break;
        umma::fence_after_sync();
        STAMP();                                         // 10 batch 4 complete
        {
            // VD / 4 columns per thread: the output rows exist in both lane halves
            constexpr int NC = VD / 4;
            const int col0 = ch * (VD / 2) + (qrow ? 0 : NC);
            float t[NC];
            if (NC == 32) umma::tmem_ld32(umma::tmem_addr(tbase + gpt::TM_O, warp, col0), reinterpret_cast<float(&)[32]>(t));
            else umma::tmem_ld16(umma::tmem_addr(tbase + gpt::TM_O, warp, col0), reinterpret_cast<float(&)[16]>(t));
#pragma unroll
            for (int c2 = 0; c2 < NC / 16; ++c2) {
                uint32_t w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) w[e] = pack_bf16(t[c2 * 16 + e * 2], t[c2 * 16 + e * 2 + 1]);
                st_global_32B(p.o + (rowbase + (long)i * p.H) * VD + col0 + c2 * 16, w);
            }
        }
        umma::fence_before_sync();
        bar_compute();                                   // the small tables are rewritten for the next item
        STAMP();                                         // 11 output stored
    }
    umma::fence_before_sync();
    bar_work();
}

template <int VD>
static int launch_prep_tc(GdnParams& p, cudaStream_t stream) {
    const long BT = (long)p.B * p.T;
    int rc;
    if ((rc = tma::make_panel_map(&p.tm_q, p.q, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_k, p.k, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_v, p.v, BT, p.H, p.V, CH)) != 0) return rc;
    int dev = 0, sms = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    const int nitems = p.B * p.NT * p.H;
    const int grid = nitems < sms ? nitems : sms;
    auto kern = gdn_chunk_prep_tc_kernel<VD>;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PrepTcSmem::total)) != cudaSuccess) return (int)e;
    kern<<<grid, gpt::NTHREADS, PrepTcSmem::total, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

int gdn_prep_tc_dispatch(const GdnParams& p0, cudaStream_t stream) {
    if (p0.K != gpt::KD) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    GdnParams p = p0;
    if (p.V == 128) return launch_prep_tc<128>(p, stream);
    if (p.V == 64) return launch_prep_tc<64>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace llattn

#ifdef LLATTN_STAMPS
extern "C" int llattn_debug_read_stamps_gdn_prep(long long* host_dst) {
    return (int)cudaMemcpyFromSymbol(host_dst, llattn::g_stamps, sizeof(llattn::g_stamps));
}
#endif
