// Log-linear Gated DeltaNet chunkwise backward for sm_100a: the chunk-local part.
//
// Reference being replaced: the chunk-local kernels called by hattention/chunkwise_hgdn.py:799-1010
// (chunk_bwd_kernel_dqkwg intra part, bwd_prepare_wy_repr, chunk_bwd_kernel_o_intra and the torch
// glue).  One CTA per (batch, head, chunk) turns the gradients with respect to the chunk matrices
// qd, wd, kd, u (from the level stage) and d_o into gradients with respect to q, k, v, beta, g and the
// intra-chunk columns of lambda.  Forward being differentiated (G = in-chunk cumulative log decay,
// gl = G at the chunk end, Gamma_ij = exp(G_i - G_j), Lambda_ij = lambda[i, bit_length(i^j)]):
//     KK = k k^T           A = stril(beta_i KK_ij)       Aw = (I + A)^-1      Au = (I + A * Gamma)^-1
//     w = Aw (beta k)      u = Au (beta v)               QK = tril(q k^T)
//     kd = k exp(gl - G)   wd = w exp(G)                 qd = exp(G) (q - QK w)
//     X = QK Aw            P = X * Gamma * beta_j * Lambda               o_intra = P v
// Aw and Au come from the forward; d(M^-1) = -M^-T dM^-1 M^-T turns their gradients into dA.
#include "llattn_common.cuh"
#include "llattn_gdn.h"
#include "tc_common.cuh"

namespace llattn {

template <int KD, int VD>
struct ChunkBwdSmem {
    static constexpr int LDK = KD + PAD, LDV = VD + PAD, LDP = CH + PAD;
    static constexpr size_t q_off = 0;                                   // bf16 [64][LDK]
    static constexpr size_t k_off = q_off + 1ull * CH * LDK * 2;
    static constexpr size_t w_off = k_off + 1ull * CH * LDK * 2;          // w
    static constexpr size_t dqd_off = w_off + 1ull * CH * LDK * 2;        // -(d_qd exp(G))
    static constexpr size_t dw_off = dqd_off + 1ull * CH * LDK * 2;       // dw
    static constexpr size_t v_off = dw_off + 1ull * CH * LDK * 2;         // bf16 [64][LDV]
    static constexpr size_t do_off = v_off + 1ull * CH * LDV * 2;
    static constexpr size_t du_off = do_off + 1ull * CH * LDV * 2;
    static constexpr size_t qk_off = du_off + 1ull * CH * LDV * 2;        // bf16 [64][LDP] tril(q k^T), later dKK
    static constexpr size_t aw_off = qk_off + 1ull * CH * LDP * 2;
    static constexpr size_t au_off = aw_off + 1ull * CH * LDP * 2;
    static constexpr size_t kk_off = au_off + 1ull * CH * LDP * 2;        // k k^T
    static constexpr size_t ta_off = kk_off + 1ull * CH * LDP * 2;        // Aw*beta_j, P, dAw, dAu
    static constexpr size_t tb_off = ta_off + 1ull * CH * LDP * 2;        // dX, dAw Aw^T, dAu Au^T
    static constexpr size_t dqk_off = tb_off + 1ull * CH * LDP * 2;       // dQK
    static constexpr size_t f_off = dqk_off + 1ull * CH * LDP * 2;        // floats
    // floats: G[64] beta[64] eG[64] eGk[64] dG[64] dB[64] lam[64][8] dL[64][8] misc[8] part[22][64]
    static constexpr size_t total = f_off + (6 * CH + 2 * CH * 8 + 8 + 22 * CH) * 4;
};

// FUSED: the level-gradient kernel has already written -(d_qd exp(G)) in bf16, the per-token sums d_qd.qd + d_wd.wd - d_kd.kd and
// the chunk total of d_kd.kd (inside d_gl); otherwise a row pass over the K-wide gradients derives them here.
template <int KD, int VD, bool FUSED>
__global__ void __launch_bounds__(256, 1) gdn_bwd_chunk_kernel(const GdnParams p) {
    using SM = ChunkBwdSmem<KD, VD>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, LDP = SM::LDP;
    constexpr int NPK = KD / 32, NPV = VD / 32;       // 16-column pairs per warp for 64 x K and 64 x V results
    static_assert(KD == 128, "row passes assume one float4 per lane per row");
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sK = reinterpret_cast<bf16*>(smem + SM::k_off);
    bf16* sW = reinterpret_cast<bf16*>(smem + SM::w_off);
    bf16* sDqd = reinterpret_cast<bf16*>(smem + SM::dqd_off);
    bf16* sDW = reinterpret_cast<bf16*>(smem + SM::dw_off);
    bf16* sV = reinterpret_cast<bf16*>(smem + SM::v_off);
    bf16* sDo = reinterpret_cast<bf16*>(smem + SM::do_off);
    bf16* sDU = reinterpret_cast<bf16*>(smem + SM::du_off);
    bf16* sQK = reinterpret_cast<bf16*>(smem + SM::qk_off);
    bf16* sAw = reinterpret_cast<bf16*>(smem + SM::aw_off);
    bf16* sAu = reinterpret_cast<bf16*>(smem + SM::au_off);
    bf16* sKK = reinterpret_cast<bf16*>(smem + SM::kk_off);
    bf16* sTa = reinterpret_cast<bf16*>(smem + SM::ta_off);
    bf16* sTb = reinterpret_cast<bf16*>(smem + SM::tb_off);
    bf16* sDQK = reinterpret_cast<bf16*>(smem + SM::dqk_off);
    float* sG = reinterpret_cast<float*>(smem + SM::f_off);
    float* sBe = sG + CH;
    float* sEG = sBe + CH;
    float* sEGk = sEG + CH;
    float* sDG = sEGk + CH;
    float* sDB = sDG + CH;
    float* sLam = sDB + CH;           // [64][8]   (the dB slot itself is unused: beta gradients are summed from the partial slots)
    float* sDL = sLam + CH * 8;       // [64][8]
    float* sMisc = sDL + CH * 8;      // [0] = sum d_kd . kd
    // partial sums of the decay (G) and beta gradients, one slot per producing warp group so that no stage needs shared-memory
    // atomics: column sums are split over the four row blocks of warps, row sums over the two column halves
    float* sPart = sMisc + 8;
    float* pColG_P = sPart;                 // [4][64]  P stage
    float* pColG_A = sPart + 4 * CH;        // [4][64]  dA stage
    float* pColB_P = sPart + 8 * CH;        // [4][64]
    float* pRowG_P = sPart + 12 * CH;       // [2][64]
    float* pRowG_A = sPart + 14 * CH;       // [2][64]
    float* pRowB_V = sPart + 16 * CH;       // [2][64]  dv stage
    float* pRowB_K = sPart + 18 * CH;       // [2][64]  d(beta k) stage
    float* pRowB_A = sPart + 20 * CH;       // [2][64]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rbw = warp & 3;               // row block of the warp
#ifdef LLATTN_STAMPS
    int nstamp = 0;
    const int stamp_slot = (blockIdx.x == 3000 && (tid & 31) == 0 && (warp == 0 || warp == 7 || warp == 2)) ? (warp == 0 ? 0 : (warp == 7 ? 1 : 2)) : -1;
#endif
    STAMP();
    const int h = blockIdx.x % p.H;
    const int c = (blockIdx.x / p.H) % p.NT;
    const int b = blockIdx.x / (p.H * p.NT);
    const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
    const int r0 = (warp & 3) * 16, cw = warp >> 2;
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;

    // the small loads go first: their latency passes while the tile copies are being issued
    float gv = 0.f;
    __nv_bfloat16 bv = __float2bfloat16(0.f), lv2[2];
    if (tid < CH) {
        gv = __ldg(p.g_cum + rowbase + (long)tid * p.H);
        bv = __ldg(p.beta + rowbase + (long)tid * p.H);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int e = tid + u * 256, i = e >> 3, lv = e & 7;
        lv2[u] = (lv < INTRA_LEVELS) ? __ldg(p.l + (rowbase + (long)i * p.H) * p.L + lv) : __float2bfloat16(0.f);
    }
    float grow = 0.f;
    if (FUSED && tid < CH) grow = __ldg(p.d_grow + rowbase + (long)tid * p.H);
    // two groups: the first products (k k^T, q k^T, Aw * beta_j) wait for q, k, Aw only
    load_tile_async<CH, KD, 256>(sQ, p.q + rowbase * KD, (long)p.H * KD, tid);
    load_tile_async<CH, KD, 256>(sK, p.k + rowbase * KD, (long)p.H * KD, tid);
    load_tile_async<CH, CH, 256>(sAw, p.Aw + rowbase * CH, (long)p.H * CH, tid);
    cp_async_commit();
    load_tile_async<CH, VD, 256>(sV, p.v + rowbase * VD, (long)p.H * VD, tid);
    load_tile_async<CH, VD, 256>(sDo, p.d_o + rowbase * VD, (long)p.H * VD, tid);
    load_tile_async<CH, VD, 256>(sDU, p.d_u + rowbase * VD, (long)p.H * VD, tid);
    load_tile_async<CH, CH, 256>(sAu, p.Au + rowbase * CH, (long)p.H * CH, tid);
    if (FUSED) load_tile_async<CH, KD, 256>(sDqd, p.dqd_neg + rowbase * KD, (long)p.H * KD, tid);
    cp_async_commit();
    if (FUSED) {
        // the fp32 level gradients are read as accumulator fragments in later stages: bring their 3 x 64 rows x 512 bytes into L2 now
        const long off = (rowbase + (long)(tid >> 2) * p.H) * KD + (tid & 3) * 32;
        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p.d_wd + off));
        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p.d_kd + off));
        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p.d_qd + off));
    }
    if (tid < CH) {
        sG[tid] = gv;
        sBe[tid] = __bfloat162float(bv);
        sDG[tid] = grow;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        sLam[tid + u * 256] = __bfloat162float(lv2[u]);
        sDL[tid + u * 256] = 0.f;
    }
    if (tid == 0) sMisc[0] = 0.f;
    __syncthreads();
    STAMP();
    if (tid < CH) {
        sEG[tid] = fexp(sG[tid]);
        sEGk[tid] = fexp(sG[CH - 1] - sG[tid]);
    }
    __syncthreads();
    STAMP();

    // ---- row pass over the K-wide gradients: -(d_qd exp(G)) as a bf16 operand; the decay terms
    //      dG_i += d_qd.qd + d_wd.wd - d_kd.kd and the chunk total of d_kd.kd
    if (!FUSED) {
        float kdsum = 0.f;
        // four rows per batch: every load of a batch is issued before the first use, so a batch pays the load latency once
#pragma unroll
        for (int bt = 0; bt < CH / 32; ++bt) {
            float4 a[4], bw[4], ck[4];
            uint2 xq[4], xw[4], xk[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = (bt * 4 + u) * 8 + warp;
                const long off = (rowbase + (long)i * p.H) * KD + lane * 4;
                a[u] = __ldg(reinterpret_cast<const float4*>(p.d_qd + off));
                bw[u] = __ldg(reinterpret_cast<const float4*>(p.d_wd + off));
                ck[u] = __ldg(reinterpret_cast<const float4*>(p.d_kd + off));
                xq[u] = __ldg(reinterpret_cast<const uint2*>(p.qd + off));
                xw[u] = __ldg(reinterpret_cast<const uint2*>(p.wd + off));
                xk[u] = __ldg(reinterpret_cast<const uint2*>(p.kd + off));
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = (bt * 4 + u) * 8 + warp;
                const __nv_bfloat162 q0 = *reinterpret_cast<const __nv_bfloat162*>(&xq[u].x), q1 = *reinterpret_cast<const __nv_bfloat162*>(&xq[u].y);
                const __nv_bfloat162 w0 = *reinterpret_cast<const __nv_bfloat162*>(&xw[u].x), w1 = *reinterpret_cast<const __nv_bfloat162*>(&xw[u].y);
                const __nv_bfloat162 k0 = *reinterpret_cast<const __nv_bfloat162*>(&xk[u].x), k1 = *reinterpret_cast<const __nv_bfloat162*>(&xk[u].y);
                float dq_ = a[u].x * __bfloat162float(q0.x) + a[u].y * __bfloat162float(q0.y) + a[u].z * __bfloat162float(q1.x) + a[u].w * __bfloat162float(q1.y);
                float dw_ = bw[u].x * __bfloat162float(w0.x) + bw[u].y * __bfloat162float(w0.y) + bw[u].z * __bfloat162float(w1.x) + bw[u].w * __bfloat162float(w1.y);
                float dk_ = ck[u].x * __bfloat162float(k0.x) + ck[u].y * __bfloat162float(k0.y) + ck[u].z * __bfloat162float(k1.x) + ck[u].w * __bfloat162float(k1.y);
                float r = dq_ + dw_ - dk_;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) {
                    r += __shfl_xor_sync(0xffffffffu, r, d);
                    dk_ += __shfl_xor_sync(0xffffffffu, dk_, d);
                }
                if (lane == 0) sDG[i] += r;          // one warp per row: no other writer at this point
                kdsum += dk_;
                const float eg = -sEG[i];
                uint2 o;
                o.x = pack_bf16(a[u].x * eg, a[u].y * eg);
                o.y = pack_bf16(a[u].z * eg, a[u].w * eg);
                *reinterpret_cast<uint2*>(sDqd + i * LDK + lane * 4) = o;
            }
        }
        if (lane == 0) atomicAdd(&sMisc[0], kdsum);
    }
    cp_async_wait<1>();
    __syncthreads();
    STAMP();

    // ---- KK = k k^T, QK = tril(q k^T), Aw * beta_j
    {
        float accK[1][4][4], accQ[1][4][4];
        zero_acc(accK);
        zero_acc(accQ);
        warp_gemm<1, 2, false, false>(accK, sK, LDK, r0, sK, LDK, cw * 32, KD, lane);
        warp_gemm<1, 2, false, false>(accQ, sQ, LDK, r0, sK, LDK, cw * 32, KD, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = cw * 32 + nt * 8 + lc2;
                *reinterpret_cast<uint32_t*>(sKK + i * LDP + j) = pack_bf16(accK[0][nt][hh * 2], accK[0][nt][hh * 2 + 1]);
                *reinterpret_cast<uint32_t*>(sQK + i * LDP + j) =
                    pack_bf16(j <= i ? accQ[0][nt][hh * 2] : 0.f, j + 1 <= i ? accQ[0][nt][hh * 2 + 1] : 0.f);
            }
        for (int e = tid; e < CH * CH / 2; e += 256) {
            const int i = e / (CH / 2), j = (e % (CH / 2)) * 2;
            const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(sAw + i * LDP + j);
            *reinterpret_cast<uint32_t*>(sTa + i * LDP + j) = pack_bf16(__bfloat162float(x.x) * sBe[j], __bfloat162float(x.y) * sBe[j + 1]);
        }
    }
    cp_async_wait<0>();                        // v, do, d_u, Au (and the bf16 d_qd term) have landed
    __syncthreads();
    STAMP();

    // ---- w = (Aw * beta_j) k ;  X = QK Aw ;  dP = do v^T
    float accX[1][4][4], accP[1][4][4];
    {
        float acc[1][2 * NPK][4];
        zero_acc(acc);
        warp_gemm<1, NPK, false, true>(acc, sTa, LDP, r0, sK, LDK, cw * (KD / 2), CH, lane);
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
                *reinterpret_cast<uint32_t*>(sW + (r0 + lr + hh * 8) * LDK + cw * (KD / 2) + nt * 8 + lc2) =
                    pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
        zero_acc(accX);
        zero_acc(accP);
        warp_gemm<1, 2, false, true>(accX, sQK, LDP, r0, sAw, LDP, cw * 32, CH, lane);
        warp_gemm<1, 2, false, false>(accP, sDo, LDV, r0, sV, LDV, cw * 32, VD, lane);
    }
    __syncthreads();                           // Aw * beta_j has been consumed: its tile becomes P
    STAMP();
    {
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float cs[2] = {0.f, 0.f}, cb[2] = {0.f, 0.f};
            // G and beta of this thread's two columns: one 8-byte load each per 8-column tile
            const float2 gj2 = *reinterpret_cast<const float2*>(sG + cw * 32 + nt * 8 + lc2);
            const float2 bj2 = *reinterpret_cast<const float2*>(sBe + cw * 32 + nt * 8 + lc2);
            const float gjv[2] = {gj2.x, gj2.y}, bjv[2] = {bj2.x, bj2.y};
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8;
                const float gi = sG[i];
                float pv[2] = {0.f, 0.f}, dx[2] = {0.f, 0.f};
                // 8 x 8 block of the fragment (the same for the whole warp): above the diagonal nothing; below it every
                // element is causal and lies in one Fenwick level, whose d lambda sum goes through the four lanes of a row
                // to that row's single writer; the diagonal blocks sum their four levels the same way.
                const int ib = (r0 >> 3) + hh, jb = cw * 4 + nt;
                if (jb <= ib) {
                    const bool below = jb < ib;
                    const int levb = 35 - __clz(ib ^ jb);
                    float dls = 0.f, dlv[2] = {0.f, 0.f};
                    int dll[2] = {-1, -1};
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = cw * 32 + nt * 8 + lc2 + e;
                        if (below || j <= i) {
                            const int lev = below ? levb : level_of(i, j);
                            const float gam = fexp(gi - gjv[e]), bj = bjv[e], lm = sLam[i * 8 + lev];
                            const float x = accX[0][nt][hh * 2 + e], dp = accP[0][nt][hh * 2 + e];
                            const float xg = dp * x * gam;
                            pv[e] = x * gam * bj * lm;
                            dx[e] = dp * gam * bj * lm;
                            if (below) dls += xg * bj;
                            else { dlv[e] = xg * bj; dll[e] = lev; }
                            cb[e] += xg * lm;
                            const float s = xg * bj * lm;
                            rs[hh] += s;
                            cs[e] += s;
                        }
                    }
                    // each (row, level) sum has a single writer: the level's columns lie in one column half, and a row belongs to one warp
                    if (below) {
                        dls += __shfl_xor_sync(0xffffffffu, dls, 1);
                        dls += __shfl_xor_sync(0xffffffffu, dls, 2);
                        if ((lane & 3) == 0) sDL[i * 8 + levb] += dls;
                    } else {
#pragma unroll
                        for (int lv = 0; lv < 4; ++lv) {     // the levels inside a diagonal 8 x 8 block
                            float v = (dll[0] == lv ? dlv[0] : 0.f) + (dll[1] == lv ? dlv[1] : 0.f);
                            v += __shfl_xor_sync(0xffffffffu, v, 1);
                            v += __shfl_xor_sync(0xffffffffu, v, 2);
                            if ((lane & 3) == 0) sDL[i * 8 + lv] += v;
                        }
                    }
                }
                const int j0 = cw * 32 + nt * 8 + lc2;
                *reinterpret_cast<uint32_t*>(sTa + i * LDP + j0) = pack_bf16(pv[0], pv[1]);
                *reinterpret_cast<uint32_t*>(sTb + i * LDP + j0) = pack_bf16(dx[0], dx[1]);
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) {
                    cs[e] += __shfl_xor_sync(0xffffffffu, cs[e], d);
                    cb[e] += __shfl_xor_sync(0xffffffffu, cb[e], d);
                }
                if (lr == 0) {
                    const int j = cw * 32 + nt * 8 + lc2 + e;
                    pColG_P[rbw * CH + j] = -cs[e];
                    pColB_P[rbw * CH + j] = cb[e];
                }
            }
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            rs[hh] += __shfl_xor_sync(0xffffffffu, rs[hh], 1);
            rs[hh] += __shfl_xor_sync(0xffffffffu, rs[hh], 2);
            if ((lane & 3) == 0) pRowG_P[cw * CH + r0 + lr + hh * 8] = rs[hh];
        }
    }
    __syncthreads();
    STAMP();

    // ---- dv = P^T do + beta * (Au^T d_u) ;  dbeta_i += (Au^T d_u)_i . v_i
    {
        float acc[1][2 * NPV][4], acc2[1][2 * NPV][4];
        zero_acc(acc);
        zero_acc(acc2);
        const int c0 = cw * (VD / 2);
        warp_gemm<1, NPV, true, true>(acc, sTa, LDP, r0, sDo, LDV, c0, CH, lane);
        STAMP();
        warp_gemm<1, NPV, true, true>(acc2, sAu, LDP, r0, sDU, LDV, c0, CH, lane);
        STAMP();
        float rb[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2 * NPV; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = c0 + nt * 8 + lc2;
                const float bi = sBe[i];
                const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(sV + i * LDV + j);
                rb[hh] += acc2[0][nt][hh * 2] * __bfloat162float(x.x) + acc2[0][nt][hh * 2 + 1] * __bfloat162float(x.y);
                const float d0 = acc[0][nt][hh * 2] + bi * acc2[0][nt][hh * 2], d1 = acc[0][nt][hh * 2 + 1] + bi * acc2[0][nt][hh * 2 + 1];
                if (p.dv_bf16) *reinterpret_cast<uint32_t*>(p.dv_bf16 + (rowbase + (long)i * p.H) * VD + j) = pack_bf16(d0, d1);
                else *reinterpret_cast<float2*>(p.dv + (rowbase + (long)i * p.H) * VD + j) = make_float2(d0, d1);
            }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            rb[hh] += __shfl_xor_sync(0xffffffffu, rb[hh], 1);
            rb[hh] += __shfl_xor_sync(0xffffffffu, rb[hh], 2);
            if ((lane & 3) == 0) pRowB_V[cw * CH + r0 + lr + hh * 8] = rb[hh];
        }
    }
    STAMP();
    // ---- dQK = tril(dX Aw^T - (d_qd exp(G)) w^T)
    {
        float acc[1][4][4];
        zero_acc(acc);
        warp_gemm<1, 2, false, false>(acc, sTb, LDP, r0, sAw, LDP, cw * 32, CH, lane);
        warp_gemm<1, 2, false, false>(acc, sDqd, LDK, r0, sW, LDK, cw * 32, KD, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = cw * 32 + nt * 8 + lc2;
                *reinterpret_cast<uint32_t*>(sDQK + i * LDP + j) =
                    pack_bf16(j <= i ? acc[0][nt][hh * 2] : 0.f, j + 1 <= i ? acc[0][nt][hh * 2 + 1] : 0.f);
            }
    }
    STAMP();
    // ---- dw = d_wd exp(G) - QK^T (d_qd exp(G))
    {
        float acc[1][2 * NPK][4];
        zero_acc(acc);
        const int c0 = cw * (KD / 2);
        // the fp32 gradient fragment is requested before the product so that its latency overlaps the MMAs
        float2 pre[2 * NPK][2];
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
                pre[nt][hh] = *reinterpret_cast<const float2*>(p.d_wd + (rowbase + (long)(r0 + lr + hh * 8) * p.H) * KD + c0 + nt * 8 + lc2);
        warp_gemm<1, NPK, true, true>(acc, sQK, LDP, r0, sDqd, LDK, c0, CH, lane);
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = c0 + nt * 8 + lc2;
                const float2 d = pre[nt][hh];
                const float eg = sEG[i];
                *reinterpret_cast<uint32_t*>(sDW + i * LDK + j) = pack_bf16(acc[0][nt][hh * 2] + d.x * eg, acc[0][nt][hh * 2 + 1] + d.y * eg);
            }
    }
    __syncthreads();                           // dw and dQK complete; P has been consumed
    STAMP();
    // ---- dAw = QK^T dX + (dw k^T) * beta_j   -> tile
    {
        float acc[1][4][4], acc2[1][4][4];
        zero_acc(acc);
        zero_acc(acc2);
        warp_gemm<1, 2, true, true>(acc, sQK, LDP, r0, sTb, LDP, cw * 32, CH, lane);
        warp_gemm<1, 2, false, false>(acc2, sDW, LDK, r0, sK, LDK, cw * 32, KD, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = cw * 32 + nt * 8 + lc2;
                *reinterpret_cast<uint32_t*>(sTa + i * LDP + j) =
                    pack_bf16(acc[0][nt][hh * 2] + acc2[0][nt][hh * 2] * sBe[j], acc[0][nt][hh * 2 + 1] + acc2[0][nt][hh * 2 + 1] * sBe[j + 1]);
            }
    }
    __syncthreads();                           // dAw complete; dX and QK have been consumed
    STAMP();
    // ---- dAw Aw^T -> tile
    {
        float acc[1][4][4];
        zero_acc(acc);
        warp_gemm<1, 2, false, false>(acc, sTa, LDP, r0, sAw, LDP, cw * 32, CH, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
                *reinterpret_cast<uint32_t*>(sTb + (r0 + lr + hh * 8) * LDP + cw * 32 + nt * 8 + lc2) = pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
    }
    __syncthreads();
    STAMP();
    // ---- dA (from Aw) = -Aw^T (dAw Aw^T) ;  d(beta k) = Aw^T dw starts the dk accumulator
    float dA1[1][4][4];
    float dk_acc[1][2 * NPK][4];
    {
        zero_acc(dA1);
        warp_gemm<1, 2, true, true>(dA1, sAw, LDP, r0, sTb, LDP, cw * 32, CH, lane);
        zero_acc(dk_acc);
        const int c0 = cw * (KD / 2);
        float2 pre[2 * NPK][2];
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
                pre[nt][hh] = *reinterpret_cast<const float2*>(p.d_kd + (rowbase + (long)(r0 + lr + hh * 8) * p.H) * KD + c0 + nt * 8 + lc2);
        warp_gemm<1, NPK, true, true>(dk_acc, sAw, LDP, r0, sDW, LDK, c0, CH, lane);
        float rb[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = c0 + nt * 8 + lc2;
                const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(sK + i * LDK + j);
                rb[hh] += dk_acc[0][nt][hh * 2] * __bfloat162float(x.x) + dk_acc[0][nt][hh * 2 + 1] * __bfloat162float(x.y);
                const float bi = sBe[i];
                const float2 d = pre[nt][hh];
                const float ek = sEGk[i];
                dk_acc[0][nt][hh * 2] = dk_acc[0][nt][hh * 2] * bi + d.x * ek;
                dk_acc[0][nt][hh * 2 + 1] = dk_acc[0][nt][hh * 2 + 1] * bi + d.y * ek;
            }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            rb[hh] += __shfl_xor_sync(0xffffffffu, rb[hh], 1);
            rb[hh] += __shfl_xor_sync(0xffffffffu, rb[hh], 2);
            if ((lane & 3) == 0) pRowB_K[cw * CH + r0 + lr + hh * 8] = rb[hh];
        }
    }
    STAMP();
    // ---- dAu = (d_u v^T) * beta_j -> tile (the dAw tile has been consumed before the last barrier)
    {
        float acc[1][4][4];
        zero_acc(acc);
        warp_gemm<1, 2, false, false>(acc, sDU, LDV, r0, sV, LDV, cw * 32, VD, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int j = cw * 32 + nt * 8 + lc2;
                *reinterpret_cast<uint32_t*>(sTa + (r0 + lr + hh * 8) * LDP + j) = pack_bf16(acc[0][nt][hh * 2] * sBe[j], acc[0][nt][hh * 2 + 1] * sBe[j + 1]);
            }
    }
    __syncthreads();                           // dAu complete; (dAw Aw^T) consumed
    STAMP();
    {
        float acc[1][4][4];
        zero_acc(acc);
        warp_gemm<1, 2, false, false>(acc, sTa, LDP, r0, sAu, LDP, cw * 32, CH, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
                *reinterpret_cast<uint32_t*>(sTb + (r0 + lr + hh * 8) * LDP + cw * 32 + nt * 8 + lc2) = pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
    }
    __syncthreads();
    STAMP();
    // ---- dAg = -Au^T (dAu Au^T);  dA = dA1 + dAg * Gamma;  decay and beta terms;  dKK = beta_i dA
    {
        float dAg[1][4][4];
        zero_acc(dAg);
        warp_gemm<1, 2, true, true>(dAg, sAu, LDP, r0, sTb, LDP, cw * 32, CH, lane);
        float rs[2] = {0.f, 0.f}, rb[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float cs[2] = {0.f, 0.f};
            const float2 gjA2 = *reinterpret_cast<const float2*>(sG + cw * 32 + nt * 8 + lc2);
            const float gjA[2] = {gjA2.x, gjA2.y};
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8;
                const float gi = sG[i], bi = sBe[i];
                float dkk[2] = {0.f, 0.f};
                const float2 kkv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(sKK + i * LDP + cw * 32 + nt * 8 + lc2));
                if (cw * 4 + nt <= (r0 >> 3) + hh)       // 8 x 8 blocks above the diagonal hold no causal pair (the same for the whole warp)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = cw * 32 + nt * 8 + lc2 + e;
                    if (j < i) {
                        const float gam = fexp(gi - gjA[e]);
                        const float kk = e ? kkv.y : kkv.x;
                        const float dag = -dAg[0][nt][hh * 2 + e];
                        const float s = dag * bi * kk * gam;
                        rs[hh] += s;
                        cs[e] += s;
                        const float da = -dA1[0][nt][hh * 2 + e] + dag * gam;
                        rb[hh] += da * kk;
                        dkk[e] = bi * da;
                    }
                }
                *reinterpret_cast<uint32_t*>(sQK + i * LDP + cw * 32 + nt * 8 + lc2) = pack_bf16(dkk[0], dkk[1]);
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) cs[e] += __shfl_xor_sync(0xffffffffu, cs[e], d);
                if (lr == 0) pColG_A[rbw * CH + cw * 32 + nt * 8 + lc2 + e] = -cs[e];
            }
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            rs[hh] += __shfl_xor_sync(0xffffffffu, rs[hh], 1);
            rs[hh] += __shfl_xor_sync(0xffffffffu, rs[hh], 2);
            rb[hh] += __shfl_xor_sync(0xffffffffu, rb[hh], 1);
            rb[hh] += __shfl_xor_sync(0xffffffffu, rb[hh], 2);
            if ((lane & 3) == 0) {
                pRowG_A[cw * CH + r0 + lr + hh * 8] = rs[hh];
                pRowB_A[cw * CH + r0 + lr + hh * 8] = rb[hh];
            }
        }
    }
    __syncthreads();                           // dKK complete (in the QK tile)
    STAMP();
    // ---- dq = d_qd exp(G) + dQK k ;  dk += dQK^T q + (dKK + dKK^T) k
    {
        const int c0 = cw * (KD / 2);
        float acc[1][2 * NPK][4];
        zero_acc(acc);
        float2 pre[2 * NPK][2];
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
                pre[nt][hh] = *reinterpret_cast<const float2*>(p.d_qd + (rowbase + (long)(r0 + lr + hh * 8) * p.H) * KD + c0 + nt * 8 + lc2);
        warp_gemm<1, NPK, false, true>(acc, sDQK, LDP, r0, sK, LDK, c0, CH, lane);
        STAMP();
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = c0 + nt * 8 + lc2;
                const long off = (rowbase + (long)i * p.H) * KD + j;
                const float2 d = pre[nt][hh];
                const float eg = sEG[i];
                *reinterpret_cast<float2*>(p.dq + off) = make_float2(acc[0][nt][hh * 2] + d.x * eg, acc[0][nt][hh * 2 + 1] + d.y * eg);
            }
        STAMP();
        warp_gemm<1, NPK, true, true>(dk_acc, sDQK, LDP, r0, sQ, LDK, c0, CH, lane);
        warp_gemm<1, NPK, false, true>(dk_acc, sQK, LDP, r0, sK, LDK, c0, CH, lane);
        warp_gemm<1, NPK, true, true>(dk_acc, sQK, LDP, r0, sK, LDK, c0, CH, lane);
        STAMP();
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + lr + hh * 8, j = c0 + nt * 8 + lc2;
                *reinterpret_cast<float2*>(p.dk + (rowbase + (long)i * p.H) * KD + j) = make_float2(dk_acc[0][nt][hh * 2], dk_acc[0][nt][hh * 2 + 1]);
            }
    }
    STAMP();
    // ---- dg = reverse cumulative sum of dG (the chunk total also collects the state-decay part and
    //      the total of d_kd . kd) ;  dbeta ;  d lambda of the intra-chunk levels
    if (warp == 0) {
        // dG of a token: the row terms plus every stage's partial sums
        auto dg_total = [&](int i) {
            float t = sDG[i];
#pragma unroll
            for (int r = 0; r < 4; ++r) t += pColG_P[r * CH + i] + pColG_A[r * CH + i];
#pragma unroll
            for (int r = 0; r < 2; ++r) t += pRowG_P[r * CH + i] + pRowG_A[r * CH + i];
            return t;
        };
        float x0 = dg_total(CH - 1 - 2 * lane), x1 = dg_total(CH - 2 - 2 * lane);   // reversed order
        if (lane == 0) x0 += sMisc[0] + p.d_gl[((long)b * p.NT + c) * p.H + h];
        warp_cumsum64(x0, x1, lane);
        p.dg[rowbase + (long)(CH - 1 - 2 * lane) * p.H] = x0;
        p.dg[rowbase + (long)(CH - 2 - 2 * lane) * p.H] = x1;
    }
    if (tid >= 64 && tid < 128) {
        const int i = tid - 64;
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 4; ++r) t += pColB_P[r * CH + i];
#pragma unroll
        for (int r = 0; r < 2; ++r) t += pRowB_V[r * CH + i] + pRowB_K[r * CH + i] + pRowB_A[r * CH + i];
        p.dbeta[rowbase + (long)i * p.H] = t;
    }
    for (int e = tid; e < CH * 8; e += 256) {
        const int i = e >> 3, lv = e & 7;
        if (lv < INTRA_LEVELS) p.dl[(rowbase + (long)i * p.H) * p.L + lv] = sDL[e];
    }
    STAMP();
}

template <int KD, int VD, bool FUSED>
static int launch_chunk(const GdnParams& p, cudaStream_t stream) {
    auto kern = gdn_bwd_chunk_kernel<KD, VD, FUSED>;
    const size_t sm = ChunkBwdSmem<KD, VD>::total;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
    kern<<<p.B * p.NT * p.H, 256, sm, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

int gdn_bwd_chunk_dispatch(const GdnParams& p, cudaStream_t stream) {
    const bool fused = p.dqd_neg != nullptr && p.d_grow != nullptr;
    if (p.K == 128 && p.V == 128) return fused ? launch_chunk<128, 128, true>(p, stream) : launch_chunk<128, 128, false>(p, stream);
    if (p.K == 128 && p.V == 64) return fused ? launch_chunk<128, 64, true>(p, stream) : launch_chunk<128, 64, false>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace llattn

#ifdef LLATTN_STAMPS
extern "C" int llattn_debug_read_stamps_gdn_chunk(long long* host_dst) {
    return (int)cudaMemcpyFromSymbol(host_dst, llattn::g_stamps, sizeof(llattn::g_stamps));
}
#endif
