// Log-linear Gated DeltaNet chunkwise forward for sm_100a.
//
// Reference being replaced: hattention/chunkwise_hgdn.py:566-788 (driver) with
// fla_future/chunk_scaled_dot_kkt.py, solve_tril.py, wy_fast.py, chunk_delta_h.py and the
// kernels chunk_fwd_kernel_o_intra / chunk_fwd_kernel_o.  Mathematics (per head; G = in-chunk
// cumulative log decay, gl = G at the chunk end, Gamma_ij = exp(G_i - G_j) for j <= i):
//   A  = stril(beta_i k_i.k_j)        Aw = (I + A)^-1          w = Aw (beta k)
//   Ag = A * Gamma                    Au = (I + Ag)^-1         u = Au (beta v)
//   kd = k exp(gl - G)   wd = w exp(G)   qd_i = exp(G_i) (q_i - sum_{j<=i} (q_i.k_j) w_j)
//   intra:  o_c = ((tril(q k^T) Aw) * Gamma * beta_j * lambda[i, bit_length(i^j)]) v_c
//   levels: every level state obeys  H <- exp(gl) H + kd^T (u [if the chunk contributes] - wd H)
//           and a chunk whose bit is set reads  o_i += lambda[i, level] (qd_i . H).
// Two kernels instead of ~6 launches plus per-level torch copies:
//   gdn_chunk_prep_kernel : one CTA per (batch, head, chunk): UT transform (64x64 triangular
//       inverses by per-column forward substitution in fp32), w, u, kd, wd, qd and the intra output.
//   gdn_scan_kernel       : one CTA per (batch, head, 32-column slice of V), sequential over chunks.
//       The level states form a binary-indexed tree over chunks: a chunk reads the states of its
//       set bits; because the transition is the same linear map for every level, the states that a
//       carry merges are summed BEFORE the transition, so a chunk costs popcount(c) products
//       [qd; wd] H (readers and transition share one 128-row product) and 1 + (kept states)
//       products kd^T (.), about half of the per-level formulation.  fp32 masters in registers.
#include "llattn_common.cuh"
#include "llattn_gdn.h"
#include "llattn_mamba2.h"

namespace llattn {

// ------------------------------------------------------------------------------------------
// chunk-parallel preparation
// ------------------------------------------------------------------------------------------
template <int KD, int VD>
struct PrepSmem {
    static constexpr int LDK = KD + PAD, LDV = VD + PAD, LDP = CH + PAD, LDA = CH + 4;
    static constexpr size_t q_off = 0;                                   // bf16 [64][LDK]
    static constexpr size_t k_off = q_off + 1ull * CH * LDK * 2;
    static constexpr size_t v_off = k_off + 1ull * CH * LDK * 2;          // bf16 [64][LDV]
    static constexpr size_t bk_off = v_off + 1ull * CH * LDV * 2;         // beta*k, later w
    static constexpr size_t bv_off = bk_off + 1ull * CH * LDK * 2;        // beta*v
    static constexpr size_t a_off = bv_off + 1ull * CH * LDV * 2;         // float [64][LDA]  A
    static constexpr size_t ag_off = a_off + 1ull * CH * LDA * 4;         // float [64][LDA]  A*Gamma
    static constexpr size_t qk_off = ag_off + 1ull * CH * LDA * 4;        // bf16 [64][LDP] tril(q k^T), later P
    static constexpr size_t aw_off = qk_off + 1ull * CH * LDP * 2;        // bf16 [64][LDP]
    static constexpr size_t au_off = aw_off + 1ull * CH * LDP * 2;
    static constexpr size_t gc_off = au_off + 1ull * CH * LDP * 2;        // float [64] G
    static constexpr size_t be_off = gc_off + CH * 4;                     // float [64] beta
    static constexpr size_t lam_off = be_off + CH * 4;                    // float [64][8]
    static constexpr size_t x_off = lam_off + CH * 8 * 4;                 // float [2][64][LDA] the two inverses in fp32
    static constexpr size_t t_off = x_off + 128ull * LDA * 4;             // float [2][3][16][16] block products of the inversion
    static constexpr size_t total = t_off + 2ull * 3 * 16 * 16 * 4;
};

// FROM_SAVED = true is the backward's recomputation: G and the two inverses are read back instead of
// being solved for, and the intra-chunk output is skipped.
template <int KD, int VD, bool FROM_SAVED>
__global__ void __launch_bounds__(256, 1) gdn_chunk_prep_kernel(const GdnParams p) {
    using SM = PrepSmem<KD, VD>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, LDP = SM::LDP, LDA = SM::LDA;
    constexpr int NPK = KD / 32, NPV = VD / 32;
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sK = reinterpret_cast<bf16*>(smem + SM::k_off);
    bf16* sV = reinterpret_cast<bf16*>(smem + SM::v_off);
    bf16* sBK = reinterpret_cast<bf16*>(smem + SM::bk_off);
    bf16* sBV = reinterpret_cast<bf16*>(smem + SM::bv_off);
    float* sA = reinterpret_cast<float*>(smem + SM::a_off);
    float* sAg = reinterpret_cast<float*>(smem + SM::ag_off);
    bf16* sQK = reinterpret_cast<bf16*>(smem + SM::qk_off);
    bf16* sAw = reinterpret_cast<bf16*>(smem + SM::aw_off);
    bf16* sAu = reinterpret_cast<bf16*>(smem + SM::au_off);
    float* sGc = reinterpret_cast<float*>(smem + SM::gc_off);
    float* sBe = reinterpret_cast<float*>(smem + SM::be_off);
    float* sLam = reinterpret_cast<float*>(smem + SM::lam_off);
    float* sX = reinterpret_cast<float*>(smem + SM::x_off);
    float* sT = reinterpret_cast<float*>(smem + SM::t_off);
    // bf16 copies of wd and kd for the product kd^T wd; they take the place of A and A * Gamma once the
    // triangular solves are done
    static_assert(CH * LDK * 2 <= CH * LDA * 4, "the bf16 tiles fit the fp32 matrices they replace");
    bf16* sWdS = reinterpret_cast<bf16*>(smem + SM::a_off);
    bf16* sKdS = reinterpret_cast<bf16*>(smem + SM::ag_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int c = (blockIdx.x / p.H) % p.NT;
    const int b = blockIdx.x / (p.H * p.NT);
    const long t0 = (long)c * CH;
    const long rowbase = ((long)b * p.T + t0) * p.H + h;        // index of (b, t0, h) in (B,T,H)
    const int wr = warp & 3, wc = warp >> 2;
    const int row0 = wr * 16;
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;

    load_tile_async<CH, KD, 256>(sQ, p.q + rowbase * KD, (long)p.H * KD, tid);
    load_tile_async<CH, KD, 256>(sK, p.k + rowbase * KD, (long)p.H * KD, tid);
    load_tile_async<CH, VD, 256>(sV, p.v + rowbase * VD, (long)p.H * VD, tid);
    cp_async_commit();
    if (warp == 0) {
        if (FROM_SAVED) {
            sGc[2 * lane] = p.g_cum[rowbase + (long)(2 * lane) * p.H];
            sGc[2 * lane + 1] = p.g_cum[rowbase + (long)(2 * lane + 1) * p.H];
        } else {
            float x0 = p.g[rowbase + (long)(2 * lane) * p.H], x1 = p.g[rowbase + (long)(2 * lane + 1) * p.H];
            warp_cumsum64(x0, x1, lane);
            sGc[2 * lane] = x0;
            sGc[2 * lane + 1] = x1;
            p.g_cum[rowbase + (long)(2 * lane) * p.H] = x0;
            p.g_cum[rowbase + (long)(2 * lane + 1) * p.H] = x1;
        }
    }
    if (FROM_SAVED) {
        for (int e = tid; e < 2 * CH * (CH / 8); e += 256) {
            const int which = e / (CH * (CH / 8)), r = (e / (CH / 8)) % CH, c8 = (e % (CH / 8)) * 8;
            const bf16* src = (which ? p.Au : p.Aw) + (rowbase + (long)r * p.H) * CH + c8;
            *reinterpret_cast<uint4*>((which ? sAu : sAw) + r * LDP + c8) = *reinterpret_cast<const uint4*>(src);
        }
    }
    if (tid >= 64 && tid < 128) sBe[tid - 64] = __bfloat162float(p.beta[rowbase + (long)(tid - 64) * p.H]);
    for (int e = tid; e < CH * 8; e += 256) {
        const int i = e >> 3, lv = e & 7;
        sLam[e] = (lv < INTRA_LEVELS) ? __bfloat162float(p.l[(rowbase + (long)i * p.H) * p.L + lv]) : 0.f;
    }
    cp_async_wait<0>();
    __syncthreads();
    const float glast = sGc[CH - 1];

    // ---- A = stril(beta_i k_i.k_j), Ag = A * Gamma (fp32);  QK = tril(q k^T) (bf16)
    {
        float accK[1][4][4], accQ[1][4][4];
        zero_acc(accK);
        zero_acc(accQ);
        warp_gemm<1, 2, false, false>(accK, sK, LDK, row0, sK, LDK, wc * 32, KD, lane);
        warp_gemm<1, 2, false, false>(accQ, sQ, LDK, row0, sK, LDK, wc * 32, KD, lane);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = row0 + lr + hh * 8;
                const int j = wc * 32 + nt * 8 + lc2;
                const float bi = sBe[i], gi = sGc[i];
                float qk[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int jj = j + e;
                    if (!FROM_SAVED) {
                        const float a = (jj < i) ? bi * accK[0][nt][hh * 2 + e] : 0.f;
                        sA[i * LDA + jj] = a;
                        sAg[i * LDA + jj] = (jj < i) ? a * fexp(gi - sGc[jj]) : 0.f;
                    }
                    qk[e] = (jj <= i) ? accQ[0][nt][hh * 2 + e] : 0.f;
                }
                *reinterpret_cast<uint32_t*>(sQK + i * LDP + j) = pack_bf16(qk[0], qk[1]);
            }
    }
    // beta-scaled copies of k and v (operands of w and u)
    for (int e = tid; e < CH * KD / 2; e += 256) {
        const int i = e / (KD / 2), cc = (e % (KD / 2)) * 2;
        const float bi = sBe[i];
        __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(sK + i * LDK + cc);
        *reinterpret_cast<uint32_t*>(sBK + i * LDK + cc) = pack_bf16(__bfloat162float(x.x) * bi, __bfloat162float(x.y) * bi);
    }
    for (int e = tid; e < CH * VD / 2; e += 256) {
        const int i = e / (VD / 2), cc = (e % (VD / 2)) * 2;
        const float bi = sBe[i];
        __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(sV + i * LDV + cc);
        *reinterpret_cast<uint32_t*>(sBV + i * LDV + cc) = pack_bf16(__bfloat162float(x.x) * bi, __bfloat162float(x.y) * bi);
    }
    __syncthreads();

    // ---- (I + A)^-1 and (I + Ag)^-1 (unit lower triangular, fp32), blocked with 16 x 16 blocks:
    //      diagonal blocks by forward substitution (one column per thread, 16 rows, registers), then block diagonal
    //      by block diagonal  X_ij = -X_ii (sum_{k=j..i-1} M_ik X_kj).  The fully unrolled 64-row substitution this
    //      replaces was 80 KB of straight-line code on a 64-step dependent chain.
    if (!FROM_SAVED) {
        constexpr int BS = 16, NB = CH / BS;
        if (tid < 128) {
            const int m = tid >> 6, col = tid & 63, bi = col / BS, cc = col % BS;
            const float* M = (m ? sAg : sA) + (bi * BS) * LDA + bi * BS;
            float x[BS];
#pragma unroll
            for (int i = 0; i < BS; ++i) {
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int j4 = 0; j4 < i; j4 += 4) {
                    const float4 mm = *reinterpret_cast<const float4*>(M + i * LDA + j4);   // entries with j >= i are zero
                    a0 += mm.x * x[j4];
                    if (j4 + 1 < i) a1 += mm.y * x[j4 + 1];
                    if (j4 + 2 < i) a2 += mm.z * x[j4 + 2];
                    if (j4 + 3 < i) a3 += mm.w * x[j4 + 3];
                }
                x[i] = ((i == cc) ? 1.f : 0.f) - ((a0 + a1) + (a2 + a3));
            }
            float* X = sX + (m * CH + bi * BS) * LDA + col;
#pragma unroll
            for (int i = 0; i < BS; ++i) X[i * LDA] = x[i];
        }
        __syncthreads();
#pragma unroll 1
        for (int d = 1; d < NB; ++d) {
            const int nb = NB - d;                 // blocks on this block diagonal, per matrix
            // T_i = sum_{k = i-d .. i-1} M_ik X_{k, i-d}: a thread computes four adjacent columns of one row
            for (int it = tid; it < 2 * nb * BS * 4; it += 256) {
                const int cq = it & 3, r = (it >> 2) & 15, ib = (it >> 6) % nb, m = (it >> 6) / nb;
                const int i = d + ib, j = i - d;
                const float* Mrow = (m ? sAg : sA) + (i * BS + r) * LDA + j * BS;
                const float* Xc = sX + (m * CH + j * BS) * LDA + j * BS + cq * 4;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (int kb = 0; kb < d; ++kb) {
#pragma unroll
                    for (int k4 = 0; k4 < BS; k4 += 4) {
                        const float4 mm = *reinterpret_cast<const float4*>(Mrow + kb * BS + k4);
                        const float mv[4] = {mm.x, mm.y, mm.z, mm.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float4 xv = *reinterpret_cast<const float4*>(Xc + (kb * BS + k4 + e) * LDA);
                            acc.x += mv[e] * xv.x;
                            acc.y += mv[e] * xv.y;
                            acc.z += mv[e] * xv.z;
                            acc.w += mv[e] * xv.w;
                        }
                    }
                }
                *reinterpret_cast<float4*>(sT + ((m * 3 + ib) * BS + r) * BS + cq * 4) = acc;
            }
            __syncthreads();
            // X_{i, i-d} = -X_ii T_i
            for (int it = tid; it < 2 * nb * BS * 4; it += 256) {
                const int cq = it & 3, r = (it >> 2) & 15, ib = (it >> 6) % nb, m = (it >> 6) / nb;
                const int i = d + ib, j = i - d;
                const float* Xii = sX + (m * CH + i * BS + r) * LDA + i * BS;
                const float* T = sT + ((m * 3 + ib) * BS) * BS + cq * 4;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int k4 = 0; k4 < BS; k4 += 4) {
                    const float4 xx = *reinterpret_cast<const float4*>(Xii + k4);
                    const float xs[4] = {xx.x, xx.y, xx.z, xx.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float4 tv = *reinterpret_cast<const float4*>(T + (k4 + e) * BS);
                        acc.x -= xs[e] * tv.x;
                        acc.y -= xs[e] * tv.y;
                        acc.z -= xs[e] * tv.z;
                        acc.w -= xs[e] * tv.w;
                    }
                }
                *reinterpret_cast<float4*>(sX + (m * CH + i * BS + r) * LDA + j * BS + cq * 4) = acc;
            }
            __syncthreads();
        }
        // bf16 copies for the products below and, as whole rows (16-byte stores), for the backward
        for (int e = tid; e < 2 * CH * (CH / 8); e += 256) {
            const int which = e / (CH * (CH / 8)), r = (e / (CH / 8)) % CH, c8 = (e % (CH / 8)) * 8;
            const float* X = sX + (which * CH + r) * LDA + c8;
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                // blocks above the block diagonal were never written: they are zero
                const bool z = (c8 / BS) > (r / BS);
                w[q] = z ? 0u : pack_bf16(X[2 * q], X[2 * q + 1]);
            }
            const uint4 v4 = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>((which ? sAu : sAw) + r * LDP + c8) = v4;
            *reinterpret_cast<uint4*>((which ? p.Au : p.Aw) + (rowbase + (long)r * p.H) * CH + c8) = v4;
        }
    }
    __syncthreads();

    // ---- w = Aw (beta k) -> wd = w exp(G);  u = Au (beta v);  kd = k exp(gl - G)
    {
        float acc[1][2 * NPK][4];
        zero_acc(acc);
        const int colk = wc * (KD / 2);
        warp_gemm<1, NPK, false, true>(acc, sAw, LDP, row0, sBK, LDK, colk, CH, lane);
        __syncthreads();                       // every warp is done reading beta*k: reuse the buffer for w
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = row0 + lr + hh * 8;
                const int cc = colk + nt * 8 + lc2;
                const float eg = fexp(sGc[i]);
                *reinterpret_cast<uint32_t*>(sBK + i * LDK + cc) = pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
                const uint32_t wdx = pack_bf16(acc[0][nt][hh * 2] * eg, acc[0][nt][hh * 2 + 1] * eg);
                *reinterpret_cast<uint32_t*>(p.wd + (rowbase + (long)i * p.H) * KD + cc) = wdx;
                *reinterpret_cast<uint32_t*>(sWdS + i * LDK + cc) = wdx;
            }
    }
    {
        float acc[1][2 * NPV][4];
        zero_acc(acc);
        const int colv = wc * (VD / 2);
        warp_gemm<1, NPV, false, true>(acc, sAu, LDP, row0, sBV, LDV, colv, CH, lane);
#pragma unroll
        for (int nt = 0; nt < 2 * NPV; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = row0 + lr + hh * 8;
                *reinterpret_cast<uint32_t*>(p.u + (rowbase + (long)i * p.H) * VD + colv + nt * 8 + lc2) =
                    pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
            }
    }
    for (int e = tid; e < CH * KD / 2; e += 256) {
        const int i = e / (KD / 2), cc = (e % (KD / 2)) * 2;
        const float sc = fexp(glast - sGc[i]);
        __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(sK + i * LDK + cc);
        const uint32_t kdx = pack_bf16(__bfloat162float(x.x) * sc, __bfloat162float(x.y) * sc);
        *reinterpret_cast<uint32_t*>(p.kd + (rowbase + (long)i * p.H) * KD + cc) = kdx;
        *reinterpret_cast<uint32_t*>(sKdS + i * LDK + cc) = kdx;
    }
    __syncthreads();                           // w is complete in shared memory

    // ---- qd = exp(G) (q - tril(q k^T) w)
    {
        float acc[1][2 * NPK][4];
        zero_acc(acc);
        const int colk = wc * (KD / 2);
        warp_gemm<1, NPK, false, true>(acc, sQK, LDP, row0, sBK, LDK, colk, CH, lane);
#pragma unroll
        for (int nt = 0; nt < 2 * NPK; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = row0 + lr + hh * 8;
                const int cc = colk + nt * 8 + lc2;
                const float eg = fexp(sGc[i]);
                __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(sQ + i * LDK + cc);
                *reinterpret_cast<uint32_t*>(p.qd + (rowbase + (long)i * p.H) * KD + cc) =
                    pack_bf16((__bfloat162float(x.x) - acc[0][nt][hh * 2]) * eg, (__bfloat162float(x.y) - acc[0][nt][hh * 2 + 1]) * eg);
            }
    }
    // ---- Wd = (exp(gl) - 1) I - kd^T wd (K x K): with it the transition of a level state is  H' = H + Wd H
    //      (+ kd^T u), one accumulating product per level for the sequential scans instead of two dependent ones
    if (p.wk != nullptr) {
        const float decm1 = fexp(glast) - 1.f;
        float acc[1][KD / 8][4];
        zero_acc(acc);
        const int m0 = warp * 16;              // 8 warps x 16 rows = K = 128
        static_assert(KD == 128, "one 16-row block of Wd per warp");
        warp_gemm<1, KD / 16, true, true>(acc, sKdS, LDK, m0, sWdS, LDK, 0, CH, lane);
        bf16* dst = p.wk + ((((long)b * p.NT + c) * KD) * p.H + h) * KD;
#pragma unroll
        for (int nt = 0; nt < KD / 8; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int r = m0 + lr + hh * 8, cc = nt * 8 + lc2;
                const float x0 = -acc[0][nt][hh * 2] + (r == cc ? decm1 : 0.f), x1 = -acc[0][nt][hh * 2 + 1] + (r == cc + 1 ? decm1 : 0.f);
                *reinterpret_cast<uint32_t*>(dst + (long)r * p.H * KD + cc) = pack_bf16(x0, x1);
            }
    }
    if (FROM_SAVED) return;
    // ---- P = (tril(q k^T) Aw) * Gamma * beta_j * lambda ; o = P v
    {
        float acc[1][4][4];
        zero_acc(acc);
        warp_gemm<1, 2, false, true>(acc, sQK, LDP, row0, sAw, LDP, wc * 32, CH, lane);
        __syncthreads();                       // qd product above is done with tril(q k^T): overwrite it with P
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = row0 + lr + hh * 8;
                const int j = wc * 32 + nt * 8 + lc2;
                const float gi = sGc[i];
                float pv[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int jj = j + e;
                    pv[e] = (jj <= i) ? acc[0][nt][hh * 2 + e] * fexp(gi - sGc[jj]) * sBe[jj] * sLam[i * 8 + level_of(i, jj)] : 0.f;
                }
                *reinterpret_cast<uint32_t*>(sQK + i * LDP + j) = pack_bf16(pv[0], pv[1]);
            }
    }
    __syncthreads();
    {
        float acc[1][2 * NPV][4];
        zero_acc(acc);
        const int colv = wc * (VD / 2);
        warp_gemm<1, NPV, false, true>(acc, sQK, LDP, row0, sV, LDV, colv, CH, lane);
#pragma unroll
        for (int nt = 0; nt < 2 * NPV; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = row0 + lr + hh * 8;
                *reinterpret_cast<uint32_t*>(p.o + (rowbase + (long)i * p.H) * VD + colv + nt * 8 + lc2) =
                    pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
            }
    }
}

// ------------------------------------------------------------------------------------------
// sequential scan over chunks with binary-indexed level states
// ------------------------------------------------------------------------------------------

template <int KD>
struct ScanSmem {
    static constexpr int LDK = KD + PAD, LDS = GDN_VS + PAD;
    static constexpr size_t qw_off = 0;                                         // bf16 [128][LDK]: rows 0..63 qd, 64..127 wd (single buffer)
    static constexpr size_t kd_off = qw_off + 1ull * 128 * LDK * 2;             // bf16 [2][64][LDK]
    static constexpr size_t u_off = kd_off + 2ull * CH * LDK * 2;               // bf16 [2][64][LDS]
    static constexpr size_t st_off = u_off + 2ull * CH * LDS * 2;               // bf16 [MAXLEV][KD][LDS] state copies
    static constexpr size_t vh_off = st_off + (size_t)GDN_MAXLEV * KD * LDS * 2;   // bf16 [MAXLEV+1][64][LDS] (u - Z) operands
    static constexpr size_t lam_off = vh_off + (size_t)(GDN_MAXLEV + 1) * CH * LDS * 2;   // float [2][64][MAXLEV]
    static constexpr size_t gl_off = lam_off + 2ull * CH * GDN_MAXLEV * 4;      // float [2]
    static constexpr size_t total = gl_off + 16;
};

// SAVE = true also writes, for every chunk, the bf16 level states that the chunk reads:
// hs[((b*H + h)*nvs + vs)*NT + c][level][KD][32] (the backward's recomputation, or a forward whose caller
// keeps the workspace for the backward); OUT = false skips the output (recomputation only).
template <int KD, bool SAVE, bool OUT>
__global__ void __launch_bounds__(256, 1) gdn_scan_kernel(const GdnParams p) {
    using SM = ScanSmem<KD>;
    constexpr int LDK = SM::LDK, LDS = SM::LDS;
    constexpr int MT = KD / 128;               // state rows per warp = 16 * MT (8 warps over KD rows)
    static_assert(KD % 128 == 0, "state rows are split over 8 warps");
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQW = reinterpret_cast<bf16*>(smem + SM::qw_off);
    bf16* sKd = reinterpret_cast<bf16*>(smem + SM::kd_off);
    bf16* sU = reinterpret_cast<bf16*>(smem + SM::u_off);
    bf16* sSt = reinterpret_cast<bf16*>(smem + SM::st_off);
    bf16* sVh = reinterpret_cast<bf16*>(smem + SM::vh_off);
    float* sLam = reinterpret_cast<float*>(smem + SM::lam_off);
    float* sGl = reinterpret_cast<float*>(smem + SM::gl_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nvs = p.V / GDN_VS;
    const int vs = blockIdx.x % nvs;
    const int h = (blockIdx.x / nvs) % p.H;
    const int b = blockIdx.x / (nvs * p.H);
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
    const int nlev = p.NLEV;                   // ceil(log2(NT))

    // qd / wd feed the first product of a chunk only, so one buffer is refilled as soon as that
    // product is done; kd and u (second product) are double buffered
    auto issue_qw = [&](int c) {
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
        load_tile_async<CH, KD, 256>(sQW, p.qd + rowbase * KD, (long)p.H * KD, tid);
        load_tile_async<CH, KD, 256>(sQW + 64 * LDK, p.wd + rowbase * KD, (long)p.H * KD, tid);
        cp_async_commit();
    };
    auto issue_ku = [&](int c, int st) {
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
        load_tile_async<CH, KD, 256>(sKd + st * CH * LDK, p.kd + rowbase * KD, (long)p.H * KD, tid);
        load_tile_async<CH, GDN_VS, 256>(sU + st * CH * LDS, p.u + rowbase * p.V + vs * GDN_VS, (long)p.H * p.V, tid);
        cp_async_commit();
    };
    float lam_reg[(CH * GDN_MAXLEV + 255) / 256];
    float gl_reg = 0.f;
    auto fetch_small = [&](int c) {
        const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
#pragma unroll
        for (int i = 0; i < (CH * GDN_MAXLEV + 255) / 256; ++i) {
            const int e = tid + i * 256;
            const int row = e / GDN_MAXLEV, lv = e % GDN_MAXLEV;
            lam_reg[i] = (row < CH && lv < nlev) ? __bfloat162float(p.l[(rowbase + (long)row * p.H) * p.L + INTRA_LEVELS + lv]) : 0.f;
        }
        if (tid == 0) gl_reg = p.g_cum[rowbase + (long)(CH - 1) * p.H];
    };
    auto store_small = [&](int st) {
#pragma unroll
        for (int i = 0; i < (CH * GDN_MAXLEV + 255) / 256; ++i) {
            const int e = tid + i * 256;
            if (e < CH * GDN_MAXLEV) sLam[st * CH * GDN_MAXLEV + e] = lam_reg[i];
        }
        if (tid == 0) sGl[st] = gl_reg;
    };

    // fp32 masters: this warp holds rows [warp*16*MT, +16*MT) x 32 columns of every level state
    float M[GDN_MAXLEV][MT][4][4];
#pragma unroll
    for (int lv = 0; lv < GDN_MAXLEV; ++lv) zero_acc(M[lv]);

    issue_qw(0);
    issue_ku(0, 0);
    fetch_small(0);
    store_small(0);

    for (int c = 0; c < p.NT; ++c) {
        const int st = c & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (c + 1 < p.NT) {
            issue_ku(c + 1, st ^ 1);
            fetch_small(c + 1);
        }
        if (SAVE) {
            bf16* dst = p.hs + ((size_t)blockIdx.x * p.NT + c) * nlev * (KD * GDN_VS);
            for (int lv = 0; lv < nlev; ++lv) {
                if (!((c >> lv) & 1)) continue;
                for (int e = tid; e < KD * (GDN_VS / 8); e += 256) {
                    const int r = e / (GDN_VS / 8), c8 = (e % (GDN_VS / 8)) * 8;
                    *reinterpret_cast<uint4*>(dst + (size_t)lv * KD * GDN_VS + r * GDN_VS + c8) =
                        *reinterpret_cast<const uint4*>(sSt + lv * KD * LDS + r * LDS + c8);
                }
            }
        }
        if (OUT && c == p.NT - 1 && p.final_states != nullptr) {
            // prefill hand-off: the level states every token of the last chunk starts from.  Level 7 + lv holds the block
            // of 2^lv chunks for each set bit lv of c (the binary-indexed tree as it stands before this chunk); the
            // caller steps the last chunk's tokens through the decode kernel, which fills levels 0..6.
            float* dst = p.final_states + ((long)b * p.H + h) * KD * p.V * p.L;
#pragma unroll
            for (int lv = 0; lv < GDN_MAXLEV; ++lv) {
                if (lv < nlev && ((c >> lv) & 1)) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int row = warp * 16 * MT + mt * 16 + lr + (e >> 1) * 8;
                                const int col = vs * GDN_VS + nt * 8 + lc2 + (e & 1);
                                dst[((long)row * p.V + col) * p.L + INTRA_LEVELS + lv] = M[lv][mt][nt][e];
                            }
                }
            }
        }
        const bf16* cQW = sQW;
        const bf16* cKd = sKd + st * CH * LDK;
        const bf16* cU = sU + st * CH * LDS;
        const float* cLam = sLam + st * CH * GDN_MAXLEV;
        const float dec = fexp(sGl[st]);
        const int jc = __ffs(~c) - 1;          // carry: levels 0..jc-1 merge with this chunk's own state into level jc

        // the intra-chunk part of the output rows (written by the preparation kernel) is fetched before the
        // products so that its latency is off the chunk-to-chunk chain
        uint32_t o_in[4][2];
        if (OUT && warp < 4) {
            const long rb = ((long)b * p.T + (long)c * CH) * p.H + h;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    o_in[nt][hh] = *reinterpret_cast<const uint32_t*>(p.o + (rb + (long)(warp * 16 + lr + hh * 8) * p.H) * p.V + vs * GDN_VS + nt * 8 + lc2);
        }
        // ---- [qd; wd] H for every live level: rows 0..63 feed the output, rows 64..127 the transition
        float o_acc[1][4][4];                  // warps 0..3: output rows 16*warp.., 32 columns
        float zsum[1][4][4];                   // warps 4..7: sum over the merged levels of wd H
        zero_acc(o_acc);
        zero_acc(zsum);
#pragma unroll
        for (int lv = 0; lv < GDN_MAXLEV; ++lv) {
            if (lv < nlev && ((c >> lv) & 1)) {
                float acc[1][4][4];
                zero_acc(acc);
                warp_gemm<1, 2, false, true>(acc, cQW, LDK, warp * 16, sSt + lv * KD * LDS, LDS, 0, KD, lane);
                if (warp < 4) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const float lm = cLam[(warp * 16 + lr + hh * 8) * GDN_MAXLEV + lv];
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt) {
                            o_acc[0][nt][hh * 2] += lm * acc[0][nt][hh * 2];
                            o_acc[0][nt][hh * 2 + 1] += lm * acc[0][nt][hh * 2 + 1];
                        }
                    }
                } else if (lv < jc) {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) zsum[0][nt][e] += acc[0][nt][e];
                } else {
                    // a level that stays on its own: operand -wd H
                    bf16* dst = sVh + (lv + 1) * CH * LDS;
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh)
                            *reinterpret_cast<uint32_t*>(dst + ((warp - 4) * 16 + lr + hh * 8) * LDS + nt * 8 + lc2) =
                                pack_bf16(-acc[0][nt][hh * 2], -acc[0][nt][hh * 2 + 1]);
                }
            }
        }
        if (warp >= 4) {
            // merged group (levels below the carry plus this chunk's own writes): operand u - sum wd H
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = (warp - 4) * 16 + lr + hh * 8;
                    __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(cU + i * LDS + nt * 8 + lc2);
                    *reinterpret_cast<uint32_t*>(sVh + i * LDS + nt * 8 + lc2) =
                        pack_bf16(__bfloat162float(x.x) - zsum[0][nt][hh * 2], __bfloat162float(x.y) - zsum[0][nt][hh * 2 + 1]);
                }
        } else if (OUT) {
            // output rows: add the intra-chunk part and store
            const long rowbase = ((long)b * p.T + (long)c * CH) * p.H + h;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    bf16* go = p.o + (rowbase + (long)(warp * 16 + lr + hh * 8) * p.H) * p.V + vs * GDN_VS + nt * 8 + lc2;
                    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&o_in[nt][hh]);
                    *reinterpret_cast<uint32_t*>(go) =
                        pack_bf16(__bfloat162float(x.x) + o_acc[0][nt][hh * 2], __bfloat162float(x.y) + o_acc[0][nt][hh * 2 + 1]);
                }
        }
        __syncthreads();
        if (c + 1 < p.NT) issue_qw(c + 1);

        // ---- transition: merged group -> level jc ; every other live level on its own
        if (c + 1 < p.NT) {
            float nm[MT][4][4];
            zero_acc(nm);
            warp_gemm<MT, 2, true, true>(nm, cKd, LDK, warp * 16 * MT, sVh, LDS, 0, CH, lane);
#pragma unroll
            for (int lv = 0; lv < GDN_MAXLEV; ++lv) {
                if (lv < jc && lv < nlev) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) nm[mt][nt][e] += dec * M[lv][mt][nt][e];
                }
            }
#pragma unroll
            for (int lv = 0; lv < GDN_MAXLEV; ++lv) {
                if (lv >= nlev) continue;
                bool write = false;
                if (lv == jc) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) M[lv][mt][nt][e] = nm[mt][nt][e];
                    write = true;
                } else if (lv > jc && ((c >> lv) & 1)) {
                    float tr[MT][4][4];
                    zero_acc(tr);
                    warp_gemm<MT, 2, true, true>(tr, cKd, LDK, warp * 16 * MT, sVh + (lv + 1) * CH * LDS, LDS, 0, CH, lane);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) M[lv][mt][nt][e] = dec * M[lv][mt][nt][e] + tr[mt][nt][e];
                    write = true;
                }
                if (write) {
                    bf16* dst = sSt + lv * KD * LDS;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh)
                                *reinterpret_cast<uint32_t*>(dst + (warp * 16 * MT + mt * 16 + lr + hh * 8) * LDS + nt * 8 + lc2) =
                                    pack_bf16(M[lv][mt][nt][hh * 2], M[lv][mt][nt][hh * 2 + 1]);
                }
            }
            store_small(st ^ 1);
        }
        // no barrier here: the one at the top of the next chunk orders these writes before their readers
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
template <int KD, int VD, bool BWD, bool KEEP = false>
static int launch_gdn_fwd(const GdnParams& p, cudaStream_t stream) {
    cudaError_t e;
    if (!BWD && KD == 128 && g_use_tensor_core_path.load()) {
        int rc = gdn_prep_tc_dispatch(p, stream);
        if (rc != 0) return rc;
    } else {
        auto kern = gdn_chunk_prep_kernel<KD, VD, BWD>;
        const size_t sm = PrepSmem<KD, VD>::total;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
        kern<<<p.B * p.NT * p.H, 256, sm, stream>>>(p); LLATTN_LAUNCHED();
    }
    if (KD == 128 && g_use_tensor_core_path.load()) return gdn_scan_tc_dispatch(p, BWD ? 2 : (KEEP ? 1 : 0), stream);
    {
        auto kern = gdn_scan_kernel<KD, BWD || KEEP, !BWD>;
        const size_t sm = ScanSmem<KD>::total;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
        kern<<<p.B * p.H * (p.V / GDN_VS), 256, sm, stream>>>(p); LLATTN_LAUNCHED();
    }
    return (int)cudaGetLastError();
}

int gdn_fwd_dispatch(const GdnParams& p, cudaStream_t stream) {
    if (p.K == 128 && p.V == 128) return launch_gdn_fwd<128, 128, false>(p, stream);
    if (p.K == 128 && p.V == 64) return launch_gdn_fwd<128, 64, false>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

// forward that also leaves the level states (and the chunk matrices) in the workspace for the backward
int gdn_fwd_keep_dispatch(const GdnParams& p, cudaStream_t stream) {
    if (p.K == 128 && p.V == 128) return launch_gdn_fwd<128, 128, false, true>(p, stream);
    if (p.K == 128 && p.V == 64) return launch_gdn_fwd<128, 64, false, true>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

// recomputation for the backward: w, u, kd, wd, qd from the saved inverses, then the scan with the
// level states written out
int gdn_recompute_dispatch(const GdnParams& p, cudaStream_t stream) {
    if (p.K == 128 && p.V == 128) return launch_gdn_fwd<128, 128, true>(p, stream);
    if (p.K == 128 && p.V == 64) return launch_gdn_fwd<128, 64, true>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace llattn
