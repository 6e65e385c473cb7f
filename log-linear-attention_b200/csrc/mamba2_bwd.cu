// Log-linear Mamba-2 chunkwise backward for sm_100a.
//
// Reference being replaced: hattention/chunkwise.py:1286-1597 (driver) with kernels
// chunk_bwd_kernel_dh (:299-470), chunk_bwd_kernel_dqkwg (:663-958), chunk_bwd_kernel_dv
// (:973-1115).  Same segment / Fenwick organisation as the forward (see mamba2_fwd.cu):
//
//   m2_bwd_fwdorder_kernel : per (batch, head, segment), chunks in order.  Recomputes the low
//       level states; produces dq (intra + low levels), the intra part of dk, dlambda for the
//       intra and low levels.
//   m2_bwd_revorder_kernel : per (batch, head, segment), chunks in reverse.  Keeps the adjoint
//       low level states (readers insert (q*scale)^T do, contributors read the sum of the levels
//       whose bit is clear) plus the adjoint of the segment summary; produces dv and the level
//       part of dk.
//   m2_hi_bwd_q_kernel / m2_seg_dstate_kernel / m2_seg_dscan_kernel : the high levels at
//       segment granularity (dq, dlambda of readers; adjoint of the segment summaries).
//   m2_dg_kernel : dg = reverse in-chunk cumsum of (q_t.dq_t - k_t.dk_t) plus, per chunk, the
//       gradient carried across the chunk's end, assembled from per-chunk / per-level scalar
//       totals written by the kernels above (the reference's dG bookkeeping,
//       chunkwise.py:793-874, 938, 1596, without materialising h and dh).
// dq / dk are accumulated over the heads of a group in fp32 with red.global.add and converted to
// bf16 at the end (the reference writes per-head bf16 tensors and sums them on the host,
// chunkwise.py:1583-1591).
#include "llattn_common.cuh"
#include "llattn_mamba2.h"

namespace llattn {

// store a 16 x (8*NT) per-warp fp32 fragment block into a fp32 group accumulator with red.add
template <int NT>
__device__ __forceinline__ void red_tile(float* base, long row_stride, int row0, int col0, const float (&acc)[1][NT][4], int lane) {
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float* dst = base + (long)(row0 + lr + hh * 8) * row_stride + col0 + nt * 8 + lc2;
            red_add_f32x2(dst, acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
        }
}

// per-row dot product of a fragment block with a bf16 smem tile; result valid in every lane of a quad
template <int NT>
__device__ __forceinline__ void rowdot_tile(float (&out)[2], const float (&acc)[1][NT][4], const bf16* s, int ld, int row0, int col0, int lane) {
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(s + (row0 + lr + hh * 8) * ld + col0 + nt * 8 + lc2);
            sum += acc[0][nt][hh * 2] * __bfloat162float(x.x) + acc[0][nt][hh * 2 + 1] * __bfloat162float(x.y);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        out[hh] = sum;
    }
}

// ------------------------------------------------------------------------------------------
// forward-order pass
// ------------------------------------------------------------------------------------------
template <int KD, int VD, int MLOW>
struct Bwd1Smem {
    static constexpr int LDK = KD + PAD, LDV = VD + PAD, LDP = CH + PAD;
    static constexpr size_t q_off = 0;
    static constexpr size_t k_off = q_off + 2ull * CH * LDK * 2;
    static constexpr size_t v_off = k_off + 2ull * CH * LDK * 2;
    static constexpr size_t do_off = v_off + 2ull * CH * LDV * 2;
    static constexpr size_t ds_off = do_off + 2ull * CH * LDV * 2;
    static constexpr size_t vs_off = ds_off + 1ull * CH * LDP * 2;
    static constexpr size_t h_off = vs_off + 1ull * CH * LDV * 2;
    static constexpr size_t lam_off = h_off + (size_t)MLOW * KD * LDV * 2;    // float [2][64*MAX_L]
    static constexpr size_t g_off = lam_off + 2ull * CH * MAX_L * 4;
    static constexpr size_t gc_off = g_off + 2ull * CH * 4;
    static constexpr size_t dl_off = gc_off + CH * 4;                          // float [2][64][16]
    static constexpr size_t total = dl_off + 2ull * CH * 16 * 4;
};

template <int KD, int VD, int MLOW>
__global__ void __launch_bounds__(256, 1) m2_bwd_fwdorder_kernel(const Mamba2Params p) {
    using SM = Bwd1Smem<KD, VD, MLOW>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, LDP = SM::LDP;
    constexpr int SEG = 1 << MLOW, MT = KD / 64, NPS = VD / 32, NPK = KD / 32;
    static_assert(INTRA_LEVELS + MLOW <= 16, "dl staging too small");
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sK = reinterpret_cast<bf16*>(smem + SM::k_off);
    bf16* sV = reinterpret_cast<bf16*>(smem + SM::v_off);
    bf16* sDO = reinterpret_cast<bf16*>(smem + SM::do_off);
    bf16* sDS = reinterpret_cast<bf16*>(smem + SM::ds_off);
    bf16* sVs = reinterpret_cast<bf16*>(smem + SM::vs_off);
    bf16* sH = reinterpret_cast<bf16*>(smem + SM::h_off);
    float* sLam = reinterpret_cast<float*>(smem + SM::lam_off);
    float* sG = reinterpret_cast<float*>(smem + SM::g_off);
    float* sGc = reinterpret_cast<float*>(smem + SM::gc_off);
    float* sDL = reinterpret_cast<float*>(smem + SM::dl_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % p.NS;
    const int b = blockIdx.x / (p.H * p.NS);
    const int grp = h / (p.H / p.G);
    const int L = p.L;
    const int nc = min(SEG, p.NT - r * SEG);
    const int wr = warp & 3, wc = warp >> 2;
    const int row0 = wr * 16;
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;

    auto issue_tiles = [&](int cl, int st) {
        const long t0 = (long)(r * SEG + cl) * CH;
        load_tile_async<CH, KD, 256>(sQ + st * CH * LDK, p.q + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, tid);
        load_tile_async<CH, KD, 256>(sK + st * CH * LDK, p.k + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, tid);
        load_tile_async<CH, VD, 256>(sV + st * CH * LDV, p.v + (((long)b * p.T + t0) * p.H + h) * VD, (long)p.H * VD, tid);
        load_tile_async<CH, VD, 256>(sDO + st * CH * LDV, p.d_o + (((long)b * p.T + t0) * p.H + h) * VD, (long)p.H * VD, tid);
        cp_async_commit();
    };
    float lam_reg[(CH * MAX_L) / 256];
    float g_reg = 0.f;
    auto fetch_small = [&](int cl) {
        const long t0 = (long)(r * SEG + cl) * CH;
#pragma unroll
        for (int i = 0; i < (CH * MAX_L) / 256; ++i) {
            int e = tid + i * 256;
            int row = e / L, col = e % L;
            lam_reg[i] = (row < CH) ? __bfloat162float(p.l[(((long)b * p.T + t0 + row) * p.H + h) * L + col]) : 0.f;
        }
        if (tid < CH) g_reg = p.g[((long)b * p.T + t0 + tid) * p.H + h];
    };
    auto store_small = [&](int st) {
#pragma unroll
        for (int i = 0; i < (CH * MAX_L) / 256; ++i) {
            int e = tid + i * 256;
            if (e < CH * L) sLam[st * CH * MAX_L + e] = lam_reg[i];
        }
        if (tid < CH) sG[st * CH + tid] = g_reg;
    };

    float M[MLOW > 0 ? MLOW : 1][MT][2 * NPS][4];
    float dsum[MLOW > 0 ? MLOW : 1];
#pragma unroll
    for (int i = 0; i < (MLOW > 0 ? MLOW : 1); ++i) dsum[i] = 0.f;

    issue_tiles(0, 0);
    fetch_small(0);
    store_small(0);

    for (int cl = 0; cl < nc; ++cl) {
        const int st = cl & 1;
        const long t0 = (long)(r * SEG + cl) * CH;
        if (cl + 1 < nc) {
            issue_tiles(cl + 1, st ^ 1);
            fetch_small(cl + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp == 0) {
            float x0 = sG[st * CH + 2 * lane], x1 = sG[st * CH + 2 * lane + 1];
            warp_cumsum64(x0, x1, lane);
            sGc[2 * lane] = x0;
            sGc[2 * lane + 1] = x1;
        }
        __syncthreads();
        const bf16* cQ = sQ + st * CH * LDK;
        const bf16* cK = sK + st * CH * LDK;
        const bf16* cV = sV + st * CH * LDV;
        const bf16* cDO = sDO + st * CH * LDV;
        const float* cLam = sLam + st * CH * MAX_L;
        const float glast = sGc[CH - 1];

        // ---- S = q k^T, dP = do v^T ; dS = dP * decay * lambda -> sDS ; dlambda (intra) bins
        {
            float accS[1][4][4], accP[1][4][4];
            zero_acc(accS);
            zero_acc(accP);
            warp_gemm<1, 2, false, false>(accS, cQ, LDK, row0, cK, LDK, wc * 32, KD, lane);
            warp_gemm<1, 2, false, false>(accP, cDO, LDV, row0, cV, LDV, wc * 32, VD, lane);
            float bins[2][INTRA_LEVELS];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                for (int lv = 0; lv < INTRA_LEVELS; ++lv) bins[hh][lv] = 0.f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = row0 + lr + hh * 8;
                    const int j = wc * 32 + nt * 8 + lc2;
                    const float gi = sGc[i];
                    float dsv[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int jj = j + e;
                        float val = 0.f;
                        if (jj <= i) {
                            const int lev = level_of(i, jj);
                            const float ed = accP[0][nt][hh * 2 + e] * fexp(gi - sGc[jj]);
                            const float es = ed * accS[0][nt][hh * 2 + e];
#pragma unroll
                            for (int lv = 0; lv < INTRA_LEVELS; ++lv) bins[hh][lv] += (lev == lv) ? es : 0.f;
                            val = ed * cLam[i * L + lev];
                        }
                        dsv[e] = val;
                    }
                    *reinterpret_cast<uint32_t*>(sDS + i * LDP + j) = pack_bf16(dsv[0], dsv[1]);
                }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                for (int lv = 0; lv < INTRA_LEVELS; ++lv) {
                    float x = bins[hh][lv];
                    x += __shfl_xor_sync(0xffffffffu, x, 1);
                    x += __shfl_xor_sync(0xffffffffu, x, 2);
                    if ((lane & 3) == 0) sDL[(wc * CH + row0 + lr + hh * 8) * 16 + lv] = x;
                }
        }
        for (int e = tid; e < CH * VD / 2; e += 256) {
            const int j = e / (VD / 2), c = (e % (VD / 2)) * 2;
            const float sc = fexp(glast - sGc[j]);
            __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(cV + j * LDV + c);
            *reinterpret_cast<uint32_t*>(sVs + j * LDV + c) =
                pack_bf16(__bfloat162float(vv.x) * sc, __bfloat162float(vv.y) * sc);
        }
        __syncthreads();

        float wrow[2] = {0.f, 0.f};    // q.dq - k.dk (intra) for this warp's rows / column half
        // ---- dq = dS k + sum over set low bits lambda*scale * (do . H^T) ; dlambda of those levels
        {
            float acc[1][2 * NPK][4];
            zero_acc(acc);
            const int colk = wc * (KD / 2);
            warp_gemm<1, NPK, false, true>(acc, sDS, LDP, row0, cK, LDK, colk, CH, lane);
#pragma unroll
            for (int lv = 0; lv < MLOW; ++lv) {
                if ((cl >> lv) & 1) {
                    float tmp[1][2 * NPK][4];
                    zero_acc(tmp);
                    warp_gemm<1, NPK, false, false>(tmp, cDO, LDV, row0, sH + lv * KD * LDV, LDV, colk, VD, lane);
                    float rd[2];
                    rowdot_tile<2 * NPK>(rd, tmp, cQ, LDK, row0, colk, lane);
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = row0 + lr + hh * 8;
                        const float sc = fexp(sGc[i] + dsum[lv]);
                        const float rs = cLam[i * L + INTRA_LEVELS + lv] * sc;
                        if ((lane & 3) == 0) sDL[(wc * CH + i) * 16 + INTRA_LEVELS + lv] = sc * rd[hh];
#pragma unroll
                        for (int nt = 0; nt < 2 * NPK; ++nt) {
                            acc[0][nt][hh * 2] += rs * tmp[0][nt][hh * 2];
                            acc[0][nt][hh * 2 + 1] += rs * tmp[0][nt][hh * 2 + 1];
                        }
                    }
                } else {
                    if ((lane & 3) == 0) {
                        sDL[(wc * CH + row0 + lr) * 16 + INTRA_LEVELS + lv] = 0.f;
                        sDL[(wc * CH + row0 + lr + 8) * 16 + INTRA_LEVELS + lv] = 0.f;
                    }
                }
            }
            float rd[2];
            rowdot_tile<2 * NPK>(rd, acc, cQ, LDK, row0, colk, lane);
            wrow[0] += rd[0];
            wrow[1] += rd[1];
            red_tile<2 * NPK>(p.dq_acc + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, row0, colk, acc, lane);
        }
        // ---- dk (intra) = dS^T q
        {
            float acc[1][2 * NPK][4];
            zero_acc(acc);
            const int colk = wc * (KD / 2);
            warp_gemm<1, NPK, true, true>(acc, sDS, LDP, row0, cQ, LDK, colk, CH, lane);
            float rd[2];
            rowdot_tile<2 * NPK>(rd, acc, cK, LDK, row0, colk, lane);
            wrow[0] -= rd[0];
            wrow[1] -= rd[1];
            red_tile<2 * NPK>(p.dk_acc + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, row0, colk, acc, lane);
        }
        if ((lane & 3) == 0) {
            float* wp = p.wq + ((long)b * p.T + t0) * p.H + h;
            red_add_f32(wp + (long)(row0 + lr) * p.H, wrow[0]);
            red_add_f32(wp + (long)(row0 + lr + 8) * p.H, wrow[1]);
        }

        // ---- recompute KV_c and carry the low level states (same as the forward)
        if (MLOW > 0 && cl + 1 < nc) {
            const int j = __ffs(~cl) - 1;
            if (j < MLOW) {
                float kv[MT][2 * NPS][4];
                zero_acc(kv);
                warp_gemm<MT, NPS, true, true>(kv, cK, LDK, wr * 16 * MT, sVs, LDV, wc * (VD / 2), CH, lane);
#pragma unroll
                for (int lv = 0; lv < MLOW; ++lv) {
                    if (lv < j) {
                        const float dec = fexp(dsum[lv] + glast);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                            for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
                                for (int e = 0; e < 4; ++e) kv[mt][nt][e] += dec * M[lv][mt][nt][e];
                    }
                }
#pragma unroll
                for (int lv = 0; lv < MLOW; ++lv) {
                    if (lv == j) {
                        bf16* dst = sH + lv * KD * LDV;
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                            for (int nt = 0; nt < 2 * NPS; ++nt) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) M[lv][mt][nt][e] = kv[mt][nt][e];
#pragma unroll
                                for (int hh = 0; hh < 2; ++hh) {
                                    const int rr = wr * 16 * MT + mt * 16 + lr + hh * 8;
                                    const int cc = wc * (VD / 2) + nt * 8 + lc2;
                                    *reinterpret_cast<uint32_t*>(dst + rr * LDV + cc) =
                                        pack_bf16(kv[mt][nt][hh * 2], kv[mt][nt][hh * 2 + 1]);
                                }
                            }
                        dsum[lv] = 0.f;
                    } else {
                        dsum[lv] += glast;
                    }
                }
            } else {
#pragma unroll
                for (int lv = 0; lv < MLOW; ++lv) dsum[lv] += glast;
            }
        }
        if (cl + 1 < nc) store_small(st ^ 1);
        __syncthreads();
        // ---- dlambda for the intra and low levels of this chunk (single writer per entry)
        for (int e = tid; e < CH * (INTRA_LEVELS + MLOW); e += 256) {
            const int i = e / (INTRA_LEVELS + MLOW), lv = e % (INTRA_LEVELS + MLOW);
            if (lv < L) p.dl[(((long)b * p.T + t0 + i) * p.H + h) * L + lv] = sDL[i * 16 + lv] + sDL[(CH + i) * 16 + lv];
        }
        // reader totals Z[c][lv] = sum_i lambda_i * dlambda_i for the low levels read by this chunk
        if (warp < MLOW && ((cl >> warp) & 1)) {
            const int col = INTRA_LEVELS + warp;
            float z = 0.f;
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int i = lane + rr * 32;
                z += cLam[i * L + col] * (sDL[i * 16 + col] + sDL[(CH + i) * 16 + col]);
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) z += __shfl_xor_sync(0xffffffffu, z, d);
            if (lane == 0) p.Zc[(((long)b * p.H + h) * p.NT + r * SEG + cl) * p.LZ + warp] = z;
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// reverse-order pass
// ------------------------------------------------------------------------------------------
template <int KD, int VD, int MLOW>
struct Bwd2Smem {
    static constexpr int LDK = KD + PAD, LDV = VD + PAD, LDP = CH + PAD;
    static constexpr size_t q_off = 0;
    static constexpr size_t k_off = q_off + 2ull * CH * LDK * 2;
    static constexpr size_t v_off = k_off + 2ull * CH * LDK * 2;
    static constexpr size_t do_off = v_off + 2ull * CH * LDV * 2;
    static constexpr size_t p_off = do_off + 2ull * CH * LDV * 2;
    static constexpr size_t vs_off = p_off + 1ull * CH * LDP * 2;
    static constexpr size_t dkv_off = vs_off + 1ull * CH * LDV * 2;            // bf16 [KD][LDV]
    static constexpr size_t qs_off = dkv_off + 1ull * KD * LDV * 2;            // bf16 [64][LDK]
    static constexpr size_t lam_off = qs_off + 1ull * CH * LDK * 2;            // float [2][64*MAX_L]
    static constexpr size_t g_off = lam_off + 2ull * CH * MAX_L * 4;
    static constexpr size_t gc_off = g_off + 2ull * CH * 4;
    static constexpr size_t y_off = gc_off + CH * 4;                           // float [8][MLOW+1]
    static constexpr size_t total = y_off + 8 * (MLOW + 1) * 4 + 16;
};

template <int KD, int VD, int MLOW>
__global__ void __launch_bounds__(256, 1) m2_bwd_revorder_kernel(const Mamba2Params p) {
    using SM = Bwd2Smem<KD, VD, MLOW>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, LDP = SM::LDP;
    constexpr int SEG = 1 << MLOW, MT = KD / 64, NPS = VD / 32, NPK = KD / 32;
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sK = reinterpret_cast<bf16*>(smem + SM::k_off);
    bf16* sV = reinterpret_cast<bf16*>(smem + SM::v_off);
    bf16* sDO = reinterpret_cast<bf16*>(smem + SM::do_off);
    bf16* sP = reinterpret_cast<bf16*>(smem + SM::p_off);
    bf16* sVs = reinterpret_cast<bf16*>(smem + SM::vs_off);
    bf16* sDKV = reinterpret_cast<bf16*>(smem + SM::dkv_off);
    bf16* sQs = reinterpret_cast<bf16*>(smem + SM::qs_off);
    float* sLam = reinterpret_cast<float*>(smem + SM::lam_off);
    float* sG = reinterpret_cast<float*>(smem + SM::g_off);
    float* sGc = reinterpret_cast<float*>(smem + SM::gc_off);
    float* sY = reinterpret_cast<float*>(smem + SM::y_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % p.NS;
    const int b = blockIdx.x / (p.H * p.NS);
    const int grp = h / (p.H / p.G);
    const int L = p.L;
    const int nc = min(SEG, p.NT - r * SEG);
    const int wr = warp & 3, wc = warp >> 2;
    const int row0 = wr * 16;
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;

    auto issue_tiles = [&](int cl, int st) {
        const long t0 = (long)(r * SEG + cl) * CH;
        load_tile_async<CH, KD, 256>(sQ + st * CH * LDK, p.q + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, tid);
        load_tile_async<CH, KD, 256>(sK + st * CH * LDK, p.k + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, tid);
        load_tile_async<CH, VD, 256>(sV + st * CH * LDV, p.v + (((long)b * p.T + t0) * p.H + h) * VD, (long)p.H * VD, tid);
        load_tile_async<CH, VD, 256>(sDO + st * CH * LDV, p.d_o + (((long)b * p.T + t0) * p.H + h) * VD, (long)p.H * VD, tid);
        cp_async_commit();
    };
    float lam_reg[(CH * MAX_L) / 256];
    float g_reg = 0.f;
    auto fetch_small = [&](int cl) {
        const long t0 = (long)(r * SEG + cl) * CH;
#pragma unroll
        for (int i = 0; i < (CH * MAX_L) / 256; ++i) {
            int e = tid + i * 256;
            int row = e / L, col = e % L;
            lam_reg[i] = (row < CH) ? __bfloat162float(p.l[(((long)b * p.T + t0 + row) * p.H + h) * L + col]) : 0.f;
        }
        if (tid < CH) g_reg = p.g[((long)b * p.T + t0 + tid) * p.H + h];
    };
    auto store_small = [&](int st) {
#pragma unroll
        for (int i = 0; i < (CH * MAX_L) / 256; ++i) {
            int e = tid + i * 256;
            if (e < CH * L) sLam[st * CH * MAX_L + e] = lam_reg[i];
        }
        if (tid < CH) sG[st * CH + tid] = g_reg;
    };

    // adjoint low level states and the adjoint of this segment's summary (index MLOW)
    float RM[MLOW + 1][MT][2 * NPS][4];
#pragma unroll
    for (int lv = 0; lv <= MLOW; ++lv) zero_acc(RM[lv]);
    if (p.NS > 1 && r < p.NS - 1) {
        const float* dH = p.seg_dHf + (((long)b * p.H + h) * p.NS + r) * KD * VD;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int rr = wr * 16 * MT + mt * 16 + lr + hh * 8;
                    const int cc = wc * (VD / 2) + nt * 8 + lc2;
                    float2 x = *reinterpret_cast<const float2*>(dH + rr * VD + cc);
                    RM[MLOW][mt][nt][hh * 2] = x.x;
                    RM[MLOW][mt][nt][hh * 2 + 1] = x.y;
                }
    }

    issue_tiles(nc - 1, 0);
    fetch_small(nc - 1);
    store_small(0);

    for (int it = 0; it < nc; ++it) {
        const int cl = nc - 1 - it;
        const int st = it & 1;
        const long t0 = (long)(r * SEG + cl) * CH;
        if (it + 1 < nc) {
            issue_tiles(cl - 1, st ^ 1);
            fetch_small(cl - 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp == 0) {
            float x0 = sG[st * CH + 2 * lane], x1 = sG[st * CH + 2 * lane + 1];
            warp_cumsum64(x0, x1, lane);
            sGc[2 * lane] = x0;
            sGc[2 * lane + 1] = x1;
        }
        __syncthreads();
        const bf16* cQ = sQ + st * CH * LDK;
        const bf16* cK = sK + st * CH * LDK;
        const bf16* cV = sV + st * CH * LDV;
        const bf16* cDO = sDO + st * CH * LDV;
        const float* cLam = sLam + st * CH * MAX_L;
        const float glast = sGc[CH - 1];

        // ---- P = (q k^T) * decay * lambda -> sP
        {
            float acc[1][4][4];
            zero_acc(acc);
            warp_gemm<1, 2, false, false>(acc, cQ, LDK, row0, cK, LDK, wc * 32, KD, lane);
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
                        float val = 0.f;
                        if (jj <= i) val = acc[0][nt][hh * 2 + e] * fexp(gi - sGc[jj]) * cLam[i * L + level_of(i, jj)];
                        pv[e] = val;
                    }
                    *reinterpret_cast<uint32_t*>(sP + i * LDP + j) = pack_bf16(pv[0], pv[1]);
                }
        }
        for (int e = tid; e < CH * VD / 2; e += 256) {
            const int j = e / (VD / 2), c = (e % (VD / 2)) * 2;
            const float sc = fexp(glast - sGc[j]);
            __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(cV + j * LDV + c);
            *reinterpret_cast<uint32_t*>(sVs + j * LDV + c) =
                pack_bf16(__bfloat162float(vv.x) * sc, __bfloat162float(vv.y) * sc);
        }
        // ---- dKV_c = adjoint of the chunk summary: segment adjoint + levels whose bit is clear
        {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        float x0 = RM[MLOW][mt][nt][hh * 2], x1 = RM[MLOW][mt][nt][hh * 2 + 1];
#pragma unroll
                        for (int lv = 0; lv < MLOW; ++lv)
                            if (!((cl >> lv) & 1)) {
                                x0 += RM[lv][mt][nt][hh * 2];
                                x1 += RM[lv][mt][nt][hh * 2 + 1];
                            }
                        const int rr = wr * 16 * MT + mt * 16 + lr + hh * 8;
                        const int cc = wc * (VD / 2) + nt * 8 + lc2;
                        *reinterpret_cast<uint32_t*>(sDKV + rr * LDV + cc) = pack_bf16(x0, x1);
                    }
        }
        __syncthreads();

        // ---- Y[c][lv] = <KV_c, adjoint state lv> for the levels this chunk contributes to
        {
            float kv[MT][2 * NPS][4];
            zero_acc(kv);
            warp_gemm<MT, NPS, true, true>(kv, cK, LDK, wr * 16 * MT, sVs, LDV, wc * (VD / 2), CH, lane);
#pragma unroll
            for (int lv = 0; lv <= MLOW; ++lv) {
                float y = 0.f;
                if (lv == MLOW || !((cl >> lv) & 1)) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) y += kv[mt][nt][e] * RM[lv][mt][nt][e];
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) y += __shfl_xor_sync(0xffffffffu, y, d);
                if (lane == 0) sY[warp * (MLOW + 1) + lv] = y;
            }
        }

        // ---- dv = P^T do + decay_j * (k . dKV)
        {
            float acc[1][2 * NPS][4], tmp[1][2 * NPS][4];
            zero_acc(acc);
            zero_acc(tmp);
            const int col0 = wc * (VD / 2);
            warp_gemm<1, NPS, true, true>(acc, sP, LDP, row0, cDO, LDV, col0, CH, lane);
            warp_gemm<1, NPS, false, true>(tmp, cK, LDK, row0, sDKV, LDV, col0, KD, lane);
            bf16* gdv = p.dv + (((long)b * p.T + t0) * p.H + h) * VD;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int j = row0 + lr + hh * 8;
                const float sc = fexp(glast - sGc[j]);
#pragma unroll
                for (int nt = 0; nt < 2 * NPS; ++nt)
                    *reinterpret_cast<uint32_t*>(gdv + (long)j * p.H * VD + col0 + nt * 8 + lc2) =
                        pack_bf16(acc[0][nt][hh * 2] + sc * tmp[0][nt][hh * 2], acc[0][nt][hh * 2 + 1] + sc * tmp[0][nt][hh * 2 + 1]);
            }
        }
        // ---- dk (levels) = Vs . dKV^T
        {
            float acc[1][2 * NPK][4];
            zero_acc(acc);
            const int colk = wc * (KD / 2);
            warp_gemm<1, NPK, false, false>(acc, sVs, LDV, row0, sDKV, LDV, colk, VD, lane);
            float rd[2];
            rowdot_tile<2 * NPK>(rd, acc, cK, LDK, row0, colk, lane);
            if ((lane & 3) == 0) {
                float* wp = p.wq + ((long)b * p.T + t0) * p.H + h;
                red_add_f32(wp + (long)(row0 + lr) * p.H, -rd[0]);
                red_add_f32(wp + (long)(row0 + lr + 8) * p.H, -rd[1]);
            }
            red_tile<2 * NPK>(p.dk_acc + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, row0, colk, acc, lane);
        }
        // ---- move the adjoint states back across chunk cl: decay, reset, reader insertions
        {
            const float dec = fexp(glast);
#pragma unroll
            for (int lv = 0; lv <= MLOW; ++lv) {
                const bool reset = (lv < MLOW) && ((cl & ((2 << lv) - 1)) == 0);
                const float f = reset ? 0.f : dec;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) RM[lv][mt][nt][e] *= f;
            }
        }
#pragma unroll
        for (int lv = 0; lv < MLOW; ++lv) {
            if ((cl >> lv) & 1) {
                __syncthreads();     // previous users of sQs are done
                for (int e = tid; e < CH * KD / 2; e += 256) {
                    const int i = e / (KD / 2), c = (e % (KD / 2)) * 2;
                    const float rs = cLam[i * L + INTRA_LEVELS + lv] * fexp(sGc[i]);
                    __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(cQ + i * LDK + c);
                    *reinterpret_cast<uint32_t*>(sQs + i * LDK + c) = pack_bf16(__bfloat162float(x.x) * rs, __bfloat162float(x.y) * rs);
                }
                __syncthreads();
                warp_gemm<MT, NPS, true, true>(RM[lv], sQs, LDK, wr * 16 * MT, cDO, LDV, wc * (VD / 2), CH, lane);
            }
        }
        if (it + 1 < nc) store_small(st ^ 1);
        __syncthreads();
        if (tid <= MLOW) {
            float y = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) y += sY[w * (MLOW + 1) + tid];
            p.Yc[(((long)b * p.H + h) * p.NT + r * SEG + cl) * (MLOW + 1) + tid] = y;
        }
    }
}

// ------------------------------------------------------------------------------------------
// high levels, reader side: dq and dlambda of chunk c in segment r > 0
//   R = do . H0[r][j]^T ; dlambda[t, 7+MLOW+j] = s_i (R_i . q_i) ; dq_i += lambda s_i R_i,
//   s_i = exp(G_i + D_before_c)
// ------------------------------------------------------------------------------------------
template <int KD, int VD>
struct HiBwdSmem {
    static constexpr int LDK = KD + PAD, LDV = VD + PAD;
    static constexpr size_t q_off = 0;
    static constexpr size_t do_off = q_off + 1ull * CH * LDK * 2;
    static constexpr size_t h_off = do_off + 1ull * CH * LDV * 2;
    static constexpr size_t gc_off = h_off + 2ull * KD * LDV * 2;
    static constexpr size_t red_off = gc_off + CH * 4;
    static constexpr size_t dl_off = red_off + 16 * 4;             // float [2][64]
    static constexpr size_t total = dl_off + 2 * CH * 4;
};

template <int KD, int VD, int MLOW>
__global__ void __launch_bounds__(256, 1) m2_hi_bwd_q_kernel(const Mamba2Params p) {
    using SM = HiBwdSmem<KD, VD>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, SEG = 1 << MLOW, NPK = KD / 32;
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sDO = reinterpret_cast<bf16*>(smem + SM::do_off);
    bf16* sH = reinterpret_cast<bf16*>(smem + SM::h_off);
    float* sGc = reinterpret_cast<float*>(smem + SM::gc_off);
    float* sRed = reinterpret_cast<float*>(smem + SM::red_off);
    float* sDL = reinterpret_cast<float*>(smem + SM::dl_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int c = SEG + (blockIdx.x / p.H) % (p.NT - SEG);
    const int b = blockIdx.x / (p.H * (p.NT - SEG));
    const int r = c / SEG, cl = c % SEG;
    const int grp = h / (p.H / p.G);
    const long t0 = (long)c * CH;
    const int wr = warp & 3, wc = warp >> 2;
    const int row0 = wr * 16, colk = wc * (KD / 2);
    const int lr = lane >> 2;
    const long KV = (long)KD * VD;
    const bf16* H0 = p.seg_H0 + (((long)b * p.H + h) * p.NS + r) * p.LH * KV;

    auto issue_state = [&](int j, int slot) {
        load_tile_async<KD, VD, 256>(sH + slot * KD * LDV, H0 + (long)j * KV, VD, tid);
        cp_async_commit();
    };
    load_tile_async<CH, KD, 256>(sQ, p.q + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, tid);
    load_tile_async<CH, VD, 256>(sDO, p.d_o + (((long)b * p.T + t0) * p.H + h) * VD, (long)p.H * VD, tid);
    cp_async_commit();
    int j = __ffs(r) - 1;
    issue_state(j, 0);

    float part = 0.f;
    {
        const float* gp = p.g + ((long)b * p.T + (long)r * SEG * CH) * p.H + h;
        for (int i = tid; i < cl * CH; i += 256) part += gp[(long)i * p.H];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
        if (lane == 0) sRed[warp] = part;
    }
    if (warp == 0) {
        const float* gp = p.g + ((long)b * p.T + t0) * p.H + h;
        float x0 = gp[(long)(2 * lane) * p.H], x1 = gp[(long)(2 * lane + 1) * p.H];
        warp_cumsum64(x0, x1, lane);
        sGc[2 * lane] = x0;
        sGc[2 * lane + 1] = x1;
    }
    __syncthreads();
    float dbefore = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) dbefore += sRed[w];

    float acc[1][2 * NPK][4];
    zero_acc(acc);
    int rem = r & (r - 1);
    int slot = 0;
    while (true) {
        const int jn = rem ? (__ffs(rem) - 1) : -1;
        if (jn >= 0) {
            issue_state(jn, slot ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        float tmp[1][2 * NPK][4];
        zero_acc(tmp);
        warp_gemm<1, NPK, false, false>(tmp, sDO, LDV, row0, sH + slot * KD * LDV, LDV, colk, VD, lane);
        float rd[2];
        rowdot_tile<2 * NPK>(rd, tmp, sQ, LDK, row0, colk, lane);
        const int lcol = INTRA_LEVELS + MLOW + j;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int i = row0 + lr + hh * 8;
            const float sc = fexp(sGc[i] + dbefore);
            const float lam = __bfloat162float(p.l[(((long)b * p.T + t0 + i) * p.H + h) * p.L + lcol]);
            if ((lane & 3) == 0) sDL[wc * CH + i] = sc * rd[hh];
            const float rs = lam * sc;
#pragma unroll
            for (int nt = 0; nt < 2 * NPK; ++nt) {
                acc[0][nt][hh * 2] += rs * tmp[0][nt][hh * 2];
                acc[0][nt][hh * 2 + 1] += rs * tmp[0][nt][hh * 2 + 1];
            }
        }
        __syncthreads();
        if (tid < CH) p.dl[(((long)b * p.T + t0 + tid) * p.H + h) * p.L + lcol] = sDL[tid] + sDL[CH + tid];
        if (warp == 2) {
            float z = 0.f;
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int i = lane + rr * 32;
                z += __bfloat162float(p.l[(((long)b * p.T + t0 + i) * p.H + h) * p.L + lcol]) * (sDL[i] + sDL[CH + i]);
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) z += __shfl_xor_sync(0xffffffffu, z, d);
            if (lane == 0) p.Zc[(((long)b * p.H + h) * p.NT + c) * p.LZ + MLOW + j] = z;
        }
        if (jn < 0) break;
        j = jn;
        rem &= rem - 1;
        slot ^= 1;
    }
    float rd[2];
    rowdot_tile<2 * NPK>(rd, acc, sQ, LDK, row0, colk, lane);
    if ((lane & 3) == 0) {
        float* wp = p.wq + ((long)b * p.T + t0) * p.H + h;
        red_add_f32(wp + (long)(row0 + lr) * p.H, rd[0]);
        red_add_f32(wp + (long)(row0 + lr + 8) * p.H, rd[1]);
    }
    red_tile<2 * NPK>(p.dq_acc + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, row0, colk, acc, lane);
}

// ------------------------------------------------------------------------------------------
// high levels, reader summaries: for segment r >= 1 and high level j with bit j of r set
//   dF[r][j] = sum_{chunks c of r} (q_c * lambda[:, 7+MLOW+j] * exp(G + D_before_c))^T do_c
// (the adjoint of H0[r][j]; fp32 K x V)
// ------------------------------------------------------------------------------------------
template <int KD, int VD, int MLOW>
struct SegDSmem {
    static constexpr int LDK = KD + PAD, LDV = VD + PAD, SEG = 1 << MLOW;
    static constexpr size_t q_off = 0;
    static constexpr size_t do_off = q_off + 2ull * CH * LDK * 2;
    static constexpr size_t qs_off = do_off + 2ull * CH * LDV * 2;
    static constexpr size_t g_off = qs_off + 1ull * CH * LDK * 2;      // float [SEG*64]
    static constexpr size_t tot_off = g_off + (size_t)SEG * CH * 4;
    static constexpr size_t total = tot_off + SEG * 4 + 16;
};

template <int KD, int VD, int MLOW>
__global__ void __launch_bounds__(256, 1) m2_seg_dstate_kernel(const Mamba2Params p) {
    using SM = SegDSmem<KD, VD, MLOW>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, SEG = SM::SEG, MT = KD / 64, NPS = VD / 32;
    const int j = blockIdx.y;
    const int h = blockIdx.x % p.H;
    const int r = 1 + (blockIdx.x / p.H) % (p.NS - 1);
    const int b = blockIdx.x / (p.H * (p.NS - 1));
    if (!((r >> j) & 1)) return;
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sDO = reinterpret_cast<bf16*>(smem + SM::do_off);
    bf16* sQs = reinterpret_cast<bf16*>(smem + SM::qs_off);
    float* sGs = reinterpret_cast<float*>(smem + SM::g_off);
    float* sTot = reinterpret_cast<float*>(smem + SM::tot_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = h / (p.H / p.G);
    const int nc = min(SEG, p.NT - r * SEG);
    const int wr = warp & 3, wc = warp >> 2;
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
    const int lcol = INTRA_LEVELS + MLOW + j;

    auto issue_tiles = [&](int cl, int st) {
        const long t0 = (long)(r * SEG + cl) * CH;
        load_tile_async<CH, KD, 256>(sQ + st * CH * LDK, p.q + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, tid);
        load_tile_async<CH, VD, 256>(sDO + st * CH * LDV, p.d_o + (((long)b * p.T + t0) * p.H + h) * VD, (long)p.H * VD, tid);
        cp_async_commit();
    };
    issue_tiles(0, 0);
    for (int c = warp; c < nc; c += 8) {
        const float* gp = p.g + ((long)b * p.T + (long)(r * SEG + c) * CH) * p.H + h;
        float x0 = gp[(long)(2 * lane) * p.H], x1 = gp[(long)(2 * lane + 1) * p.H];
        warp_cumsum64(x0, x1, lane);
        sGs[c * CH + 2 * lane] = x0;
        sGs[c * CH + 2 * lane + 1] = x1;
        if (lane == 31) sTot[c] = x1;
    }
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int c = 0; c < nc; ++c) {
            float t = sTot[c];
            sTot[c] = run;
            run += t;
        }
    }
    __syncthreads();

    float acc[MT][2 * NPS][4];
    zero_acc(acc);
    for (int cl = 0; cl < nc; ++cl) {
        const int st = cl & 1;
        const long t0 = (long)(r * SEG + cl) * CH;
        if (cl + 1 < nc) {
            issue_tiles(cl + 1, st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* cQ = sQ + st * CH * LDK;
        const float off = sTot[cl];
        for (int e = tid; e < CH * KD / 2; e += 256) {
            const int i = e / (KD / 2), c = (e % (KD / 2)) * 2;
            const float lam = __bfloat162float(p.l[(((long)b * p.T + t0 + i) * p.H + h) * p.L + lcol]);
            const float rs = lam * fexp(off + sGs[cl * CH + i]);
            __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(cQ + i * LDK + c);
            *reinterpret_cast<uint32_t*>(sQs + i * LDK + c) = pack_bf16(__bfloat162float(x.x) * rs, __bfloat162float(x.y) * rs);
        }
        __syncthreads();
        warp_gemm<MT, NPS, true, true>(acc, sQs, LDK, wr * 16 * MT, sDO + st * CH * LDV, LDV, wc * (VD / 2), CH, lane);
        __syncthreads();
    }
    float* dF = p.seg_dF + ((((long)b * p.H + h) * p.NS + r) * p.LH + j) * KD * VD;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int rr = wr * 16 * MT + mt * 16 + lr + hh * 8;
                const int cc = wc * (VD / 2) + nt * 8 + lc2;
                *reinterpret_cast<float2*>(dF + rr * VD + cc) = make_float2(acc[mt][nt][hh * 2], acc[mt][nt][hh * 2 + 1]);
            }
}

// ------------------------------------------------------------------------------------------
// reverse per-level scan over segments (elementwise in K x V): adjoint of m2_seg_scan_kernel.
//   for r = NS-1 .. 0 : dHseg[r] = sum_{j: bit j of r clear} dH_j ; then dH_j is zeroed when
//   r % 2^(j+1) == 0, else decayed by exp(D_r) ; then dF[r][j] is added when bit j of r is set.
// ------------------------------------------------------------------------------------------
constexpr int MAX_LH_B = 10;

template <int MAXLH>
__global__ void __launch_bounds__(256) m2_seg_dscan_kernel(const Mamba2Params p, int KV) {
    const long bh = blockIdx.y;
    const int e4 = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (e4 >= KV) return;
    const float* dF = p.seg_dF + bh * p.NS * p.LH * KV + e4;
    const float* F = p.seg_F + bh * p.NS * KV + e4;
    const float* D = p.seg_D + bh * p.NS;
    float* dH = p.seg_dHf + bh * p.NS * KV + e4;
    float* Yseg = p.Yseg + bh * p.NS * p.LH;
    const int lane = threadIdx.x & 31;
    float st[MAXLH][4];
#pragma unroll
    for (int j = 0; j < MAXLH; ++j) st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f;
    // the recurrence itself is only in registers; the loads of segment r - 2 are issued right after the arithmetic of segment r
    // (two register sets used alternately), so that a thread has up to two segments' worth of loads in flight
    struct Loads {
        float4 f;
        float4 dF[MAXLH];
        float d;
    };
    auto fetch = [&](Loads& L, int r) {
        L.f = (r >= 0 && r < p.NS - 1) ? __ldg(reinterpret_cast<const float4*>(F + (long)r * KV)) : make_float4(0.f, 0.f, 0.f, 0.f);
        L.d = (r >= 0 && r < p.NS - 1) ? __ldg(D + r) : 0.f;
#pragma unroll
        for (int j = 0; j < MAXLH; ++j)
            L.dF[j] = (r >= 0 && j < p.LH && ((r >> j) & 1)) ? __ldg(reinterpret_cast<const float4*>(dF + ((long)r * p.LH + j) * KV))
                                                             : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto process = [&](const Loads& L, int r) {
        float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 f = L.f;
        const float d = (r < p.NS - 1) ? __expf(L.d) : 0.f;
#pragma unroll
        for (int j = 0; j < MAXLH; ++j) {
            if (j < p.LH) {
                const bool bit = (r >> j) & 1;
                if (!bit) {
                    out.x += st[j][0]; out.y += st[j][1]; out.z += st[j][2]; out.w += st[j][3];
                    if (r < p.NS - 1) {
                        // <F_r, adjoint of level j after segment r>
                        float y = f.x * st[j][0] + f.y * st[j][1] + f.z * st[j][2] + f.w * st[j][3];
#pragma unroll
                        for (int dd = 16; dd > 0; dd >>= 1) y += __shfl_xor_sync(0xffffffffu, y, dd);
                        if (lane == 0) atomicAdd(Yseg + (long)r * p.LH + j, y);
                    }
                }
                const int period = 2 << j;
                if ((r % period) == 0) {
                    st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f;
                } else {
                    st[j][0] *= d; st[j][1] *= d; st[j][2] *= d; st[j][3] *= d;
                }
                if (bit) {
                    st[j][0] += L.dF[j].x; st[j][1] += L.dF[j].y; st[j][2] += L.dF[j].z; st[j][3] += L.dF[j].w;
                }
            }
        }
        if (r < p.NS - 1) *reinterpret_cast<float4*>(dH + (long)r * KV) = out;
    };
    Loads A, B;
    fetch(A, p.NS - 1);
    fetch(B, p.NS - 2);
    for (int r = p.NS - 1; r >= 0; r -= 2) {
        process(A, r);
        fetch(A, r - 2);
        if (r - 1 >= 0) {
            process(B, r - 1);
            fetch(B, r - 3);
        }
    }
}

// ------------------------------------------------------------------------------------------
// small elementwise kernels
// ------------------------------------------------------------------------------------------
// raw g from its in-chunk inclusive cumulative sum (what the forward returns and autograd saves)
__global__ void m2_uncumsum_kernel(const float* __restrict__ gc, float* __restrict__ g, long BT, int H) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= BT * H) return;
    const long t = idx / H;
    float x = gc[idx];
    if ((t % CH) != 0) x -= gc[idx - H];
    g[idx] = x;
}

// dg for one (batch, head) per CTA.
//   dg[r] = sum_{t >= r, t in chunk(r)} w[t]  +  X[chunk(r)]
// w[t] = q_t.dq_t - k_t.dk_t is the gradient w.r.t. the in-chunk cumulative sum G_t (the
// reference's dg before its reverse in-chunk cumsum, chunkwise.py:793-874, 1596); X[c] is the
// gradient that reaches the end of chunk c from every (target, source) pair that straddles it
// (the reference's dg_last: sum_j dk_j.k_j + exp(g_last) sum h*dh, chunkwise.py:865-874).  For
// level l and the block pair that contains c, X gets: the running sum of the contributor totals
// Y over the block's contributor chunks up to c (bit l of c clear), or the sum of the reader
// totals Z over the reader chunks after c (bit set).  Sums never extend beyond one block pair, so
// rounding differences between the two sides do not accumulate along the sequence.
template <int MLOW>
__global__ void __launch_bounds__(256) m2_dg_kernel(const Mamba2Params p, float* __restrict__ dg) {
    extern __shared__ float sx[];
    constexpr int SEG = 1 << MLOW;
    float* X = sx;                 // [NT]  (combined-high prefix inside a segment)
    float* XS = sx + p.NT;         // [NS]  (sum over high levels of the prefix over earlier segments)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H, b = blockIdx.x / p.H;
    const long bh = (long)b * p.H + h;
    // blockIdx.y selects a slice of 64 chunks for the token pass; every CTA of a (batch, head)
    // rebuilds the small per-chunk table X (a few thousand scalar operations)
    const int c_begin = blockIdx.y * 64, c_end = min(p.NT, c_begin + 64);
    const float* Zc = p.Zc + bh * p.NT * p.LZ;
    const float* Yc = p.Yc + bh * p.NT * (MLOW + 1);
    const float* Yseg = p.Yseg + bh * p.NS * p.LH;
    // stage the per-chunk scalar tables in shared memory: the sweeps below are serial chains
    float* sZ = sx + p.NT + p.NS;                       // [NT][LZ]
    float* sY = sZ + p.NT * p.LZ;                       // [NT][MLOW+1]
    float* sYs = sY + p.NT * (MLOW + 1);                // [NS][LH]
    for (int i = tid; i < p.NT + p.NS; i += 256) sx[i] = 0.f;
    // eight loads per thread are in flight before the first of them is stored
    for (int i0 = 0; i0 < p.NT * p.LZ; i0 += 8 * 256) {
        float tmp[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * 256 + tid, c = i / p.LZ, lvz = i - c * p.LZ;
            tmp[u] = (i < p.NT * p.LZ && ((c >> lvz) & 1)) ? __ldg(Zc + i) : 0.f;          // only reader entries were written
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * 256 + tid;
            if (i < p.NT * p.LZ) sZ[i] = tmp[u];
        }
    }
    for (int i0 = 0; i0 < p.NT * (MLOW + 1); i0 += 4 * 256) {
        float tmp[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 256 + tid;
            tmp[u] = (i < p.NT * (MLOW + 1)) ? __ldg(Yc + i) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 256 + tid;
            if (i < p.NT * (MLOW + 1)) sY[i] = tmp[u];
        }
    }
    for (int i = tid; i < p.NS * p.LH; i += 256) sYs[i] = __ldg(Yseg + i);
    __syncthreads();
    int nlev = 0;
    while ((1 << nlev) < p.NT) ++nlev;          // inter-chunk levels in use
    // every level writes its own row XL[lv][c] (no shared-memory atomics); rows are summed per chunk below
    float* XL = sYs + p.NS * (p.LH > 0 ? p.LH : 1);     // [nlev][NT]
    // One level per warp and round.  Within a block pair of 2^(lv+1) chunks the contributor sweep runs forwards over the first
    // half (inclusive running sum of Y) and the reader sweep backwards over the second half (running sum of Z, exclusive): the
    // half-blocks are independent, so each lane takes one (block, sweep) with the same branch-free loop and the longest chain is
    // 2^lv steps instead of two passes over all chunks.
    for (int lv = warp; lv < nlev; lv += 8) {
        const int hl = 1 << lv, period = 2 << lv;
        float* xl = XL + lv * p.NT;
        for (int c = lane; c < p.NT; c += 32) xl[c] = 0.f;
        __syncwarp();
        const int nblk = (p.NT + period - 1) / period;
        for (int t = lane; t < 2 * nblk; t += 32) {
            const int base = (t >> 1) * period;
            const bool rev = t & 1;
            const bool active = rev || lv < MLOW;
            const float* src = rev ? sZ + lv : sY + lv;
            const int stride = rev ? p.LZ : (MLOW + 1);
            const int c0 = rev ? base + period - 1 : base, dir = rev ? -1 : 1;
            float run = 0.f;
            for (int k = 0; k < hl; ++k) {
                const int c = c0 + dir * k;
                if (active && c < p.NT) {
                    const float v = src[c * stride];
                    xl[c] = rev ? run : run + v;
                    run += v;
                }
            }
        }
        if (lv >= MLOW && lane == 31) {
            // contributor totals of the high levels live per segment
            const int j = lv - MLOW, pj = 2 << j;
            float run = 0.f;
            for (int r = 0; r < p.NS; ++r) {
                if ((r & (pj - 1)) == 0) run = 0.f;
                if (!((r >> j) & 1)) {
                    atomicAdd(&XS[r], run);
                    if (r < p.NS - 1) run += sYs[r * p.LH + j];
                }
            }
        }
    }
    if (warp == (nlev & 7)) {
        // combined high levels: running sum inside each segment, one segment per lane (on the warp with the fewest levels)
        for (int c0 = lane * SEG; c0 < p.NT; c0 += 32 * SEG) {
            float run = 0.f;
            for (int c = c0; c < c0 + SEG && c < p.NT; ++c) {
                run += sY[c * (MLOW + 1) + MLOW];
                X[c] = run;
            }
        }
    }
    __syncthreads();
    // a warp's (up to eight) chunks: all loads first
    float w0[8], w1[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int c = c_begin + warp + u * 8;
        const long base = ((long)b * p.T + (long)c * CH) * p.H + h;
        w0[u] = (c < c_end) ? __ldg(p.wq + base + (long)(63 - 2 * lane) * p.H) : 0.f;
        w1[u] = (c < c_end) ? __ldg(p.wq + base + (long)(62 - 2 * lane) * p.H) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int c = c_begin + warp + u * 8;
        if (c >= c_end) break;
        const long base = ((long)b * p.T + (long)c * CH) * p.H + h;
        float x0 = w0[u], x1 = w1[u];
        warp_cumsum64(x0, x1, lane);
        float add = X[c] + XS[c / SEG];
        for (int lv = 0; lv < nlev; ++lv) add += XL[lv * p.NT + c];
        dg[base + (long)(63 - 2 * lane) * p.H] = x0 + add;
        dg[base + (long)(62 - 2 * lane) * p.H] = x1 + add;
    }
}

__global__ void m2_cast_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long n) {
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        float4 x = *reinterpret_cast<const float4*>(src + i);
        uint2 o;
        o.x = pack_bf16(x.x, x.y);
        o.y = pack_bf16(x.z, x.w);
        *reinterpret_cast<uint2*>(dst + i) = o;
    } else {
        for (long k = i; k < n; ++k) dst[k] = __float2bfloat16(src[k]);
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
template <typename KernT>
static cudaError_t set_smem(KernT kern, size_t bytes) {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <int KD, int VD, int MLOW>
static int launch_bwd(Mamba2Params p, cudaStream_t stream) {
    cudaError_t e;
    constexpr int SEG = 1 << MLOW;
    const int KV = KD * VD;
    if (p.NS > 1) {
        // forward high-level states: recomputed unless the caller kept the forward call's workspace
        int rc = p.reuse_states ? 0 : mamba2_fwd_states_dispatch(p, stream);
        if (rc != 0) return rc;
        const bool hi_tc = (KD == 128 && VD == 64 && (p.NT % 2) == 0 && p.L <= 20 && p.LH <= 10 && g_use_tensor_core_path.load());
        if (hi_tc) {
            rc = mamba2_hi_bwd_tc_launch(p, stream);
            if (rc != 0) return rc;
        } else {
            {
                auto kern = m2_hi_bwd_q_kernel<KD, VD, MLOW>;
                if ((e = set_smem(kern, HiBwdSmem<KD, VD>::total)) != cudaSuccess) return (int)e;
                kern<<<p.B * p.H * (p.NT - SEG), 256, HiBwdSmem<KD, VD>::total, stream>>>(p); LLATTN_LAUNCHED();
            }
            {
                auto kern = m2_seg_dstate_kernel<KD, VD, MLOW>;
                if ((e = set_smem(kern, SegDSmem<KD, VD, MLOW>::total)) != cudaSuccess) return (int)e;
                dim3 grid(p.B * p.H * (p.NS - 1), p.LH);
                kern<<<grid, 256, SegDSmem<KD, VD, MLOW>::total, stream>>>(p); LLATTN_LAUNCHED();
            }
        }
        {
            dim3 grid((KV / 4 + 255) / 256, p.B * p.H);
            if (p.LH <= 5) { m2_seg_dscan_kernel<5><<<grid, 256, 0, stream>>>(p, KV); LLATTN_LAUNCHED(); }
            else { m2_seg_dscan_kernel<MAX_LH_B><<<grid, 256, 0, stream>>>(p, KV); LLATTN_LAUNCHED(); }
        }
    }
    const bool use_tc = (KD == 128 && VD == 64 && (p.NT % 2) == 0 && p.L <= 20 && g_use_tensor_core_path.load());
    if (use_tc) {
        int rc = mamba2_bwd1_tc_launch(p, stream);
        if (rc != 0) return rc;
    } else {
        auto kern = m2_bwd_fwdorder_kernel<KD, VD, MLOW>;
        if ((e = set_smem(kern, Bwd1Smem<KD, VD, MLOW>::total)) != cudaSuccess) return (int)e;
        kern<<<p.B * p.H * p.NS, 256, Bwd1Smem<KD, VD, MLOW>::total, stream>>>(p); LLATTN_LAUNCHED();
    }
    if (use_tc) {
        int rc = mamba2_bwd2_tc_launch(p, stream);
        if (rc != 0) return rc;
    } else {
        auto kern = m2_bwd_revorder_kernel<KD, VD, MLOW>;
        if ((e = set_smem(kern, Bwd2Smem<KD, VD, MLOW>::total)) != cudaSuccess) return (int)e;
        kern<<<p.B * p.H * p.NS, 256, Bwd2Smem<KD, VD, MLOW>::total, stream>>>(p); LLATTN_LAUNCHED();
    }
    return (int)cudaGetLastError();
}

int mamba2_bwd_dispatch(Mamba2Params p, cudaStream_t stream) {
    if (p.K == 128 && p.V == 64) return launch_bwd<128, 64, M2_MLOW>(p, stream);
    if (p.K == 64 && p.V == 64) return launch_bwd<64, 64, M2_MLOW>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

void mamba2_uncumsum(const float* gc, float* g, long BT, int H, cudaStream_t stream) {
    const long n = BT * H;
    m2_uncumsum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(gc, g, BT, H); LLATTN_LAUNCHED();
}

int mamba2_dg(const Mamba2Params& p, float* dg, cudaStream_t stream) {
    dim3 grid(p.B * p.H, (p.NT + 63) / 64);
    const size_t smem = (size_t)(p.NT + p.NS + p.NT * p.LZ + p.NT * (M2_MLOW + 1) + p.NS * (p.LH > 0 ? p.LH : 1) + (size_t)p.LZ * p.NT) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(m2_dg_kernel<M2_MLOW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    m2_dg_kernel<M2_MLOW><<<grid, 256, smem, stream>>>(p, dg); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

void cast_f32_to_bf16(const float* src, void* dst, long n, cudaStream_t stream) {
    const long thr = (n + 3) / 4;
    m2_cast_bf16_kernel<<<(unsigned)((thr + 255) / 256), 256, 0, stream>>>(src, reinterpret_cast<bf16*>(dst), n); LLATTN_LAUNCHED();
}

}  // namespace llattn
