// Log-linear Mamba-2 (scalar decay) chunkwise forward for sm_100a.
//
// Function computed (reference: hattention/chunkwise.py:1118-1275 driver, kernels :110-280 and
// :488-647; definition hattention/base.py:75-98, 334-349):
//   o[t] = sum_{s<=t} lambda[t, bit_length(t^s)] * exp(sum_{r=s+1..t} g[r]) * (q[t].k[s]) * v[s]
//
// Organisation (instead of one scan launch plus one output launch per level, with a full
// (B,NT,H,K,V) state tensor round-tripping HBM per level):
//   * m2_chunk_fwd_kernel : one CTA per (batch, head, segment of 2^MLOW chunks).  Walks the
//     chunks of its segment in order; per chunk computes the masked intra-chunk product, the
//     chunk summary KV_c = k^T (v * decay), and keeps the MLOW low Fenwick level states on chip:
//     fp32 masters in registers (merged upward on carry, exactly a binary-indexed tree over
//     chunks) and a bf16 copy in shared memory that later chunks read as an MMA operand.
//   * levels whose period exceeds a segment ("high" levels) only need one summary per segment:
//     m2_seg_state_kernel  : F_r = sum_j k_j^T v_j exp(G_segend - G_j)            (fp32, K x V)
//     m2_seg_scan_kernel   : per-level scan over segments -> H0[r, level] in bf16 for readers
//     m2_hi_out_kernel     : o_c = sum_{high levels set in r} lambda * exp(G) * (q_c . H0)
//     and the chunk kernel adds that partial output to its own before the single final store.
#include "llattn_common.cuh"
#include "llattn_mamba2.h"

namespace llattn {

// ------------------------------------------------------------------------------------------
// chunk kernel
// ------------------------------------------------------------------------------------------
template <int KD, int VD, int MLOW>
struct FwdSmem {
    static constexpr int LDK = KD + PAD;
    static constexpr int LDV = VD + PAD;
    static constexpr int LDP = CH + PAD;
    static constexpr size_t q_off = 0;
    static constexpr size_t k_off = q_off + 2ull * CH * LDK * 2;
    static constexpr size_t v_off = k_off + 2ull * CH * LDK * 2;
    static constexpr size_t p_off = v_off + 2ull * CH * LDV * 2;
    static constexpr size_t vs_off = p_off + 1ull * CH * LDP * 2;
    static constexpr size_t h_off = vs_off + 1ull * CH * LDV * 2;
    static constexpr size_t lam_off = h_off + (size_t)MLOW * KD * LDV * 2;      // float [2][64][MAX_L]
    static constexpr size_t g_off = lam_off + 2ull * CH * MAX_L * 4;           // float [2][64]
    static constexpr size_t gc_off = g_off + 2ull * CH * 4;                     // float [64]
    static constexpr size_t total = gc_off + CH * 4;
};

template <int KD, int VD, int MLOW>
__global__ void __launch_bounds__(256, 1) m2_chunk_fwd_kernel(const Mamba2Params p) {
    using SM = FwdSmem<KD, VD, MLOW>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, LDP = SM::LDP;
    constexpr int SEG = 1 << MLOW;
    constexpr int MT = KD / 64;        // state rows per warp = 16*MT (4 warp rows)
    constexpr int NPS = VD / 32;       // state / output column pairs per warp (2 warp cols)
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sK = reinterpret_cast<bf16*>(smem + SM::k_off);
    bf16* sV = reinterpret_cast<bf16*>(smem + SM::v_off);
    bf16* sP = reinterpret_cast<bf16*>(smem + SM::p_off);
    bf16* sVs = reinterpret_cast<bf16*>(smem + SM::vs_off);
    bf16* sH = reinterpret_cast<bf16*>(smem + SM::h_off);
    float* sLam = reinterpret_cast<float*>(smem + SM::lam_off);
    float* sG = reinterpret_cast<float*>(smem + SM::g_off);
    float* sGc = reinterpret_cast<float*>(smem + SM::gc_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % p.NS;
    const int b = blockIdx.x / (p.H * p.NS);
    const int grp = h / (p.H / p.G);
    const int L = p.L;
    const int nc = min(SEG, p.NT - r * SEG);
    const bool hi_init = (p.o_has_high != 0) && (r != 0);

    const int wr = warp & 3, wc = warp >> 2;
    const int row0 = wr * 16;                 // token rows of this warp in 64 x * tiles
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;

    auto issue_tiles = [&](int cl, int st) {
        const long t0 = (long)(r * SEG + cl) * CH;
        const bf16* gq = p.q + (((long)b * p.T + t0) * p.G + grp) * KD;
        const bf16* gk = p.k + (((long)b * p.T + t0) * p.G + grp) * KD;
        const bf16* gv = p.v + (((long)b * p.T + t0) * p.H + h) * VD;
        load_tile_async<CH, KD, 256>(sQ + st * CH * LDK, gq, (long)p.G * KD, tid);
        load_tile_async<CH, KD, 256>(sK + st * CH * LDK, gk, (long)p.G * KD, tid);
        load_tile_async<CH, VD, 256>(sV + st * CH * LDV, gv, (long)p.H * VD, tid);
        cp_async_commit();
    };
    // lambda and g of one chunk go through registers (2-byte / strided elements)
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

    float M[MLOW > 0 ? MLOW : 1][MT][2 * NPS][4];   // fp32 masters of the low level states
    float dsum[MLOW > 0 ? MLOW : 1];                // log decay accumulated since each was formed
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
            float* gc = p.g_cum + ((long)b * p.T + t0) * p.H + h;
            gc[(long)(2 * lane) * p.H] = x0;
            gc[(long)(2 * lane + 1) * p.H] = x1;
        }
        __syncthreads();
        const bf16* cQ = sQ + st * CH * LDK;
        const bf16* cK = sK + st * CH * LDK;
        const bf16* cV = sV + st * CH * LDV;
        const float* cLam = sLam + st * CH * MAX_L;
        const float glast = sGc[CH - 1];

        // ---- S = q k^T, masked / decayed / lambda-weighted -> sP (bf16)
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
        // ---- Vs = v * exp(G_last - G_j)
        for (int e = tid; e < CH * VD / 2; e += 256) {
            const int j = e / (VD / 2), c = (e % (VD / 2)) * 2;
            const float sc = fexp(glast - sGc[j]);
            __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(cV + j * LDV + c);
            *reinterpret_cast<uint32_t*>(sVs + j * LDV + c) =
                pack_bf16(__bfloat162float(vv.x) * sc, __bfloat162float(vv.y) * sc);
        }
        __syncthreads();

        // ---- O = P v + sum over set low bits of rowscale * (q . H_level) (+ high-level partial)
        {
            float acc[1][2 * NPS][4];
            const int col0 = wc * (VD / 2);
            bf16* go = p.o + (((long)b * p.T + t0) * p.H + h) * VD;
            if (hi_init) {
#pragma unroll
                for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = row0 + lr + hh * 8;
                        __nv_bfloat162 ov = *reinterpret_cast<const __nv_bfloat162*>(go + (long)i * p.H * VD + col0 + nt * 8 + lc2);
                        acc[0][nt][hh * 2] = __bfloat162float(ov.x);
                        acc[0][nt][hh * 2 + 1] = __bfloat162float(ov.y);
                    }
            } else {
                zero_acc(acc);
            }
            warp_gemm<1, NPS, false, true>(acc, sP, LDP, row0, cV, LDV, col0, CH, lane);
#pragma unroll
            for (int lv = 0; lv < MLOW; ++lv) {
                if ((cl >> lv) & 1) {
                    float tmp[1][2 * NPS][4];
                    zero_acc(tmp);
                    warp_gemm<1, NPS, false, true>(tmp, cQ, LDK, row0, sH + lv * KD * LDV, LDV, col0, KD, lane);
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int i = row0 + lr + hh * 8;
                        const float rs = cLam[i * L + INTRA_LEVELS + lv] * fexp(sGc[i] + dsum[lv]);
#pragma unroll
                        for (int nt = 0; nt < 2 * NPS; ++nt) {
                            acc[0][nt][hh * 2] += rs * tmp[0][nt][hh * 2];
                            acc[0][nt][hh * 2 + 1] += rs * tmp[0][nt][hh * 2 + 1];
                        }
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = row0 + lr + hh * 8;
                    *reinterpret_cast<uint32_t*>(go + (long)i * p.H * VD + col0 + nt * 8 + lc2) =
                        pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
                }
        }

        // ---- KV_c = k^T Vs and the Fenwick carry over the low levels
        if (MLOW > 0 && cl + 1 < nc) {
            const int j = __ffs(~cl) - 1;   // number of trailing one bits of cl
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
    }
}

// ------------------------------------------------------------------------------------------
// segment summary  F_r = sum_{tokens j of segment r} k_j^T v_j exp(G_end - G_j),  D_r = sum g
// ------------------------------------------------------------------------------------------
template <int KD, int VD, int MLOW>
struct SegSmem {
    static constexpr int LDK = KD + PAD;
    static constexpr int LDV = VD + PAD;
    static constexpr int SEG = 1 << MLOW;
    static constexpr size_t k_off = 0;
    static constexpr size_t v_off = k_off + 2ull * CH * LDK * 2;
    static constexpr size_t vs_off = v_off + 2ull * CH * LDV * 2;
    static constexpr size_t g_off = vs_off + 1ull * CH * LDV * 2;        // float [SEG*64] cumulative
    static constexpr size_t tot_off = g_off + (size_t)SEG * CH * 4;      // float [SEG]
    static constexpr size_t total = tot_off + SEG * 4 + 16;
};

template <int KD, int VD, int MLOW>
__global__ void __launch_bounds__(256, 1) m2_seg_state_kernel(const Mamba2Params p) {
    using SM = SegSmem<KD, VD, MLOW>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, SEG = SM::SEG;
    constexpr int MT = KD / 64, NPS = VD / 32;
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sK = reinterpret_cast<bf16*>(smem + SM::k_off);
    bf16* sV = reinterpret_cast<bf16*>(smem + SM::v_off);
    bf16* sVs = reinterpret_cast<bf16*>(smem + SM::vs_off);
    float* sGs = reinterpret_cast<float*>(smem + SM::g_off);
    float* sTot = reinterpret_cast<float*>(smem + SM::tot_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % (p.NS - 1);      // the last segment has no reader
    const int b = blockIdx.x / (p.H * (p.NS - 1));
    const int grp = h / (p.H / p.G);
    const int wr = warp & 3, wc = warp >> 2;
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;

    auto issue_tiles = [&](int cl, int st) {
        const long t0 = (long)(r * SEG + cl) * CH;
        const bf16* gk = p.k + (((long)b * p.T + t0) * p.G + grp) * KD;
        const bf16* gv = p.v + (((long)b * p.T + t0) * p.H + h) * VD;
        load_tile_async<CH, KD, 256>(sK + st * CH * LDK, gk, (long)p.G * KD, tid);
        load_tile_async<CH, VD, 256>(sV + st * CH * LDV, gv, (long)p.H * VD, tid);
        cp_async_commit();
    };
    issue_tiles(0, 0);
    // cumulative log decay from the segment start, inclusive
    for (int c = warp; c < SEG; c += 8) {
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
        for (int c = 0; c < SEG; ++c) {
            float t = sTot[c];
            sTot[c] = run;
            run += t;
        }
        sTot[SEG] = run;
    }
    __syncthreads();
    const float gend = sTot[SEG];

    float acc[MT][2 * NPS][4];
    zero_acc(acc);
    for (int cl = 0; cl < SEG; ++cl) {
        const int st = cl & 1;
        if (cl + 1 < SEG) {
            issue_tiles(cl + 1, st ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* cV = sV + st * CH * LDV;
        const float off = sTot[cl];
        for (int e = tid; e < CH * VD / 2; e += 256) {
            const int j = e / (VD / 2), c = (e % (VD / 2)) * 2;
            const float sc = fexp(gend - (off + sGs[cl * CH + j]));
            __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(cV + j * LDV + c);
            *reinterpret_cast<uint32_t*>(sVs + j * LDV + c) =
                pack_bf16(__bfloat162float(vv.x) * sc, __bfloat162float(vv.y) * sc);
        }
        __syncthreads();
        warp_gemm<MT, NPS, true, true>(acc, sK + st * CH * LDK, LDK, wr * 16 * MT, sVs, LDV, wc * (VD / 2), CH, lane);
        __syncthreads();
    }
    float* F = p.seg_F + (((long)b * p.H + h) * p.NS + r) * KD * VD;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int rr = wr * 16 * MT + mt * 16 + lr + hh * 8;
                const int cc = wc * (VD / 2) + nt * 8 + lc2;
                *reinterpret_cast<float2*>(F + rr * VD + cc) = make_float2(acc[mt][nt][hh * 2], acc[mt][nt][hh * 2 + 1]);
            }
    if (tid == 0) p.seg_D[((long)b * p.H + h) * p.NS + r] = gend;
}

// ------------------------------------------------------------------------------------------
// per-level scan over segments (elementwise in K x V).  For level j and segment r with bit j of
// r set, H0[r][j] is the state before segment r, i.e. the reference's per-level scan
// (chunkwise.py:179-266) run at segment granularity: store; zero after r % 2^(j+1) == 2^(j+1)-1,
// else decay by exp(D_r); add F_r when bit j of r is clear.
// ------------------------------------------------------------------------------------------
constexpr int MAX_LH = 10;

__global__ void __launch_bounds__(256) m2_seg_scan_kernel(const Mamba2Params p, int KV) {
    const long bh = blockIdx.y;
    const int e4 = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (e4 >= KV) return;
    const float* F = p.seg_F + bh * p.NS * KV + e4;
    const float* D = p.seg_D + bh * p.NS;
    bf16* H0 = p.seg_H0 + bh * p.NS * p.LH * KV + e4;
    float st[MAX_LH][4];
#pragma unroll
    for (int j = 0; j < MAX_LH; ++j) st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f;
    // the recurrence is in registers; the summaries of eight segments are requested together so that a thread pays the load
    // latency once per eight segments
    constexpr int RB = 8;
    for (int r0 = 0; r0 < p.NS; r0 += RB) {
      float4 fb[RB];
      float db[RB];
#pragma unroll
      for (int u = 0; u < RB; ++u) {
          const int r = r0 + u;
          fb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          db[u] = 0.f;
          if (r < p.NS - 1) {
              fb[u] = __ldg(reinterpret_cast<const float4*>(F + (long)r * KV));
              db[u] = __ldg(D + r);
          }
      }
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        const int r = r0 + u;
        if (r >= p.NS) break;
        const float4 f = fb[u];
        const float d = (r < p.NS - 1) ? __expf(db[u]) : 0.f;
#pragma unroll
        for (int j = 0; j < MAX_LH; ++j) {
            if (j < p.LH) {
                const bool bit = (r >> j) & 1;
                if (bit) {
                    uint2 pk;
                    pk.x = pack_bf16(st[j][0], st[j][1]);
                    pk.y = pack_bf16(st[j][2], st[j][3]);
                    *reinterpret_cast<uint2*>(H0 + ((long)r * p.LH + j) * KV) = pk;
                }
                const int period = 2 << j;
                if ((r % period) == period - 1) {
                    st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f;
                } else {
                    st[j][0] *= d; st[j][1] *= d; st[j][2] *= d; st[j][3] *= d;
                }
                if (!bit) {
                    st[j][0] += f.x; st[j][1] += f.y; st[j][2] += f.z; st[j][3] += f.w;
                }
            }
        }
      }
    }
}

// ------------------------------------------------------------------------------------------
// high-level output partial: one CTA per chunk of every segment r > 0
//   o_c[i] = sum_{j: bit j of r} lambda[t, 7+MLOW+j] exp(G_i + D_before_c) (q_i . H0[r][j])
// ------------------------------------------------------------------------------------------
template <int KD, int VD>
struct HiSmem {
    static constexpr int LDK = KD + PAD;
    static constexpr int LDV = VD + PAD;
    static constexpr size_t q_off = 0;
    static constexpr size_t h_off = q_off + 1ull * CH * LDK * 2;
    static constexpr size_t gc_off = h_off + 2ull * KD * LDV * 2;
    static constexpr size_t red_off = gc_off + CH * 4;
    static constexpr size_t total = red_off + 16 * 4;
};

template <int KD, int VD, int MLOW>
__global__ void __launch_bounds__(256, 1) m2_hi_out_kernel(const Mamba2Params p) {
    using SM = HiSmem<KD, VD>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, SEG = 1 << MLOW, NPS = VD / 32;
    extern __shared__ __align__(16) unsigned char smem[];
    bf16* sQ = reinterpret_cast<bf16*>(smem + SM::q_off);
    bf16* sH = reinterpret_cast<bf16*>(smem + SM::h_off);
    float* sGc = reinterpret_cast<float*>(smem + SM::gc_off);
    float* sRed = reinterpret_cast<float*>(smem + SM::red_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int c = SEG + (blockIdx.x / p.H) % (p.NT - SEG);     // chunks of segment 0 have no high level
    const int b = blockIdx.x / (p.H * (p.NT - SEG));
    const int r = c / SEG, cl = c % SEG;
    const int grp = h / (p.H / p.G);
    const long t0 = (long)c * CH;
    const int wr = warp & 3, wc = warp >> 2;
    const int row0 = wr * 16, col0 = wc * (VD / 2);
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
    const long KV = (long)KD * VD;
    const bf16* H0 = p.seg_H0 + (((long)b * p.H + h) * p.NS + r) * p.LH * KV;

    auto issue_state = [&](int j, int slot) {
        load_tile_async<KD, VD, 256>(sH + slot * KD * LDV, H0 + (long)j * KV, VD, tid);
        cp_async_commit();
    };
    load_tile_async<CH, KD, 256>(sQ, p.q + (((long)b * p.T + t0) * p.G + grp) * KD, (long)p.G * KD, tid);
    cp_async_commit();
    // first set bit
    int j = __ffs(r) - 1;
    issue_state(j, 0);

    // log decay of the chunks of this segment that precede chunk c
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

    float acc[1][2 * NPS][4];
    zero_acc(acc);
    int rem = r & (r - 1);      // remaining set bits after j
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
        float tmp[1][2 * NPS][4];
        zero_acc(tmp);
        warp_gemm<1, NPS, false, true>(tmp, sQ, LDK, row0, sH + slot * KD * LDV, LDV, col0, KD, lane);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int i = row0 + lr + hh * 8;
            const float lam = __bfloat162float(p.l[(((long)b * p.T + t0 + i) * p.H + h) * p.L + INTRA_LEVELS + MLOW + j]);
            const float rs = lam * fexp(sGc[i] + dbefore);
#pragma unroll
            for (int nt = 0; nt < 2 * NPS; ++nt) {
                acc[0][nt][hh * 2] += rs * tmp[0][nt][hh * 2];
                acc[0][nt][hh * 2 + 1] += rs * tmp[0][nt][hh * 2 + 1];
            }
        }
        __syncthreads();
        if (jn < 0) break;
        j = jn;
        rem &= rem - 1;
        slot ^= 1;
    }
    if (p.o_has_high == 2) {
        // column-chunk-major scratch read by the tcgen05 chunk kernel: [bh][pair][8-col chunk][128 rows][8]
        bf16* gh = p.o_hi + (((long)b * p.H + h) * (p.NT / 2) + (c >> 1)) * (8 * 128 * 8);
#pragma unroll
        for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = (c & 1) * CH + row0 + lr + hh * 8;
                const int cc = col0 + nt * 8;
                *reinterpret_cast<uint32_t*>(gh + ((long)(cc >> 3) * 128 + i) * 8 + lc2) =
                    pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
            }
        return;
    }
    bf16* go = p.o + (((long)b * p.T + t0) * p.H + h) * VD;
#pragma unroll
    for (int nt = 0; nt < 2 * NPS; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int i = row0 + lr + hh * 8;
            *reinterpret_cast<uint32_t*>(go + (long)i * p.H * VD + col0 + nt * 8 + lc2) =
                pack_bf16(acc[0][nt][hh * 2], acc[0][nt][hh * 2 + 1]);
        }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
template <int KD, int VD, int MLOW>
static int launch_states(Mamba2Params p, cudaStream_t stream) {
    cudaError_t e;
    if (KD == 128 && VD == 64 && g_use_tensor_core_path.load()) {
        int rc = mamba2_seg_state_tc_launch(p, stream);
        if (rc != 0) return rc;
    } else {
        auto kern = m2_seg_state_kernel<KD, VD, MLOW>;
        size_t sm = SegSmem<KD, VD, MLOW>::total;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
        kern<<<p.B * p.H * (p.NS - 1), 256, sm, stream>>>(p); LLATTN_LAUNCHED();
    }
    const int KV = KD * VD;
    dim3 grid((KV / 4 + 255) / 256, p.B * p.H);
    m2_seg_scan_kernel<<<grid, 256, 0, stream>>>(p, KV); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

template <int KD, int VD, int MLOW>
static int launch_fwd(Mamba2Params p, cudaStream_t stream) {
    cudaError_t e;
    const bool use_tc = (KD == 128 && VD == 64 && (p.NT % 2) == 0 && p.L <= 20 && g_use_tensor_core_path.load());
    if (p.NS > 1) {
        p.o_has_high = use_tc ? 2 : 1;      // 2: partial output goes to the column-chunk-major scratch
        int rc = launch_states<KD, VD, MLOW>(p, stream);
        if (rc != 0) return rc;
        if (use_tc && p.LH <= 8) {
            rc = mamba2_hi_out_tc_launch(p, stream);
            if (rc != 0) return rc;
        } else {
            auto kern = m2_hi_out_kernel<KD, VD, MLOW>;
            size_t sm = HiSmem<KD, VD>::total;
            if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
            kern<<<p.B * p.H * (p.NT - (1 << MLOW)), 256, sm, stream>>>(p); LLATTN_LAUNCHED();
        }
    }
    if (use_tc) {
        return mamba2_fwd_tc_launch(p, stream);
    }
    {
        auto kern = m2_chunk_fwd_kernel<KD, VD, MLOW>;
        size_t sm = FwdSmem<KD, VD, MLOW>::total;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return (int)e;
        kern<<<p.B * p.H * p.NS, 256, sm, stream>>>(p); LLATTN_LAUNCHED();
    }
    return (int)cudaGetLastError();
}

std::atomic<int> g_use_tensor_core_path{1};

int mamba2_fwd_dispatch(Mamba2Params p, cudaStream_t stream) {
    if (p.K == 128 && p.V == 64) return launch_fwd<128, 64, M2_MLOW>(p, stream);
    if (p.K == 64 && p.V == 64) return launch_fwd<64, 64, M2_MLOW>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

int mamba2_fwd_states_dispatch(Mamba2Params p, cudaStream_t stream) {
    if (p.K == 128 && p.V == 64) return launch_states<128, 64, M2_MLOW>(p, stream);
    if (p.K == 64 && p.V == 64) return launch_states<64, 64, M2_MLOW>(p, stream);
    return LLATTN_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace llattn
