// Segment-level ("high" Fenwick levels) kernels of the log-linear Mamba-2 path on tcgen05 / TMA
// (K = 128, V = 64, segments of 2^MLOW chunks = 2^(MLOW-1) pairs of 128 tokens).  Same mathematics
// as m2_seg_state_kernel / m2_hi_out_kernel (mamba2_fwd.cu) and m2_seg_dstate_kernel /
// m2_hi_bwd_q_kernel (mamba2_bwd.cu); one CTA per (batch, head, segment) handles every high level
// of its segment, so q / do / k / v tiles and the level states are loaded once per segment.
//   seg_state  : F_r      = sum_pairs k^T (v * exp(G_end - G))                      (fp32 K x V)
//   hi_out     : o_hi     = sum_{j set in r} lambda_j exp(G) * (q H0[r][j])         (bf16, column-chunk-major scratch)
//   seg_dstate : dF[r][j] = sum_pairs q^T (do * lambda_j exp(G))                     (fp32 K x V per set level)
//   hi_bwd_q   : dlambda_j = exp(G) (do . (q H0_j)) ; dq += (do * lambda_j exp(G)) H0_j^T   (TMA reduce-add)
// G is the cumulative log decay from the start of the segment (inclusive).
#include "tc_common.cuh"

namespace llattn {

namespace tcs {
constexpr int MAXLH = 5;            // high levels handled by these kernels (T <= 64 * 2^(MLOW+5))
}

__device__ __forceinline__ uint32_t box_offset_f32(int row, int col) {
    return (uint32_t)(row * 128 + (((col >> 2) ^ (row & 7)) << 4) + (col & 3) * 4);
}

// cumulative log decay of a whole segment (SEG chunks) from its start, inclusive, into sGs[SEG*64];
// all 256 compute threads call it; returns after a bar_compute
template <int SEG>
__device__ __forceinline__ void segment_cumsum(const Mamba2Params& p, int b, int h, int r, int nchunks, float* sGs, float* sTot,
                                               int warp, int lane, int tid) {
    for (int c = warp; c < nchunks; c += 8) {
        const float* gp = p.g + ((long)b * p.T + (long)(r * SEG + c) * CH) * p.H + h;
        float x0 = gp[(long)(2 * lane) * p.H], x1 = gp[(long)(2 * lane + 1) * p.H];
        warp_cumsum64(x0, x1, lane);
        sGs[c * CH + 2 * lane] = x0;
        sGs[c * CH + 2 * lane + 1] = x1;
        if (lane == 31) sTot[c] = x1;
    }
    bar_compute();
    if (tid == 0) {
        float run = 0.f;
        for (int c = 0; c < nchunks; ++c) {
            const float t = sTot[c];
            sTot[c] = run;
            run += t;
        }
        sTot[SEG] = run;
    }
    bar_compute();
    for (int i = tid; i < nchunks * CH; i += 256) sGs[i] += sTot[i / CH];
    bar_compute();
}

// ------------------------------------------------------------------------------------------
// backward: reader summaries dF[r][j] and, in the same pass over the segment, dq / dlambda of the
// high levels.  Per pair: T_j = q H0_j (one 64-column slot, level after level), dlambda_j and
// the scaled copy do * (lambda_j exp(G)); then dq (+)= that copy times H0_j^T and dF_j += q^T times it.
// ------------------------------------------------------------------------------------------
template <int MLOW>
struct HiBwdTcSmem {
    static constexpr int SEG = 1 << MLOW;
    static constexpr uint32_t q_off = 0;                                   // 32 KB
    static constexpr uint32_t do_off = q_off + tc::Q_BYTES;                // 16 KB
    static constexpr uint32_t h_off = do_off + tc::V_BYTES;                // MAXLH x 16 KB states
    static constexpr uint32_t dos_off = h_off + tcs::MAXLH * tc::H_BYTES;  // MAXLH x 16 KB scaled do ; first 64 KB double as fp32 staging
    static constexpr uint32_t gs_off = dos_off + tcs::MAXLH * tc::V_BYTES; // float [SEG*64] + [SEG+1]
    static constexpr uint32_t misc_off = gs_off + (SEG * 64 + SEG + 32) * 4;  // float [2][128][MAXLH+1] dlambda halves
    static constexpr uint32_t bar_off = misc_off + 2 * 128 * (tcs::MAXLH + 1) * 4;
    static constexpr uint32_t sink_off = bar_off + 128;                    // uint32 [256], written only (tile release)
    static constexpr uint32_t total = sink_off + 256 * 4 + 1024;
};

template <int MLOW>
__global__ void __launch_bounds__(tc::NTHREADS, 1) m2_hi_bwd_tc_kernel(const __grid_constant__ Mamba2Params p) {
    using SM = HiBwdTcSmem<MLOW>;
    constexpr int SEG = SM::SEG, NDLH = tcs::MAXLH + 1;
    // tensor memory: dF slots 0..4 (64 columns each), dq (128 columns), T (64 columns).  The level reads
    // T_j use three adjacent 64-column slots: the two halves of dq (only written after every T of the pair
    // has been consumed) and T.
    constexpr int TM_DF = 0, TM_DQ = 320;      // the third T slot is the 64 columns after dq (448..511)
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = smem + SM::q_off;
    unsigned char* sDO = smem + SM::do_off;
    unsigned char* sH = smem + SM::h_off;
    unsigned char* sDOs = smem + SM::dos_off;
    unsigned char* sStage = smem + SM::dos_off;
    float* sGs = reinterpret_cast<float*>(smem + SM::gs_off);
    float* sTot = sGs + SEG * 64;
    float* sDL = reinterpret_cast<float*>(smem + SM::misc_off);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* barT = bars + 0;       // [2] first / second chain of level reads complete ([2] unused)
    uint64_t* barB = bars + 3;       // second batch of a pair complete
    uint64_t* full_q = bars + 4;     // q tile of a pair
    uint64_t* full_do = bars + 5;    // do tile of a pair
    uint64_t* full_h = bars + 6;     // the level states of the segment
    uint64_t* empty_q = bars + 7;    // second batch done: q may be overwritten
    uint64_t* empty_do = bars + 8;   // every compute thread holds its do row in registers (256 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 104);
    uint32_t* sink = reinterpret_cast<uint32_t*>(smem + SM::sink_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef LLATTN_STAMPS
    // one CTA's life: entry, before / after the segment's cumulative decay, top of each pair, end of the pairs, reader summaries
    // written, reduce-adds complete, exit (thread 0)
    int nstamp = 0;
    const int stamp_slot = (blockIdx.x == 700 && tid == 0) ? 0 : -1;
#endif
    STAMP();
    const int h = blockIdx.x % p.H;
    const int r = 1 + (blockIdx.x / p.H) % (p.NS - 1);
    const int b = blockIdx.x / (p.H * (p.NS - 1));
    const int grp = h / (p.H / p.G);
    const int nchunks = min(SEG, p.NT - r * SEG);
    const int npairs = nchunks / 2;
    // set high levels of this segment inside this launch's window of five levels, in increasing order
    int lev[tcs::MAXLH], nl = 0;
#pragma unroll
    for (int jj = 0; jj < tcs::MAXLH; ++jj) {
        const int j = p.lev_lo + jj;
        if (j < p.LH && ((r >> j) & 1)) lev[nl++] = j;
    }
    if (nl == 0) return;             // nothing to read in this window (uniform for the CTA)

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) umma::mbar_init(&bars[i], 1);
        umma::mbar_init(empty_do, 256);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    constexpr uint32_t ID_KK128 = umma::idesc_bf16(128, 128, false, false);
    constexpr uint32_t ID_MM64 = umma::idesc_bf16(128, 64, true, true);
    auto t_slot = [&](int i) -> uint32_t { return (uint32_t)(TM_DQ + (i % 3) * 64); };   // three adjacent 64-column slots

    if (warp >= tc::MMA_WARP) {
        RegisterSplit<120, 192>::release();
        if (warp == tc::MMA_WARP + 1) {
            if (lane == 0) {
                // level states of the segment: rows of the (B*H*NS*LH*K, V) matrix
                tma::expect_tx(full_h, nl * tc::H_BYTES);
                for (int i = 0; i < nl; ++i) {
                    const int row0 = ((((b * p.H + h) * p.NS + r) * p.LH) + lev[i]) * tc::KD;
                    tma::load_panel(sH + i * tc::H_BYTES, &p.tm_h0, 0, 0, row0, full_h);
                }
                const int brow = b * p.T + r * SEG * CH;
                for (int pl = 0; pl < npairs; ++pl) {
                    const int row0 = brow + pl * tc::PT;
                    if (pl >= 1 && !umma::mbar_wait(empty_do, (pl - 1) & 1, abort_flag)) break;
                    tma::expect_tx(full_do, tc::V_BYTES);
                    tma::load_panel(sDO, &p.tm_do, 0, h, row0, full_do);
                    if (pl >= 1 && !umma::mbar_wait(empty_q, (pl - 1) & 1, abort_flag)) break;
                    tma::expect_tx(full_q, tc::Q_BYTES);
                    tma::load_panel(sQ, &p.tm_q, 0, grp, row0, full_q);
                    tma::load_panel(sQ + tc::Q_BYTES / 2, &p.tm_q, 64, grp, row0, full_q);
                }
            }
            return;
        }
        if (warp > tc::MMA_WARP) return;
        umma::tmem_alloc(tmem_slot, tc::TM_COLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        const uint32_t aQ = umma::smem_addr(sQ), aH = umma::smem_addr(sH), aDOs = umma::smem_addr(sDOs);
        if (lane == 0) umma::mbar_wait(full_h, 0, abort_flag);
        for (int pl = 0; pl < npairs; ++pl) {
            if (lane == 0) umma::mbar_wait(full_q, pl & 1, abort_flag);
            __syncwarp();
            umma::fence_after_sync();
            // The issue of a tcgen05.mma costs about as much for N = 64 as for N = 256, so the level reads of up
            // to three levels are ONE chain of eight instructions: the level states are adjacent 64-column
            // panels of an MN-major B operand and their results adjacent tensor-memory slots.
            {
                const int n0 = nl < 3 ? nl : 3;
                if (lane == 0) {
                    umma::gemm_km<tc::PT, tc::KD, tc::KD>(tbase + TM_DQ, aQ, aH, umma::idesc_bf16(128, 64 * n0, false, true), false);
                    umma::commit(&barT[0]);
                }
                __syncwarp();
                if (nl > 3) {
                    bar_work();                      // the three slots have been read by the compute warps
                    umma::fence_after_sync();
                    if (lane == 0) {
                        umma::gemm_km<tc::PT, tc::KD, tc::KD>(tbase + TM_DQ, aQ, aH + 3 * tc::H_BYTES,
                                                              umma::idesc_bf16(128, 64 * (nl - 3), false, true), false);
                        umma::commit(&barT[1]);
                    }
                    __syncwarp();
                }
            }
            umma::fence_before_sync();
            bar_work();                              // scaled copies of do are written, every T consumed
            umma::fence_after_sync();
            if (lane == 0) {
                // reader summaries of up to four levels per chain (N = 256), then dq over all levels
                const int n0 = nl < 4 ? nl : 4;
                umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase + TM_DF, aQ, aDOs, umma::idesc_bf16(128, 64 * n0, true, true), pl > 0);
                if (nl > 4)
                    umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase + TM_DF + 4 * 64, aQ, aDOs + 4 * tc::V_BYTES, ID_MM64, pl > 0);
                for (int i = 0; i < nl; ++i)
                    umma::gemm_kk<tc::PT, tc::KD, tc::VD>(tbase + TM_DQ, aDOs + i * tc::V_BYTES, aH + i * tc::H_BYTES, ID_KK128, i > 0);
                umma::commit(barB);
                // q is free as soon as the batch is done: let the producer refill it while dq is read out
                umma::mbar_wait(barB, pl & 1, abort_flag);
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(empty_q)) : "memory");
            }
            __syncwarp();
            umma::fence_before_sync();
            bar_work();                              // end of the pair: dq has left tensor memory
            umma::fence_after_sync();
            if (*abort_flag) break;
        }
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();
        umma::tmem_dealloc(tbase, tc::TM_COLS);
        return;
    }

    // ================= warps 0..7 =================
    RegisterSplit<120, 192>::acquire();
    const int rb = warp & 3;
    const int row = rb * 32 + lane;
    const int ch = warp >> 2;
    STAMP();
    segment_cumsum<SEG>(p, b, h, r, nchunks, sGs, sTot, warp, lane, tid);
    STAMP();
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;
    uint32_t phT[2] = {0, 0};

    // this row's lambda of the levels read: requested one pair ahead, so that the loads' latency is not part of a pair
    bf16 lam_next[tcs::MAXLH];
    auto fetch_lambda = [&](int pl) {
        const long t0 = (long)(r * SEG) * CH + (long)pl * tc::PT;
        const bf16* lrow = p.l + (((long)b * p.T + t0 + row) * p.H + h) * p.L + INTRA_LEVELS + MLOW;
#pragma unroll
        for (int i = 0; i < tcs::MAXLH; ++i)
            if (i < nl) lam_next[i] = lrow[lev[i]];
    };
    fetch_lambda(0);

    for (int pl = 0; pl < npairs; ++pl) {
        STAMP();
        const long t0 = (long)(r * SEG) * CH + (long)pl * tc::PT;
        const float sc = fexp(sGs[pl * tc::PT + row]);          // exp(G_i) from the segment start
        float lamv[tcs::MAXLH];
#pragma unroll
        for (int i = 0; i < tcs::MAXLH; ++i) lamv[i] = (i < nl) ? __bfloat162float(lam_next[i]) : 0.f;
        if (pl + 1 < npairs) fetch_lambda(pl + 1);
        umma::mbar_wait(full_do, pl & 1, abort_flag);
        uint4 dox[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) dox[c] = *reinterpret_cast<const uint4*>(sDO + umma::tile_offset(row, ch * 32 + c * 8, tc::PT));
        {
            // every thread holds its do row in registers: hand the tile back to the producer (the release must
            // follow the loads, see release_tile_after_loads)
            const uint32_t x = dox[0].x ^ dox[0].y ^ dox[0].z ^ dox[0].w ^ dox[1].x ^ dox[1].y ^ dox[1].z ^ dox[1].w ^
                               dox[2].x ^ dox[2].y ^ dox[2].z ^ dox[2].w ^ dox[3].x ^ dox[3].y ^ dox[3].z ^ dox[3].w;
            release_tile_after_loads(empty_do, sink + tid, x);
        }
        float* myDL = sDL + (ch * 128 + row) * NDLH;
        for (int i = 0; i < nl; ++i) {
            if (i == 0 || i == 3) {                  // one completion per chain of level reads
                umma::mbar_wait(&barT[i / 3], phT[i / 3], abort_flag);
                phT[i / 3] ^= 1;
                umma::fence_after_sync();
            }
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + t_slot(i), warp, ch * 32), t);
            if (i == 2 && nl > 3) {
                umma::fence_before_sync();
                bar_work();                          // the three slots may be reused
            }
            if (i < 4) {
                // The staging area of the previous pair's dq tile is the memory of the first four scaled copies: box i of
                // the reduce-add (its own bulk group) must have been read before copy i is written.  Waiting box by box
                // lets the first copy start after a quarter of the read.
                if (tid == 0) {
                    if (i == 0) tma::wait_group_read<3>();
                    else if (i == 1) tma::wait_group_read<2>();
                    else if (i == 2) tma::wait_group_read<1>();
                    else tma::wait_group_read<0>();
                }
                bar_compute();
            }
            const float rs = lamv[i] * sc;
            float dot = 0.f;
            unsigned char* dst = sDOs + i * tc::V_BYTES;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(&dox[c]);
                uint32_t outw[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[e]);
                    const float a0 = __bfloat162float(v2.x), a1 = __bfloat162float(v2.y);
                    dot += a0 * t[c * 8 + e * 2] + a1 * t[c * 8 + e * 2 + 1];
                    outw[e] = pack_bf16(a0 * rs, a1 * rs);
                }
                *reinterpret_cast<uint4*>(dst + umma::tile_offset(row, ch * 32 + c * 8, tc::PT)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
            }
            myDL[i] = sc * dot;
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();                                  // scaled copies written; second batch may start
        umma::fence_after_sync();
        // ---- dlambda out, reader totals Z per chunk, q.dq contribution
        {
            // the two warps of a lane quarter take alternate levels
            float* gdl = p.dl + (((long)b * p.T + t0 + row) * p.H + h) * p.L + INTRA_LEVELS + MLOW;
            float wsum = 0.f;
            for (int i = ch; i < nl; i += 2) {
                const float dlv = sDL[row * NDLH + i] + sDL[(128 + row) * NDLH + i];
                gdl[lev[i]] = dlv;
                float z = lamv[i] * dlv;
                wsum += z;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) z += __shfl_xor_sync(0xffffffffu, z, d);
                if (lane == 0) sTot[SEG + 1 + rb * tcs::MAXLH + i] = z;        // per 32-row block
            }
            if (ch < nl) red_add_f32(p.wq + ((long)b * p.T + t0 + row) * p.H + h, wsum);
        }
        umma::mbar_wait(barB, pl & 1, abort_flag);
        umma::fence_after_sync();
        if (nl < 4) {
            // boxes nl..3 of the previous pair's reduce-add were not waited for above
            if (tid == 0) tma::wait_group_read<0>();
            bar_compute();
        }
        // ---- dq tile -> fp32 staging (the scaled copies are no longer needed) -> TMA reduce-add
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + TM_DQ, warp, ch * 64 + hb * 32), t);
            unsigned char* box = sStage + (ch * 2 + hb) * 16384;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<float4*>(box + box_offset_f32(row, c * 4)) = make_float4(t[c * 4], t[c * 4 + 1], t[c * 4 + 2], t[c * 4 + 3]);
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_compute();
        if (tid == 0) {
            const int grow = b * p.T + (int)t0;
#pragma unroll
            for (int bx = 0; bx < 4; ++bx) {
                tma::reduce_add_box(&p.tm_dq, bx * 32, grp, grow, sStage + bx * 16384);
                tma::commit_group();                 // one group per box: the next pair waits for them one by one
            }
        }
        if (tid < 2 * nl) {
            const int i = tid >> 1, cpart = tid & 1;
            const float z = sTot[SEG + 1 + (cpart * 2) * tcs::MAXLH + i] + sTot[SEG + 1 + (cpart * 2 + 1) * tcs::MAXLH + i];
            const long cidx = ((long)b * p.H + h) * p.NT + r * SEG + pl * 2 + cpart;
            p.Zc[cidx * p.LZ + MLOW + lev[i]] = z;
        }
        umma::fence_before_sync();
        bar_work();                                  // end of the pair
        umma::fence_after_sync();
        if (*abort_flag) break;
    }
    STAMP();
    // ---- dF[r][j] out
    for (int i = 0; i < nl; ++i) {
        float t[32];
        umma::tmem_ld32(umma::tmem_addr(tbase + TM_DF + i * 64, warp, ch * 32), t);
        float* dF = p.seg_dF + ((((long)b * p.H + h) * p.NS + r) * p.LH + lev[i]) * tc::KD * tc::VD + row * tc::VD + ch * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) w[e] = __float_as_uint(t[c * 8 + e]);
            st_global_32B(dF + c * 8, w);            // a thread owns its row: 32-byte stores fill whole sectors
        }
    }
    STAMP();
    if (tid == 0) tma::wait_group0();
    STAMP();
    umma::fence_before_sync();
    bar_work();
    STAMP();
}

// ------------------------------------------------------------------------------------------
// forward: partial output of the high levels, o_hi = sum_j lambda_j exp(G) (q H0[r][j])
// ------------------------------------------------------------------------------------------
template <int MLOW, int MAXL>
struct HiOutTcSmem {
    static constexpr int SEG = 1 << MLOW;
    static constexpr uint32_t q_off = 0;                                   // [2] 32 KB
    static constexpr uint32_t h_off = q_off + 2 * tc::Q_BYTES;
    static constexpr uint32_t gs_off = h_off + MAXL * tc::H_BYTES;
    static constexpr uint32_t bar_off = gs_off + (SEG * 64 + SEG + 32) * 4;
    static constexpr uint32_t total = bar_off + 128 + 1024;
};

template <int MLOW, int MAXL>
__global__ void __launch_bounds__(tc::NTHREADS, 1) m2_hi_out_tc_kernel(const __grid_constant__ Mamba2Params p) {
    using SM = HiOutTcSmem<MLOW, MAXL>;
    static_assert(MAXL * 64 <= tc::TM_COLS, "one 64-column tensor-memory slot per level");
    constexpr int SEG = SM::SEG;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = smem + SM::q_off;
    unsigned char* sH = smem + SM::h_off;
    float* sGs = reinterpret_cast<float*>(smem + SM::gs_off);
    float* sTot = sGs + SEG * 64;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* barA = bars + 0;       // level reads of a pair complete
    uint64_t* full_q = bars + 1;     // [2]
    uint64_t* full_h = bars + 3;
    uint64_t* empty_q = bars + 4;    // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 64);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 72);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = 1 + (blockIdx.x / p.H) % (p.NS - 1);
    const int b = blockIdx.x / (p.H * (p.NS - 1));
    const int grp = h / (p.H / p.G);
    const int nchunks = min(SEG, p.NT - r * SEG);
    const int npairs = nchunks / 2;
    int lev[MAXL], nl = 0;
#pragma unroll
    for (int j = 0; j < MAXL; ++j)
        if (j < p.LH && ((r >> j) & 1)) lev[nl++] = j;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 6; ++i) umma::mbar_init(&bars[i], 1);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    if (warp >= tc::MMA_WARP) {
        RegisterSplit<56, 224>::release();
        if (warp == tc::MMA_WARP + 1) {
            if (lane == 0) {
                tma::expect_tx(full_h, nl * tc::H_BYTES);
                for (int i = 0; i < nl; ++i) {
                    const int row0 = ((((b * p.H + h) * p.NS + r) * p.LH) + lev[i]) * tc::KD;
                    tma::load_panel(sH + i * tc::H_BYTES, &p.tm_h0, 0, 0, row0, full_h);
                }
                const int brow = b * p.T + r * SEG * CH;
                for (int pl = 0; pl < npairs; ++pl) {
                    const int st = pl & 1, row0 = brow + pl * tc::PT;
                    if (pl >= 2 && !umma::mbar_wait(&empty_q[st], ((pl - 2) >> 1) & 1, abort_flag)) break;
                    tma::expect_tx(&full_q[st], tc::Q_BYTES);
                    tma::load_panel(sQ + st * tc::Q_BYTES, &p.tm_q, 0, grp, row0, &full_q[st]);
                    tma::load_panel(sQ + st * tc::Q_BYTES + tc::Q_BYTES / 2, &p.tm_q, 64, grp, row0, &full_q[st]);
                }
            }
            return;
        }
        if (warp > tc::MMA_WARP) return;
        umma::tmem_alloc(tmem_slot, tc::TM_COLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        if (lane == 0) umma::mbar_wait(full_h, 0, abort_flag);
        for (int pl = 0; pl < npairs; ++pl) {
            const int st = pl & 1;
            bar_work();                              // the slots of the previous pair have been read
            umma::fence_after_sync();
            if (lane == 0) {
                umma::mbar_wait(&full_q[st], (pl >> 1) & 1, abort_flag);
                // adjacent level states / adjacent result slots: chains of up to four levels (N = 256)
                for (int i0 = 0; i0 < nl; i0 += 4) {
                    const int n = (nl - i0) < 4 ? (nl - i0) : 4;
                    umma::gemm_km<tc::PT, tc::KD, tc::KD>(tbase + i0 * 64, umma::smem_addr(sQ + st * tc::Q_BYTES),
                                                          umma::smem_addr(sH + i0 * tc::H_BYTES),
                                                          umma::idesc_bf16(128, 64 * n, false, true), false);
                }
                umma::commit(barA);
                umma::commit(&empty_q[st]);
            }
            __syncwarp();
            if (*abort_flag) break;
        }
        umma::fence_before_sync();
        bar_work();
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::tmem_dealloc(tbase, tc::TM_COLS);
        return;
    }

    RegisterSplit<56, 224>::acquire();
    const int rb = warp & 3;
    const int row = rb * 32 + lane;
    const int ch = warp >> 2;
    segment_cumsum<SEG>(p, b, h, r, nchunks, sGs, sTot, warp, lane, tid);
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;

    for (int pl = 0; pl < npairs; ++pl) {
        const long t0 = (long)(r * SEG) * CH + (long)pl * tc::PT;
        const float sc = fexp(sGs[pl * tc::PT + row]);
        const bf16* lrow = p.l + (((long)b * p.T + t0 + row) * p.H + h) * p.L + INTRA_LEVELS + MLOW;
        float lamv[MAXL];
#pragma unroll
        for (int i = 0; i < MAXL; ++i) lamv[i] = (i < nl) ? __bfloat162float(lrow[lev[i]]) * sc : 0.f;
        umma::fence_before_sync();
        bar_work();
        umma::mbar_wait(barA, pl & 1, abort_flag);
        umma::fence_after_sync();
        float o[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = 0.f;
        for (int i = 0; i < nl; ++i) {
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + i * 64, warp, ch * 32), t);
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] += lamv[i] * t[e];
        }
        // column-chunk-major scratch [bh][pair][8-col chunk][128 rows][8]
        bf16* gh = p.o_hi + ((((long)b * p.H + h) * (p.NT / 2) + (r * (SEG / 2) + pl)) * 8 + ch * 4) * (tc::PT * 8) + row * 8;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(gh + c * tc::PT * 8) =
                make_uint4(pack_bf16(o[c * 8], o[c * 8 + 1]), pack_bf16(o[c * 8 + 2], o[c * 8 + 3]),
                           pack_bf16(o[c * 8 + 4], o[c * 8 + 5]), pack_bf16(o[c * 8 + 6], o[c * 8 + 7]));
        if (*abort_flag) break;
    }
    umma::fence_before_sync();
    bar_work();
}

// ------------------------------------------------------------------------------------------
// forward: segment summaries F_r = sum_j k_j^T v_j exp(G_end - G_j), D_r = G_end
// ------------------------------------------------------------------------------------------
template <int MLOW>
struct SegStateTcSmem {
    static constexpr int SEG = 1 << MLOW;
    static constexpr uint32_t k_off = 0;                                   // [2] 32 KB
    static constexpr uint32_t v_off = k_off + 2 * tc::Q_BYTES;             // [2] 16 KB
    static constexpr uint32_t vs_off = v_off + 2 * tc::V_BYTES;            // [2] 16 KB
    static constexpr uint32_t gs_off = vs_off + 2 * tc::V_BYTES;
    static constexpr uint32_t bar_off = gs_off + (SEG * 64 + SEG + 32) * 4;
    static constexpr uint32_t total = bar_off + 128 + 1024;
};

template <int MLOW>
__global__ void __launch_bounds__(tc::NTHREADS, 1) m2_seg_state_tc_kernel(const __grid_constant__ Mamba2Params p) {
    using SM = SegStateTcSmem<MLOW>;
    constexpr int SEG = SM::SEG, SEGP = SEG / 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sK = smem + SM::k_off;
    unsigned char* sV = smem + SM::v_off;
    unsigned char* sVs = smem + SM::vs_off;
    float* sGs = reinterpret_cast<float*>(smem + SM::gs_off);
    float* sTot = sGs + SEG * 64;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* barF = bars + 0;
    uint64_t* full_kv = bars + 1;    // [2]
    uint64_t* empty_kv = bars + 3;   // [2] tensor core is done with the k / v / Vs stage
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 64);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 72);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % (p.NS - 1);          // the last segment has no reader
    const int b = blockIdx.x / (p.H * (p.NS - 1));
    const int grp = h / (p.H / p.G);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 5; ++i) umma::mbar_init(&bars[i], 1);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;
    constexpr uint32_t ID_MM64 = umma::idesc_bf16(128, 64, true, true);

    if (warp >= tc::MMA_WARP) {
        RegisterSplit<56, 224>::release();
        if (warp == tc::MMA_WARP + 1) {
            if (lane == 0) {
                const int brow = b * p.T + r * SEG * CH;
                for (int pl = 0; pl < SEGP; ++pl) {
                    const int st = pl & 1, row0 = brow + pl * tc::PT;
                    if (pl >= 2 && !umma::mbar_wait(&empty_kv[st], ((pl - 2) >> 1) & 1, abort_flag)) break;
                    tma::expect_tx(&full_kv[st], tc::Q_BYTES + tc::V_BYTES);
                    tma::load_panel(sK + st * tc::Q_BYTES, &p.tm_k, 0, grp, row0, &full_kv[st]);
                    tma::load_panel(sK + st * tc::Q_BYTES + tc::Q_BYTES / 2, &p.tm_k, 64, grp, row0, &full_kv[st]);
                    tma::load_panel(sV + st * tc::V_BYTES, &p.tm_v, 0, h, row0, &full_kv[st]);
                }
            }
            return;
        }
        if (warp > tc::MMA_WARP) return;
        umma::tmem_alloc(tmem_slot, 64);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        for (int pl = 0; pl < SEGP; ++pl) {
            const int st = pl & 1;
            bar_work();                              // Vs of this pair is written
            umma::fence_after_sync();
            if (lane == 0) {
                umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase, umma::smem_addr(sK + st * tc::Q_BYTES),
                                                      umma::smem_addr(sVs + st * tc::V_BYTES), ID_MM64, pl > 0);
                umma::commit(&empty_kv[st]);
                if (pl == SEGP - 1) umma::commit(barF);
            }
            __syncwarp();
            if (*abort_flag) break;
        }
        umma::fence_before_sync();
        bar_work();
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::tmem_dealloc(tbase, 64);
        return;
    }

    RegisterSplit<56, 224>::acquire();
    const int rb = warp & 3;
    const int row = rb * 32 + lane;
    const int ch = warp >> 2;
    segment_cumsum<SEG>(p, b, h, r, SEG, sGs, sTot, warp, lane, tid);
    const float gend = sTot[SEG];
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;

    for (int pl = 0; pl < SEGP; ++pl) {
        const int st = pl & 1;
        umma::mbar_wait(&full_kv[st], (pl >> 1) & 1, abort_flag);
        if (pl >= 2) umma::mbar_wait(&empty_kv[st], ((pl - 2) >> 1) & 1, abort_flag);     // Vs stage is free
#pragma unroll
        for (int i = tid; i < tc::PT * (tc::VD / 8); i += 256) {
            const int j = i / (tc::VD / 8), c = (i % (tc::VD / 8)) * 8;
            const float sc = fexp(gend - sGs[pl * tc::PT + j]);
            const uint32_t off = umma::tile_offset(j, c, tc::PT);
            uint4 x = *reinterpret_cast<const uint4*>(sV + st * tc::V_BYTES + off);
            uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 v2 = *reinterpret_cast<__nv_bfloat162*>(&xw[e]);
                xw[e] = pack_bf16(__bfloat162float(v2.x) * sc, __bfloat162float(v2.y) * sc);
            }
            *reinterpret_cast<uint4*>(sVs + st * tc::V_BYTES + off) = x;
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        if (*abort_flag) break;
    }
    umma::mbar_wait(barF, 0, abort_flag);
    umma::fence_after_sync();
    {
        float t[32];
        umma::tmem_ld32(umma::tmem_addr(tbase, warp, ch * 32), t);
        float* F = p.seg_F + (((long)b * p.H + h) * p.NS + r) * tc::KD * tc::VD + row * tc::VD + ch * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) w[e] = __float_as_uint(t[c * 8 + e]);
            st_global_32B(F + c * 8, w);
        }
    }
    if (tid == 0) p.seg_D[((long)b * p.H + h) * p.NS + r] = gend;
    umma::fence_before_sync();
    bar_work();
}

int mamba2_seg_state_tc_launch(const Mamba2Params& p_in, cudaStream_t stream) {
    Mamba2Params p = p_in;
    int rc;
    const long BT = (long)p.B * p.T;
    if ((rc = tma::make_panel_map(&p.tm_k, p.k, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_v, p.v, BT, p.H, p.V, tc::PT)) != 0) return rc;
    auto kern = m2_seg_state_tc_kernel<M2_MLOW>;
    const size_t sm = SegStateTcSmem<M2_MLOW>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    kern<<<p.B * p.H * (p.NS - 1), tc::NTHREADS, sm, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

int mamba2_hi_out_tc_launch(const Mamba2Params& p_in, cudaStream_t stream) {
    Mamba2Params p = p_in;
    int rc;
    const long BT = (long)p.B * p.T;
    if ((rc = tma::make_panel_map(&p.tm_q, p.q, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_h0, p.seg_H0, (long)p.B * p.H * p.NS * p.LH * p.K, 1, p.V, tc::KD)) != 0) return rc;
    // up to five segment levels (T <= 16384) with the smaller shared-memory footprint, else up to eight
    if (p.LH <= 5) {
        auto kern = m2_hi_out_tc_kernel<M2_MLOW, 5>;
        const size_t sm = HiOutTcSmem<M2_MLOW, 5>::total;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return (int)e;
        kern<<<p.B * p.H * (p.NS - 1), tc::NTHREADS, sm, stream>>>(p); LLATTN_LAUNCHED();
    } else {
        auto kern = m2_hi_out_tc_kernel<M2_MLOW, 8>;
        const size_t sm = HiOutTcSmem<M2_MLOW, 8>::total;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return (int)e;
        kern<<<p.B * p.H * (p.NS - 1), tc::NTHREADS, sm, stream>>>(p); LLATTN_LAUNCHED();
    }
    return (int)cudaGetLastError();
}

int mamba2_hi_bwd_tc_launch(const Mamba2Params& p_in, cudaStream_t stream) {
    Mamba2Params p = p_in;
    int rc;
    const long BT = (long)p.B * p.T;
    if ((rc = tma::make_panel_map(&p.tm_q, p.q, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_do, p.d_o, BT, p.H, p.V, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_h0, p.seg_H0, (long)p.B * p.H * p.NS * p.LH * p.K, 1, p.V, tc::KD)) != 0) return rc;
    if ((rc = tma::make_f32_box_map(&p.tm_dq, p.dq_acc, BT, p.G, p.K, tc::PT)) != 0) return rc;
    auto kern = m2_hi_bwd_tc_kernel<M2_MLOW>;
    const size_t sm = HiBwdTcSmem<M2_MLOW>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    // one launch per window of five segment levels (a single one up to T = 16384); dq, the q.dq totals and
    // the per-level outputs of different windows add up or are disjoint
    for (p.lev_lo = 0; p.lev_lo < p.LH; p.lev_lo += tcs::MAXLH) {
        kern<<<p.B * p.H * (p.NS - 1), tc::NTHREADS, sm, stream>>>(p);
        LLATTN_LAUNCHED();
    }
    return (int)cudaGetLastError();
}

}  // namespace llattn

#ifdef LLATTN_STAMPS
extern "C" int llattn_debug_read_stamps_seg(long long* host_dst) {
    return (int)cudaMemcpyFromSymbol(host_dst, llattn::g_stamps, sizeof(llattn::g_stamps));
}
#endif
