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
#include "tc_common.cuh"

namespace llattn {

template <int MLOW>
struct FwdTcSmem {
    static constexpr int MP = MLOW - 1;              // pair levels kept on chip
    static constexpr uint32_t q_off = 0;
    static constexpr uint32_t v_off = q_off + tc::Q_BYTES;             // [2]
    static constexpr uint32_t k_off = v_off + 2 * tc::V_BYTES;         // [2]
    static constexpr uint32_t p_off = k_off + 2 * tc::Q_BYTES;
    static constexpr uint32_t vs_off = p_off + tc::PT * tc::PT * 2;
    static constexpr uint32_t h_off = vs_off + tc::V_BYTES;
    static constexpr uint32_t gp_off = h_off + (MP > 0 ? MP : 1) * tc::H_BYTES;   // float [2][3][128]: decay tables of this pair and the next
    static constexpr uint32_t lam_off = gp_off + 2 * 3 * 128 * 4;      // bf16 [128][L <= 32]
    static constexpr uint32_t bar_off = lam_off + 128 * (MAX_L + 2) * 2;   // 10 mbarriers + tmem slot + abort flag     // 4 mbarriers + tmem slot + abort flag
    static constexpr uint32_t total = bar_off + 128 + 1024;             // + slack for 1024-byte alignment
};

template <int MLOW>
__global__ void __launch_bounds__(tc::NTHREADS, 1) m2_chunk_fwd_tc_kernel(const __grid_constant__ Mamba2Params p) {
    using SM = FwdTcSmem<MLOW>;
    constexpr int MP = SM::MP;
    constexpr int SEGP = 1 << MP;                    // pairs per segment
    constexpr int NLAM = 8 + (MP > 0 ? MP : 1);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = smem + SM::q_off;            // single buffer, refilled as soon as S and T are done
    unsigned char* sV = smem + SM::v_off;            // [2]
    unsigned char* sK = smem + SM::k_off;            // [2]
    unsigned char* sP = smem + SM::p_off;
    unsigned char* sVs = smem + SM::vs_off;
    unsigned char* sH = smem + SM::h_off;
    float* sTab = reinterpret_cast<float*>(smem + SM::gp_off);     // [2][3][128]: per pair, G | Cf | Vf (see decay_tables)
    bf16* sLam = reinterpret_cast<bf16*>(smem + SM::lam_off);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);     // MMA completion: S, T, O, KV
    uint64_t* full_q = bars + 4;                     // TMA completion: q tile
    uint64_t* full_kv = bars + 5;                    // [2] k and v tiles of a stage
    uint64_t* empty_q = bars + 7;                    // tensor core is done reading the q tile
    uint64_t* empty_kv = bars + 8;                   // [2] ... the k and v tiles of a stage
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 80);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 88);
    static_assert(MP <= 2, "two tensor-memory slots for level reads");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % p.NS;
    const int b = blockIdx.x / (p.H * p.NS);
    const int grp = h / (p.H / p.G);
    const int L = p.L;
    const int npairs = min(SEGP, p.NT / 2 - r * SEGP);
    const bool hi_init = (p.o_has_high != 0) && (r != 0);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 10; ++i) umma::mbar_init(&bars[i], 1);
        umma::fence_mbar_init();
        *abort_flag = *p.err;                        // an earlier CTA gave up: do not pile on
    }
    __syncthreads();
    if (*abort_flag) return;                         // uniform: every thread reads the same shared word

    constexpr uint32_t ID_S = umma::idesc_bf16(128, 128, false, false);
    constexpr uint32_t ID_KM = umma::idesc_bf16(128, 64, false, true);
    constexpr uint32_t ID_MM = umma::idesc_bf16(128, 64, true, true);

    if (warp >= tc::MMA_WARP) {
        // ================= third warpgroup: one warp issues the tensor-core work =================
        RegisterSplit<56, 224>::release();
        if (warp == tc::MMA_WARP + 1) {
            // ---- TMA producer: one lane streams the tiles of the segment through the stages
            if (lane == 0) {
                const int brow = b * p.T + r * SEGP * tc::PT;
                for (int pl = 0; pl < npairs; ++pl) {
                    const int st = pl & 1, row0 = brow + pl * tc::PT;
                    if (pl >= 2 && !umma::mbar_wait(&empty_kv[st], ((pl - 2) >> 1) & 1, abort_flag)) break;
                    tma::expect_tx(&full_kv[st], tc::Q_BYTES + tc::V_BYTES);
                    tma::load_panel(sK + st * tc::Q_BYTES, &p.tm_k, 0, grp, row0, &full_kv[st]);
                    tma::load_panel(sK + st * tc::Q_BYTES + tc::Q_BYTES / 2, &p.tm_k, 64, grp, row0, &full_kv[st]);
                    tma::load_panel(sV + st * tc::V_BYTES, &p.tm_v, 0, h, row0, &full_kv[st]);
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
        bar_work();                                  // publishes the tensor-memory base address
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        for (int pl = 0; pl < npairs; ++pl) {
            const int st = pl & 1;
            const uint32_t aQ = umma::smem_addr(sQ), aK = umma::smem_addr(sK + st * tc::Q_BYTES);
            const uint32_t aV = umma::smem_addr(sV + st * tc::V_BYTES);
            // (no barrier here: the end-of-pair barrier of the previous pair is all the tensor core needs; the decay
            //  tables of this pair were written one pair ahead)
            if (lane == 0) {
                umma::mbar_wait(full_q, pl & 1, abort_flag);
                umma::mbar_wait(&full_kv[st], (pl >> 1) & 1, abort_flag);
                umma::gemm_kk<tc::PT, tc::PT, tc::KD>(tbase + tc::TM_S, aQ, aK, ID_S, false);
                umma::commit(&bars[0]);
                int slot = 0;
#pragma unroll
                for (int lv = 0; lv < MP; ++lv)
                    if ((pl >> lv) & 1) {
                        umma::gemm_km<tc::PT, tc::KD, tc::KD>(tbase + (slot == 0 ? tc::TM_T0 : tc::TM_T1), aQ,
                                                              umma::smem_addr(sH + lv * tc::H_BYTES), ID_KM, false);
                        ++slot;
                    }
                if (slot > 0) umma::commit(&bars[1]);
                umma::commit(empty_q);               // q tile may be overwritten once S and the level reads are done
            }
            __syncwarp();
            umma::fence_before_sync();
            bar_work();                              // barrier 2: P and Vs are written
            umma::fence_after_sync();
            if (lane == 0) {
                umma::gemm_km<tc::PT, tc::PT, tc::PT>(tbase + tc::TM_O, umma::smem_addr(sP), aV, ID_KM, false);
                umma::commit(&bars[2]);
                umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase + tc::TM_KV, aK, umma::smem_addr(sVs), ID_MM, false);
                umma::commit(&bars[3]);
                umma::commit(&empty_kv[st]);         // k / v stage may be refilled
            }
            __syncwarp();
            umma::fence_before_sync();
            bar_work();                              // barrier 3: end of the pair
            umma::fence_after_sync();
            if (*abort_flag) break;
        }
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();                                  // everybody is done with tensor memory
        umma::tmem_dealloc(tbase, tc::TM_COLS);
        return;
    }

    // ================= warps 0..7: loads, decay / mask / lambda, outputs, level states =================
    RegisterSplit<56, 224>::acquire();
    const int rb = warp & 3;                         // 32-row block of this thread's tensor-memory lane
    const int row = rb * 32 + lane;
    const int ch = warp >> 2;                        // column half handled by this thread

    // lambda rows of the pair (two threads per row, staged through shared memory) and raw g of the
    // pair (warps 0 and 1), fetched one pair ahead
    float g_n[4];
    constexpr int LAMR = (tc::PT * NLAM + 255) / 256;   // only the NLAM columns these kernels read are fetched
    uint32_t lam_r[LAMR];                            // one 32-bit register per 16-bit element
    uint32_t lam_rc[LAMR];                           // (row << 8) | column of each element, 0xffffffff = none
    const int NC = L < NLAM ? L : NLAM;             // columns of a lambda row that are fetched
#pragma unroll
    for (int i = 0; i < LAMR; ++i) {
        const int e = tid + i * 256;
        const int rr = e / NC, cc = e - rr * NC;
        lam_rc[i] = (rr < tc::PT) ? (uint32_t)((rr << 8) | cc) : 0xffffffffu;
    }
    auto fetch_small = [&](int pl) {
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        const unsigned short* lp = reinterpret_cast<const unsigned short*>(p.l) + (((long)b * p.T + t0) * p.H + h) * L;
#pragma unroll
        for (int i = 0; i < LAMR; ++i)
            if (lam_rc[i] != 0xffffffffu) lam_r[i] = lp[(long)(lam_rc[i] >> 8) * p.H * L + (lam_rc[i] & 255)];
    };
    // raw g of a pair: one warp (the one that builds the decay tables), four consecutive tokens per lane
    auto fetch_g = [&](int pl) {
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        const float* gp = p.g + ((long)b * p.T + t0 + 4 * lane) * p.H + h;
#pragma unroll
        for (int i = 0; i < 4; ++i) g_n[i] = gp[(long)i * p.H];
    };
    // Decay tables of pair `pl` from the g values in g_n, by one full warp: G (pair-wide inclusive cumulative sum),
    // Cf = exp(G[end of 32-block] - G[j]), Vf = exp(G[127] - G[j]); also the in-chunk cumulative sum to global memory.
    // Built one pair ahead into the other half of sTab, so that a pair starts without a barrier of its own.
    auto decay_tables = [&](int pl) {
        float* tG = sTab + (pl & 1) * 384;
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        float gq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) gq[i] = g_n[i];
        gq[1] += gq[0];
        gq[2] += gq[1];
        gq[3] += gq[2];
        float tot = gq[3];                           // inclusive scan of lane totals inside each chunk (16 lanes)
#pragma unroll
        for (int d = 1; d < 16; d <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, tot, d);
            if ((lane & 15) >= d) tot += t;
        }
        const float gla = __shfl_sync(0xffffffffu, tot, 15);        // end of the first chunk
        const float glb = __shfl_sync(0xffffffffu, tot, 31);        // end of the second chunk (in-chunk)
        const float glp = gla + glb;
        const float cbase = tot - gq[3];                            // in-chunk exclusive prefix of this lane
        const float pbase = cbase + (lane >= 16 ? gla : 0.f);       // pair-wide
        const float gend = __shfl_sync(0xffffffffu, tot, (lane & ~7) + 7) + (lane >= 16 ? gla : 0.f);
        float* gc = p.g_cum + ((long)b * p.T + t0 + 4 * lane) * p.H + h;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float G = pbase + gq[i];
            tG[4 * lane + i] = G;
            tG[128 + 4 * lane + i] = fexp(gend - G);
            tG[256 + 4 * lane + i] = fexp(glp - G);
            gc[(long)i * p.H] = cbase + gq[i];
        }
    };
    constexpr int TABLE_WARP = 4;                    // lane quarter 0 (one 32 x 32 block of the S tile): the warp with slack
    auto store_lam = [&]() {
#pragma unroll
        for (int i = 0; i < LAMR; ++i)
            if (lam_rc[i] != 0xffffffffu)
                sLam[(lam_rc[i] >> 8) * tc::LAM_LD + (lam_rc[i] & 255)] = __ushort_as_bfloat16((unsigned short)lam_r[i]);
    };
    fetch_small(0);
    store_lam();
    if (warp == TABLE_WARP) {
        fetch_g(0);
        decay_tables(0);
        if (npairs > 1) fetch_g(1);
    }
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;

    float M[MP > 0 ? MP : 1][32];     // masters: row `row` of each low pair-level state, 32 columns
    float dsum[MP > 0 ? MP : 1];
#pragma unroll
    for (int i = 0; i < (MP > 0 ? MP : 1); ++i) dsum[i] = 0.f;
    uint32_t phS = 0, phT = 0, phO = 0, phKV = 0;

    for (int pl = 0; pl < npairs; ++pl) {
#ifdef LLATTN_STAMPS
        int nstamp = 0;
        const int stamp_slot = (blockIdx.x == 300 && pl == 2) ? (tid == 0 ? 0 : (tid == 200 ? 1 : (tid == 96 ? 2 : -1))) : -1;
#endif
        STAMP();                                     // 0: top of the pair
        const int st = pl & 1;
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        const float* sGp = sTab + (pl & 1) * 384;    // tables of this pair (written while the previous pair ran)
        const float* sCf = sGp + 128;
        const float* sVf = sGp + 256;
        if (pl + 1 < npairs) fetch_small(pl + 1);
        // partial output of the high levels for this thread's row / column half (issued early, used late)
        uint4 ohi[4];
        if (hi_init) {
            // scratch layout [batch*head][pair][8-column chunk][128 rows][8]: a warp reads 512 contiguous bytes
            const bf16* gh = p.o_hi + ((((long)b * p.H + h) * (p.NT / 2) + (r * SEGP + pl)) * 8 + ch * 4) * (tc::PT * 8) + row * 8;
#pragma unroll
            for (int c = 0; c < 4; ++c) ohi[c] = *reinterpret_cast<const uint4*>(gh + c * tc::PT * 8);
        }
        STAMP();                                     // 1: small fetches issued
        umma::mbar_wait(&full_kv[st], (pl >> 1) & 1, abort_flag);      // the v tile (read below with generic loads)
        STAMP();                                     // 2: tiles landed
        STAMP();                                     // 3
        int nread = 0;
#pragma unroll
        for (int lv = 0; lv < MP; ++lv) nread += (pl >> lv) & 1;
        const float Gi = sGp[row];
        const float glp = sGp[tc::PT - 1];
        // this row's lambda: levels 0..7 inside the pair, then the low pair levels
        float lam[NLAM];
#pragma unroll
        for (int i = 0; i < NLAM; ++i) lam[i] = (i < L) ? __bfloat162float(sLam[row * tc::LAM_LD + i]) : 0.f;

        // ---- Vs = v * exp(glp - G_j)   (same swizzled offsets as v)
        {
            const unsigned char* cV = sV + st * tc::V_BYTES;
#pragma unroll
            for (int i = tid; i < tc::PT * (tc::VD / 8); i += 256) {
                const int j = i / (tc::VD / 8), c = (i % (tc::VD / 8)) * 8;
                const float sc = sVf[j];
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
        STAMP();                                     // 4: Vs written
        // ---- wait for S (and the level reads); the q tile is then free for the next pair
        umma::mbar_wait(&bars[0], phS, abort_flag);
        phS ^= 1;
        if (nread > 0) {
            umma::mbar_wait(&bars[1], phT, abort_flag);
            phT ^= 1;
        }
        umma::fence_after_sync();
        STAMP();                                     // 5: S (and T) complete
        STAMP();                                     // 6
        // ---- S -> P (bf16, K-major A operand of P v).  This thread: row `row`, and in every 32-column
        //      block jb <= rb the 16 columns [jb*32 + ch*16, +16)
        // blocks above the diagonal: zeros
#pragma unroll 1
        for (int jb = rb + 1; jb < 4; ++jb) {
            const int j0 = jb * 32 + ch * 16;
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(sP + umma::tile_offset(row, j0 + c * 8, tc::PT)) = make_uint4(0u, 0u, 0u, 0u);
        }
        // Blocks below the diagonal, four columns at a time in run-time loops (one short copy of the body instead of
        // four unrolled 16-column copies: measured faster in this kernel, where the phase has a single accumulator).
#pragma unroll 1
        for (int jb = 0; jb < rb; ++jb) {
            // one level per block, decay factorised through the block end
            const float lm = ((rb ^ jb) == 1) ? lam[6] : lam[7];
            const float rf = lm * fexp(Gi - sGp[jb * 32 + 31]);
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
                const int j0 = jb * 32 + ch * 16 + cc * 4;
                float s[4];
                umma::tmem_ld4(umma::tmem_addr(tbase + tc::TM_S, warp, j0), s);
                const float4 cf = *reinterpret_cast<const float4*>(sCf + j0);
                *reinterpret_cast<uint2*>(sP + umma::tile_offset(row, j0, tc::PT)) =
                    make_uint2(pack_bf16(s[0] * rf * cf.x, s[1] * rf * cf.y), pack_bf16(s[2] * rf * cf.z, s[3] * rf * cf.w));
            }
        }
        // diagonal block: levels 0..5, causal mask folded into the exponent.  The level of (row, column) is the position of the
        // highest bit in which they differ: per bit, "differs" is the row's own bit or its complement, so lambda is picked by
        // selects on predicates instead of comparisons per element.
        const bool B0 = lane & 1, B1 = lane & 2, B2 = lane & 4, B3 = lane & 8;
        const bool hi = (((lane >> 4) & 1) != ch);
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
            const int jc = ch * 16 + cc * 4;             // first of the four columns, inside the block
            const int j0 = rb * 32 + jc;
            float s[4];
            umma::tmem_ld4(umma::tmem_addr(tbase + tc::TM_S, warp, j0), s);
            const float4 gj = *reinterpret_cast<const float4*>(sGp + j0);
            const float gjv[4] = {gj.x, gj.y, gj.z, gj.w};
            const bool q2 = B2 != bool(cc & 1), q3 = B3 != bool(cc & 2);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int jj = jc + u;
                const bool q1 = (u & 2) ? !B1 : B1, q0 = (u & 1) ? !B0 : B0;
                float lm = q0 ? lam[1] : lam[0];
                lm = q1 ? lam[2] : lm;
                lm = q2 ? lam[3] : lm;
                lm = q3 ? lam[4] : lm;
                lm = hi ? lam[5] : lm;
                const float d = (jj <= lane) ? (Gi - gjv[u]) : -INFINITY;
                s[u] = s[u] * fexp(d) * lm;
            }
            *reinterpret_cast<uint2*>(sP + umma::tile_offset(row, j0, tc::PT)) = make_uint2(pack_bf16(s[0], s[1]), pack_bf16(s[2], s[3]));
        }
        STAMP();                                     // 7: P written
        if (warp == TABLE_WARP && pl + 1 < npairs) {
            decay_tables(pl + 1);
            if (pl + 2 < npairs) fetch_g(pl + 2);
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();                                  // barrier 2
        umma::fence_after_sync();
        STAMP();                                     // 8: after barrier 2

        // ---- output row of this thread: columns ch*32 .. +31
        float o[32];
        if (hi_init) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(&ohi[c]);
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
        if (nread > 0) {
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
        STAMP();                                     // 9: level reads accumulated
        {
            umma::mbar_wait(&bars[2], phO, abort_flag);
            phO ^= 1;
            umma::fence_after_sync();
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tc::TM_O, warp, ch * 32), t);
            // P v has completed, so the P tile is free: stage the bf16 output rows there and copy
            // them out with 8 lanes per 128-byte row (coalesced) instead of one row per lane
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 x;
                uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) xw[e] = pack_bf16(o[c * 8 + e * 2] + t[c * 8 + e * 2], o[c * 8 + e * 2 + 1] + t[c * 8 + e * 2 + 1]);
                *reinterpret_cast<uint4*>(sP + umma::tile_offset(row, ch * 32 + c * 8, tc::PT)) = x;
            }
            asm volatile("bar.sync 2, 256;\n" ::: "memory");
            bf16* go = p.o + (((long)b * p.T + t0) * p.H + h) * tc::VD;
#pragma unroll
            for (int i = tid; i < tc::PT * 8; i += 256) {
                const int rr = i >> 3, c = (i & 7) * 8;
                *reinterpret_cast<uint4*>(go + (long)rr * p.H * tc::VD + c) =
                    *reinterpret_cast<const uint4*>(sP + umma::tile_offset(rr, c, tc::PT));
            }
        }
        STAMP();                                     // 10: output stored
        // ---- pair summary and the Fenwick carry over pair levels (thread = state row `row`)
        umma::mbar_wait(&bars[3], phKV, abort_flag);
        STAMP();                                     // 11: pair summary complete
        phKV ^= 1;
        umma::fence_after_sync();
        if (MP > 0 && pl + 1 < npairs) {
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
        if (pl + 1 < npairs) store_lam();            // every read of this pair's lambda is done (barrier 2)
        STAMP();                                     // 12: states merged
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();                                  // barrier 3
        umma::fence_after_sync();
        STAMP();                                     // 13: after barrier 3
        if (*abort_flag) break;                      // uniform: read after the barrier
    }
    umma::fence_before_sync();
    bar_work();
}

int mamba2_fwd_tc_launch(const Mamba2Params& p_in, cudaStream_t stream) {
    Mamba2Params p = p_in;
    int rc;
    if ((rc = tma::make_panel_map(&p.tm_q, p.q, (long)p.B * p.T, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_k, p.k, (long)p.B * p.T, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_v, p.v, (long)p.B * p.T, p.H, p.V, tc::PT)) != 0) return rc;
    auto kern = m2_chunk_fwd_tc_kernel<M2_MLOW>;
    const size_t sm = FwdTcSmem<M2_MLOW>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    kern<<<p.B * p.H * p.NS, tc::NTHREADS, sm, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

}  // namespace llattn

#ifdef LLATTN_STAMPS
extern "C" int llattn_debug_read_stamps(long long* host_dst) {
    return (int)cudaMemcpyFromSymbol(host_dst, llattn::g_stamps, sizeof(long long) * 3 * 32);
}
#endif
