// Log-linear Mamba-2 backward, forward-order pass, on tcgen05 / TMEM / TMA (K = 128, V = 64).
// Same mathematics as m2_bwd_fwdorder_kernel (mamba2_bwd.cu): per pair of chunks (128 tokens)
//   S  = q k^T, dP = do v^T                      -> dS = dP * decay * lambda (bf16 tile), dlambda bins
//   T  = q H_level (set pair levels)              -> dlambda of those levels = s_i (do_i . T_i)
//   dq = dS k + sum_levels (do * lambda s) H^T    (level part accumulated by the tensor core itself)
//   dk = dS^T q                                   (intra part; the level part comes from the reverse pass)
//   KV = k^T (v * decay)                          -> recomputed Fenwick level states (as the forward)
// dq and dk tiles leave the SM as fp32 TMA reduce-adds into the (B,T,G,K) accumulators (one bulk
// tensor operation per 128 x 32 box instead of per-thread red.global).  The gradient w.r.t. the
// in-chunk cumulative decay uses q_i.dq_i = sum_levels lambda[i,lev] dlambda[i,lev] (o is linear in
// lambda), so only k_j.dk_j needs a pass over a tile.
#include "tc_common.cuh"

namespace llattn {

namespace tcb {
// tensor memory columns
constexpr int TB_S = 0, TB_DP = 128, TB_KV = 256, TB_T0 = 320, TB_T1 = 384;   // first batch (+ KV in the second)
constexpr int TB_DQ = 0, TB_DK = 128;                                         // second batch reuses S / dP
constexpr int NDL = 11;                         // dlambda staging columns: 8 levels inside the pair, low pair levels, tile row sum
constexpr int LAMC = 12;                        // lambda columns staged per row (levels 0..7 and the low pair levels)
}  // namespace tcb

template <int MLOW>
struct Bwd1TcSmem {
    static constexpr int MP = MLOW - 1;
    static constexpr uint32_t q_off = 0;
    static constexpr uint32_t k_off = q_off + tc::Q_BYTES;
    static constexpr uint32_t v_off = k_off + tc::Q_BYTES;
    static constexpr uint32_t do_off = v_off + tc::V_BYTES;
    static constexpr uint32_t ds_off = do_off + tc::V_BYTES;               // dS tile (32 KB) ...
    static constexpr uint32_t dos_off = ds_off + tc::PT * tc::PT * 2;      // ... + 2 scaled do tiles (32 KB): also the 64 KB fp32 staging
    static constexpr uint32_t vs_off = dos_off + 2 * tc::V_BYTES;          // Vs (16 KB)
    static constexpr uint32_t h_off = vs_off + tc::V_BYTES;
    static constexpr uint32_t gp_off = h_off + (MP > 0 ? MP : 1) * tc::H_BYTES;   // float [3][128]
    static constexpr uint32_t lam_off = gp_off + 3 * 128 * 4;              // bf16 [128][LAMC] (only the columns this kernel reads)
    static constexpr uint32_t dl_off = lam_off + 128 * tcb::LAMC * 2;      // float [2][128][NDL] dlambda halves
    static constexpr uint32_t misc_off = dl_off + 2 * 128 * tcb::NDL * 4;  // float [512]: k.dk halves, per-chunk Z partials
    static constexpr uint32_t bar_off = misc_off + 2048;                   // mbarriers, tmem slot, abort flag
    static constexpr uint32_t total = bar_off + 128 + 1024;
};

// fp32 staging box for a TMA reduce: 128 rows x 32 floats, 128-byte swizzled
__device__ __forceinline__ uint32_t box_offset(int row, int col) {
    return (uint32_t)(row * 128 + (((col >> 2) ^ (row & 7)) << 4) + (col & 3) * 4);
}

template <int MLOW>
__global__ void __launch_bounds__(tc::NTHREADS, 1) m2_bwd_fwdorder_tc_kernel(const __grid_constant__ Mamba2Params p) {
    using SM = Bwd1TcSmem<MLOW>;
    constexpr int MP = SM::MP;
    constexpr int SEGP = 1 << MP;
    constexpr int NLAM = 8 + (MP > 0 ? MP : 1);
    static_assert(MP <= 2 && NLAM < tcb::NDL, "tensor memory / staging layout");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = smem + SM::q_off;
    unsigned char* sK = smem + SM::k_off;
    unsigned char* sV = smem + SM::v_off;
    unsigned char* sDO = smem + SM::do_off;
    unsigned char* sDS = smem + SM::ds_off;
    unsigned char* sDOs = smem + SM::dos_off;
    unsigned char* sStage = smem + SM::ds_off;          // 64 KB fp32 staging for dq = dS + scaled do (free once the second batch is done)
    unsigned char* sStage2 = smem + SM::q_off;          // 64 KB fp32 staging for dk = q + k tiles (free once the second batch and the k row sums are done)
    unsigned char* sVs = smem + SM::vs_off;
    float* sDL = reinterpret_cast<float*>(smem + SM::dl_off);            // [2][128][NDL]
    float* sWk = reinterpret_cast<float*>(smem + SM::misc_off);          // [4][128] partial k.dk per 32-column box; [4][16] Z partials at +256 (consumed before boxes 2, 3 write there)
    unsigned char* sH = smem + SM::h_off;
    float* sGp = reinterpret_cast<float*>(smem + SM::gp_off);
    float* sCf = sGp + 128;
    float* sVf = sGp + 256;
    bf16* sLam = reinterpret_cast<bf16*>(smem + SM::lam_off);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* barA = bars + 0;      // first MMA batch complete
    uint64_t* barB = bars + 1;      // second MMA batch complete
    uint64_t* full_qk = bars + 2;   // TMA: q tile
    uint64_t* full_vd = bars + 3;   // TMA: v and do tiles
    uint64_t* empty_qk = bars + 4;  // the q tile may be refilled (the first half of the dk reduce-add has read it)
    uint64_t* empty_vd = bars + 5;  // v / do tiles may be refilled
    uint64_t* dq_ready = bars + 6;  // the dq tile of the pair is staged (fp32) for the store agent
    uint64_t* dk_ready = bars + 7;  // ... columns 0..63 of the dk tile (128 arrivals: the warps of column half 0)
    uint64_t* stage_free = bars + 8;   // the store agent's reduce-adds have read both staging areas
    uint64_t* barDK = bars + 9;     // the dk product (first of the second batch) is complete: the q tile is free
    uint64_t* dk_ready1 = bars + 10;   // columns 64..127 of the dk tile are staged (128 arrivals: column half 1)
    uint64_t* full_k = bars + 11;   // TMA: k tile (loaded separately: its space is released later than the q tile's)
    uint64_t* empty_k = bars + 12;  // the k tile may be refilled (the second half of the dk reduce-add has read it)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 112);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 120);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Persistent CTAs: one per SM walks the (batch, segment, head) items blockIdx.x, blockIdx.x + gridDim.x, ...  Every role
    // runs the same item / pair sequence; mbarrier parities follow the running pair count `gs` of the CTA, and what a pair
    // prepares for the next one (lambda, decay tables, TMA loads) carries over from an item's last pair to the next item's
    // first, so that neither the tail of an item (its last reduce-adds) nor the launch of a CTA is paid per item.
    const int nitems = p.B * p.H * p.NS;
    int h, r, b, grp, npairs;
    auto decode = [&](int item) {
        h = item % p.H;
        r = (item / p.H) % p.NS;
        b = item / (p.H * p.NS);
        grp = h / (p.H / p.G);
        npairs = min(SEGP, p.NT / 2 - r * SEGP);
    };
    decode(blockIdx.x);
    const int L = p.L;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 10; ++i) umma::mbar_init(&bars[i], i == 7 ? 128 : 1);
        umma::mbar_init(dk_ready1, 256);
        umma::mbar_init(full_k, 1);
        umma::mbar_init(empty_k, 1);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    constexpr uint32_t ID_KK128 = umma::idesc_bf16(128, 128, false, false);
    constexpr uint32_t ID_KM64 = umma::idesc_bf16(128, 64, false, true);
    constexpr uint32_t ID_KM128 = umma::idesc_bf16(128, 128, false, true);
    constexpr uint32_t ID_MM128 = umma::idesc_bf16(128, 128, true, true);
    constexpr uint32_t ID_MM64 = umma::idesc_bf16(128, 64, true, true);

    if (warp >= tc::MMA_WARP) {
        RegisterSplit<56, 224>::release();
        if (warp == tc::MMA_WARP + 1) {
            // ---- TMA producer
            if (lane == 0) {
                uint32_t gs = 0;
                bool ok = true;
                for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x) {
                    decode(item);
                    const int brow = b * p.T + r * SEGP * tc::PT;
                    for (int pl = 0; pl < npairs; ++pl, ++gs) {
                        const int row0 = brow + pl * tc::PT;
                        if (gs >= 1 && !umma::mbar_wait(empty_vd, (gs - 1) & 1, abort_flag)) { ok = false; break; }
                        tma::expect_tx(full_vd, 2 * tc::V_BYTES);
                        tma::load_panel(sV, &p.tm_v, 0, h, row0, full_vd);
                        tma::load_panel(sDO, &p.tm_do, 0, h, row0, full_vd);
                        if (gs >= 1 && !umma::mbar_wait(empty_qk, (gs - 1) & 1, abort_flag)) { ok = false; break; }
                        tma::expect_tx(full_qk, tc::Q_BYTES);
                        tma::load_panel(sQ, &p.tm_q, 0, grp, row0, full_qk);
                        tma::load_panel(sQ + tc::Q_BYTES / 2, &p.tm_q, 64, grp, row0, full_qk);
                        if (gs >= 1 && !umma::mbar_wait(empty_k, (gs - 1) & 1, abort_flag)) { ok = false; break; }
                        tma::expect_tx(full_k, tc::Q_BYTES);
                        tma::load_panel(sK, &p.tm_k, 0, grp, row0, full_k);
                        tma::load_panel(sK + tc::Q_BYTES / 2, &p.tm_k, 64, grp, row0, full_k);
                    }
                }
            }
            return;
        }
        if (warp == tc::MMA_WARP + 2) {
            // ---- store agent: issues the fp32 TMA reduce-adds of the staged dk / dq tiles and is the one that
            //      waits for them, so that no element-wise thread stalls on a bulk-group wait; the q / k tile space
            //      (which doubles as the dk staging area) is freed as soon as the dk reduce-add has read it
            if (lane == 0) {
                uint32_t gs = 0;
                bool ok = true;
                for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x) {
                  decode(item);
                  for (int pl = 0; pl < npairs; ++pl, ++gs) {
                    const int grow = b * p.T + (r * SEGP + pl) * tc::PT;
                    // dk first: its staging area is the q / k tile space, which the next pair's loads wait for
                    // (in two halves: columns 0..63 are staged in the q tile as soon as the dk product is complete, columns
                    // 64..127 in the k tile once the whole batch is, so that half of the reduce-add is over by then)
                    if (!umma::mbar_wait(dk_ready, gs & 1, abort_flag)) { ok = false; break; }
#pragma unroll
                    for (int bx = 0; bx < 2; ++bx) tma::reduce_add_box(&p.tm_dk, bx * 32, grp, grow, sStage2 + bx * 16384);
                    tma::commit_group();
                    tma::wait_group_read0();             // the q tile's space has been read: the next q may be loaded
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(empty_qk)) : "memory");
                    if (!umma::mbar_wait(dk_ready1, gs & 1, abort_flag)) { ok = false; break; }
#pragma unroll
                    for (int bx = 2; bx < 4; ++bx) tma::reduce_add_box(&p.tm_dk, bx * 32, grp, grow, sStage2 + bx * 16384);
                    tma::commit_group();
                    tma::wait_group_read0();
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(empty_k)) : "memory");
                    if (!umma::mbar_wait(dq_ready, gs & 1, abort_flag)) { ok = false; break; }
#pragma unroll
                    for (int bx = 0; bx < 4; ++bx) tma::reduce_add_box(&p.tm_dq, bx * 32, grp, grow, sStage + bx * 16384);
                    tma::commit_group();
                    tma::wait_group_read0();
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(stage_free)) : "memory");
                  }
                }
                tma::wait_group0();                  // every reduce-add has been performed before the CTA retires
            }
            return;
        }
        if (warp > tc::MMA_WARP) return;
        // ---- MMA issuer
        umma::tmem_alloc(tmem_slot, tc::TM_COLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        const uint32_t aQ = umma::smem_addr(sQ), aK = umma::smem_addr(sK), aV = umma::smem_addr(sV), aDO = umma::smem_addr(sDO);
        const uint32_t aDS = umma::smem_addr(sDS), aDOs = umma::smem_addr(sDOs), aVs = umma::smem_addr(sVs);
        uint32_t gs = 0;
        for (int item = blockIdx.x; item < nitems && !*abort_flag; item += gridDim.x) {
          decode(item);
          for (int pl = 0; pl < npairs; ++pl, ++gs) {
            // (no barrier here: the end-of-pair barrier of the previous pair is all the tensor core needs)
            if (lane == 0) {
                // dP needs only v and do, which land long before q and k (their space doubles as the dk staging area)
                umma::mbar_wait(full_vd, gs & 1, abort_flag);
                umma::gemm_kk<tc::PT, tc::PT, tc::VD>(tbase + tcb::TB_DP, aDO, aV, ID_KK128, false);
                // the level reads need q only; S = q k^T goes last, when the k tile (released last) has landed
                umma::mbar_wait(full_qk, gs & 1, abort_flag);
                int slot = 0;
#pragma unroll
                for (int lv = 0; lv < MP; ++lv)
                    if ((pl >> lv) & 1) {
                        umma::gemm_km<tc::PT, tc::KD, tc::KD>(tbase + (slot == 0 ? tcb::TB_T0 : tcb::TB_T1), aQ,
                                                              umma::smem_addr(sH + lv * tc::H_BYTES), ID_KM64, false);
                        ++slot;
                    }
                umma::mbar_wait(full_k, gs & 1, abort_flag);
                umma::gemm_kk<tc::PT, tc::PT, tc::KD>(tbase + tcb::TB_S, aQ, aK, ID_KK128, false);
                umma::commit(barA);
            }
            __syncwarp();
            umma::fence_before_sync();
            bar_work();                              // barrier 2: dS, scaled do and Vs are written
            umma::fence_after_sync();
            if (lane == 0) {
                // dk = dS^T q first (the q tile becomes staging space when it is complete), dq = dS k (+ level parts), KV = k^T Vs
                umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase + tcb::TB_DK, aDS, aQ, ID_MM128, false);
                umma::commit(barDK);
                umma::gemm_km<tc::PT, tc::PT, tc::PT>(tbase + tcb::TB_DQ, aDS, aK, ID_KM128, false);
                int slot = 0;
#pragma unroll
                for (int lv = 0; lv < MP; ++lv)
                    if ((pl >> lv) & 1) {
                        umma::gemm_kk<tc::PT, tc::KD, tc::VD>(tbase + tcb::TB_DQ, aDOs + slot * tc::V_BYTES,
                                                              umma::smem_addr(sH + lv * tc::H_BYTES), ID_KK128, true);
                        ++slot;
                    }
                umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase + tcb::TB_KV, aK, aVs, ID_MM64, false);
                umma::commit(barB);
                // v and do were last read (generic loads and the first batch) before barrier 2
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(empty_vd)) : "memory");
            }
            __syncwarp();
            umma::fence_before_sync();
            bar_work();                              // barrier 3: end of the pair
            umma::fence_after_sync();
            if (*abort_flag) break;
          }
        }
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();
        umma::tmem_dealloc(tbase, tc::TM_COLS);
        return;
    }

    // ================= warps 0..7 =================
    RegisterSplit<56, 224>::acquire();
    const int rb = warp & 3;
    const int row = rb * 32 + lane;
    const int ch = warp >> 2;

    float g_n[4];
    constexpr int LAMR = (tc::PT * NLAM + 255) / 256;   // only the NLAM columns these kernels read are fetched
    uint32_t lam_r[LAMR];
    uint32_t lam_rc[LAMR];
    const int NC = L < NLAM ? L : NLAM;             // columns of a lambda row that are fetched
#pragma unroll
    for (int i = 0; i < LAMR; ++i) {
        const int e = tid + i * 256;
        const int rr = e / NC, cc = e - rr * NC;
        lam_rc[i] = (rr < tc::PT) ? (uint32_t)((rr << 8) | cc) : 0xffffffffu;
    }
    // (tok0: first token of the pair counted over the whole batch, b * T + t0; hh: its head)
    auto fetch_small = [&](long tok0, int hh) {
        const unsigned short* lp = reinterpret_cast<const unsigned short*>(p.l) + (tok0 * p.H + hh) * L;
#pragma unroll
        for (int i = 0; i < LAMR; ++i)
            if (lam_rc[i] != 0xffffffffu) lam_r[i] = lp[(long)(lam_rc[i] >> 8) * p.H * L + (lam_rc[i] & 255)];
    };
    // raw g of a pair: one warp (the one that builds the decay tables), four consecutive tokens per lane
    auto fetch_g = [&](long tok0, int hh) {
        const float* gp = p.g + (tok0 + 4 * lane) * p.H + hh;
#pragma unroll
        for (int i = 0; i < 4; ++i) g_n[i] = gp[(long)i * p.H];
    };
    // Decay tables of a pair from the g values in g_n, by one full warp: G (pair-wide inclusive cumulative sum),
    // Cf = exp(G[end of 32-block] - G[j]), Vf = exp(G[127] - G[j]).  Built ahead of the pair that reads them, so that
    // a pair starts without a barrier of its own.
    auto decay_tables = [&](float* tG) {
        float gq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) gq[i] = g_n[i];
        gq[1] += gq[0];
        gq[2] += gq[1];
        gq[3] += gq[2];
        float tot = gq[3];
#pragma unroll
        for (int d = 1; d < 16; d <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, tot, d);
            if ((lane & 15) >= d) tot += t;
        }
        const float gla = __shfl_sync(0xffffffffu, tot, 15);
        const float glb = __shfl_sync(0xffffffffu, tot, 31);
        const float glp = gla + glb;
        const float pbase = tot - gq[3] + (lane >= 16 ? gla : 0.f);
        const float gend = __shfl_sync(0xffffffffu, tot, (lane & ~7) + 7) + (lane >= 16 ? gla : 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float G = pbase + gq[i];
            tG[4 * lane + i] = G;
            tG[128 + 4 * lane + i] = fexp(gend - G);
            tG[256 + 4 * lane + i] = fexp(glp - G);
        }
    };
    constexpr int TABLE_WARP = 4;                    // lane quarter 0, column half 1: the warp with the most slack
    auto store_lam = [&]() {
#pragma unroll
        for (int i = 0; i < LAMR; ++i)
            if (lam_rc[i] != 0xffffffffu)
                if ((lam_rc[i] & 255) < tcb::LAMC) sLam[(lam_rc[i] >> 8) * tcb::LAMC + (lam_rc[i] & 255)] = __ushort_as_bfloat16((unsigned short)lam_r[i]);
    };
    {
        const long tok0 = (long)b * p.T + (long)r * SEGP * tc::PT;       // first pair of the CTA's first item
        fetch_small(tok0, h);
        store_lam();
        if (warp == TABLE_WARP) {
            fetch_g(tok0, h);
            decay_tables(sGp);
        }
    }
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;

    float M[MP > 0 ? MP : 1][32];
    float dsum[MP > 0 ? MP : 1];
    uint32_t gs = 0;                                  // pairs this CTA has started: mbarrier parities
    bool alive = true;

    for (int item = blockIdx.x; item < nitems && alive; item += gridDim.x) {
      decode(item);
#pragma unroll
      for (int i = 0; i < (MP > 0 ? MP : 1); ++i) dsum[i] = 0.f;
      for (int pl = 0; pl < npairs; ++pl, ++gs) {
#ifdef LLATTN_STAMPS
        int nstamp = 0;
        const int stamp_slot = (blockIdx.x == 5 && gs == 6) ? (tid == 0 ? 0 : (tid == 200 ? 1 : (tid == 96 ? 2 : -1))) : -1;
#endif
        STAMP();   // 0 top
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        // the pair after this one: the next of the segment, or the first pair of the CTA's next item
        const int nitem = item + gridDim.x;
        const bool have_next = (pl + 1 < npairs) || (nitem < nitems);
        long ntok = (long)b * p.T + t0 + tc::PT;
        int nh = h;
        if (pl + 1 >= npairs && nitem < nitems) {
            nh = nitem % p.H;
            ntok = (long)(nitem / (p.H * p.NS)) * p.T + (long)((nitem / p.H) % p.NS) * SEGP * tc::PT;
        }
        if (have_next) {
            fetch_small(ntok, nh);
            if (warp == TABLE_WARP) fetch_g(ntok, nh);
        }
        STAMP();   // 1 small fetches issued
        int nread = 0;
#pragma unroll
        for (int lv = 0; lv < MP; ++lv) nread += (pl >> lv) & 1;
        const float Gi = sGp[row];
        const float glp = sGp[tc::PT - 1];
        float lam[NLAM];
#pragma unroll
        for (int i = 0; i < NLAM; ++i) lam[i] = (i < L) ? __bfloat162float(sLam[row * tcb::LAMC + i]) : 0.f;

        umma::mbar_wait(full_vd, gs & 1, abort_flag);
        umma::mbar_wait(full_qk, gs & 1, abort_flag);
        umma::mbar_wait(full_k, gs & 1, abort_flag);
        umma::mbar_wait(barA, gs & 1, abort_flag);
        if (gs >= 1) umma::mbar_wait(stage_free, (gs - 1) & 1, abort_flag);   // dS / scaled-do space was the dq staging area
        umma::fence_after_sync();

        STAMP();   // 2 batch A complete
        // ---- S, dP -> dS (bf16 tile) and the dlambda sums of the 8 levels inside the pair
        float bins[8];
        float wq_tile = 0.f;                         // sum_j bf16(dS_ij) S_ij: q_i.dq_i of the tile product, same rounding as dk
#pragma unroll
        for (int i = 0; i < 8; ++i) bins[i] = 0.f;
        // blocks above the diagonal: zeros
#pragma unroll 1
        for (int jb = rb + 1; jb < 4; ++jb) {
            const int j0 = jb * 32 + ch * 16;
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(sDS + umma::tile_offset(row, j0 + c * 8, tc::PT)) = make_uint4(0u, 0u, 0u, 0u);
        }
        // blocks below the diagonal: one level per block, decay factorised through the block end.  A run-time loop
        // (one copy of the body): the fully unrolled form made the loop body larger than the instruction cache.
#pragma unroll 1
        for (int jb = 0; jb < rb; ++jb) {
            const int j0 = jb * 32 + ch * 16;
            uint32_t packed[8];
            float s[16], dp[16];
            umma::tmem_ld16x2(umma::tmem_addr(tbase + tcb::TB_S, warp, j0), s, umma::tmem_addr(tbase + tcb::TB_DP, warp, j0), dp);
            const bool lev6 = ((rb ^ jb) == 1);
            const float lm = lev6 ? lam[6] : lam[7];
            const float rf = fexp(Gi - sGp[jb * 32 + 31]);
            float bsum = 0.f;
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
                const float4 cf = *reinterpret_cast<const float4*>(sCf + j0 + e);
                const float cfv[4] = {cf.x, cf.y, cf.z, cf.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float ed = dp[e + u] * rf * cfv[u];
                    bsum += ed * s[e + u];
                    const float dsv = ed * lm;
                    wq_tile += __bfloat162float(__float2bfloat16(dsv)) * s[e + u];
                    s[e + u] = dsv;
                }
                packed[e >> 1] = pack_bf16(s[e], s[e + 1]);
                packed[(e >> 1) + 1] = pack_bf16(s[e + 2], s[e + 3]);
            }
            if (lev6) bins[6] += bsum; else bins[7] += bsum;
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(sDS + umma::tile_offset(row, j0 + c * 8, tc::PT)) =
                    make_uint4(packed[c * 4], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
        }
        // diagonal block: levels 0..5, causal mask folded into the exponent
        STAMP();   // 2a blocks off the diagonal done
        {
            const int j0 = rb * 32 + ch * 16;
            uint32_t packed[8];
            float s[16], dp[16];
            umma::tmem_ld16x2(umma::tmem_addr(tbase + tcb::TB_S, warp, j0), s, umma::tmem_addr(tbase + tcb::TB_DP, warp, j0), dp);
            STAMP();   // 2b diagonal block loaded
            // The level of (row li, column jj) is the position of the highest bit in which they differ.  With the column's
            // low four bits a compile-time constant, "bit k differs" is one of the thread's own bits or its complement, so
            // lambda is picked with four selects on precomputed predicates; and the d lambda sum of level k is the sum over
            // the sibling block of size 2^(k-1) of the row's own position, taken from a binary tree of partial sums (15
            // additions and 30 selects per thread instead of six predicated additions per element).  A thread whose
            // sixteen columns lie in the other half of the 32-block (bit 4 differs) has level 5 throughout.
            const int li = lane;
            const bool B0 = li & 1, B1 = li & 2, B2 = li & 4, B3 = li & 8;
            const bool hi = (((li >> 4) & 1) != ch);
            // per half of eight columns: what the levels 0..3 would get if the row's own position lay in this half, and the half's sum
            float c_own[2], c_sib1[2], c_sib2[2], c_sib4[2], c_sum[2];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                float es[8];
#pragma unroll
                for (int e = 0; e < 8; e += 4) {
                    const float4 gj = *reinterpret_cast<const float4*>(sGp + j0 + hf * 8 + e);
                    const float gjv[4] = {gj.x, gj.y, gj.z, gj.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int ee = hf * 8 + e + u;                     // low four bits of the column
                        const int jj = ch * 16 + ee;
                        const float d = (jj <= li) ? (Gi - gjv[u]) : -INFINITY;
                        const float ed = dp[ee] * fexp(d);
                        es[e + u] = ed * s[ee];
                        const bool q3 = hf ? !B3 : B3, q2 = ((ee >> 2) & 1) ? !B2 : B2;
                        const bool q1 = ((ee >> 1) & 1) ? !B1 : B1, q0 = (ee & 1) ? !B0 : B0;
                        float lm = q0 ? lam[1] : lam[0];
                        lm = q1 ? lam[2] : lm;
                        lm = q2 ? lam[3] : lm;
                        lm = q3 ? lam[4] : lm;
                        lm = hi ? lam[5] : lm;
                        const float dsv = ed * lm;
                        wq_tile += __bfloat162float(__float2bfloat16(dsv)) * s[ee];
                        s[ee] = dsv;
                    }
                    packed[(hf * 8 + e) >> 1] = pack_bf16(s[hf * 8 + e], s[hf * 8 + e + 1]);
                    packed[((hf * 8 + e) >> 1) + 1] = pack_bf16(s[hf * 8 + e + 2], s[hf * 8 + e + 3]);
                }
                // walk down the half's tree of partial sums along the row's own bits 2, 1, 0
                const float p0 = es[0] + es[1], p1 = es[2] + es[3], p2 = es[4] + es[5], p3 = es[6] + es[7];
                const float q0s = p0 + p1, q1s = p2 + p3;
                c_sum[hf] = q0s + q1s;
                c_sib4[hf] = B2 ? q0s : q1s;
                const float e0 = B2 ? p2 : p0, e1 = B2 ? p3 : p1;
                c_sib2[hf] = B1 ? e0 : e1;
                float f4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) f4[i] = B2 ? es[4 + i] : es[i];
                const float g0 = B1 ? f4[2] : f4[0], g1 = B1 ? f4[3] : f4[1];
                c_sib1[hf] = B0 ? g0 : g1;
                c_own[hf] = B0 ? g1 : g0;
            }
            bins[0] += hi ? 0.f : (B3 ? c_own[1] : c_own[0]);
            bins[1] += hi ? 0.f : (B3 ? c_sib1[1] : c_sib1[0]);
            bins[2] += hi ? 0.f : (B3 ? c_sib2[1] : c_sib2[0]);
            bins[3] += hi ? 0.f : (B3 ? c_sib4[1] : c_sib4[0]);
            bins[4] += hi ? 0.f : (B3 ? c_sum[0] : c_sum[1]);
            bins[5] += hi ? (c_sum[0] + c_sum[1]) : 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(sDS + umma::tile_offset(row, j0 + c * 8, tc::PT)) =
                    make_uint4(packed[c * 4], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
        }
        STAMP();   // 3 dS written
        float* myDL = sDL + (ch * 128 + row) * tcb::NDL;
#pragma unroll
        for (int i = 0; i < 8; ++i) myDL[i] = bins[i];
        myDL[tcb::NDL - 1] = wq_tile;
        // ---- level reads: dlambda = s_i (do_i . T_i) ; scaled copy of do for the dq product
        {
            uint4 dox[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) dox[c] = *reinterpret_cast<const uint4*>(sDO + umma::tile_offset(row, ch * 32 + c * 8, tc::PT));
            int slot = 0;
#pragma unroll
            for (int lv = 0; lv < MP; ++lv) {
                float val = 0.f;
                if ((pl >> lv) & 1) {
                    float t[32];
                    umma::tmem_ld32(umma::tmem_addr(tbase + (slot == 0 ? tcb::TB_T0 : tcb::TB_T1), warp, ch * 32), t);
                    const float sc = fexp(Gi + dsum[lv]);
                    const float rs = lam[8 + lv] * sc;
                    float dot = 0.f;
                    unsigned char* dst = sDOs + slot * tc::V_BYTES;
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
                        *reinterpret_cast<uint4*>(dst + umma::tile_offset(row, ch * 32 + c * 8, tc::PT)) =
                            make_uint4(outw[0], outw[1], outw[2], outw[3]);
                    }
                    val = sc * dot;
                    ++slot;
                }
                myDL[8 + lv] = val;
            }
        }
        STAMP();   // 4 level reads done
        // ---- Vs = v * exp(glp - G_j)
        {
#pragma unroll
            for (int i = tid; i < tc::PT * (tc::VD / 8); i += 256) {
                const int j = i / (tc::VD / 8), c = (i % (tc::VD / 8)) * 8;
                const float sc = sVf[j];
                const uint32_t off = umma::tile_offset(j, c, tc::PT);
                uint4 x = *reinterpret_cast<const uint4*>(sV + off);
                uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v2 = *reinterpret_cast<__nv_bfloat162*>(&xw[e]);
                    xw[e] = pack_bf16(__bfloat162float(v2.x) * sc, __bfloat162float(v2.y) * sc);
                }
                *reinterpret_cast<uint4*>(sVs + off) = x;
            }
        }
        STAMP();   // 5 Vs written
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();                                  // barrier 2 (also: dlambda halves of every row are in shared memory)
        umma::fence_after_sync();
        STAMP();   // 6 after barrier 2
        // every read of this pair's decay tables is behind barrier 2 (what follows uses Gi / glp from registers):
        // one warp rebuilds them for the next pair while the second batch runs
        if (warp == TABLE_WARP && have_next) decay_tables(sGp);
        // ---- dk tile: k_j . dk_j row sums, then fp32 staging for the TMA reduce-add.  The staging area is the q / k tile space,
        //      which the next pair's loads wait for, so it is filled as early as its halves become free: columns 0..63 (the
        //      warps of column half 0) go into the q tile as soon as the dk product - issued first in the batch - is complete,
        //      columns 64..127 into the k tile once dq and KV are complete and every thread is done with its k row sums.
        // One 32-column box of the dk tile: k . dk partial row sum (slot `slot` of sWk), fp32 staging of the box
        auto dk_box = [&](int bx, int slot, bool k_tile_barrier) {
            float dkv[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tcb::TB_DK, warp, bx * 32), dkv);
            float wk_part = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 kx = *reinterpret_cast<const uint4*>(sK + umma::tile_offset(row, bx * 32 + c * 8, tc::PT));
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(&kx);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[e]);
                    wk_part += __bfloat162float(v2.x) * dkv[c * 8 + e * 2] + __bfloat162float(v2.y) * dkv[c * 8 + e * 2 + 1];
                }
            }
            sWk[slot * 128 + row] = wk_part;
            if (k_tile_barrier) bar_compute();       // every thread is done with the k tile that the boxes 2 and 3 overwrite
            unsigned char* box = sStage2 + bx * 16384;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<float4*>(box + box_offset(row, c * 4)) = make_float4(dkv[c * 4], dkv[c * 4 + 1], dkv[c * 4 + 2], dkv[c * 4 + 3]);
        };
        if (ch == 0) {
            // columns 0..63 (boxes 0, 1) by the warps of column half 0, into the q tile
            umma::mbar_wait(barDK, gs & 1, abort_flag);
            umma::fence_after_sync();
            dk_box(0, 0, false);
            dk_box(1, 1, false);
            umma::fence_async_smem();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(dk_ready)) : "memory");
        }
        // ---- while the second batch runs: dlambda out (coalesced), q.dq row sums, reader totals Z per chunk
        {
            float* gdl = p.dl + (((long)b * p.T + t0) * p.H + h) * L;
#pragma unroll
            for (int e = tid; e < tc::PT * NLAM; e += 256) {
                const int rr = e / NLAM, i = e - rr * NLAM;
                if (i < L) gdl[(long)rr * p.H * L + i] = sDL[rr * tcb::NDL + i] + sDL[(128 + rr) * tcb::NDL + i];
            }
        }
        float wq_row = 0.f;                          // valid for ch == 1 threads: q_i . dq_i  (column half 0 stages its dk half meanwhile)
        if (ch == 1) {
            float zl[NLAM];
#pragma unroll
            for (int i = 0; i < NLAM; ++i) {
                zl[i] = lam[i] * (sDL[row * tcb::NDL + i] + sDL[(128 + row) * tcb::NDL + i]);
                if (i >= 8) wq_row += zl[i];         // level reads; the 8 levels inside the pair come from the tile sum
            }
            wq_row += sDL[row * tcb::NDL + tcb::NDL - 1] + sDL[(128 + row) * tcb::NDL + tcb::NDL - 1];
#pragma unroll
            for (int i = 7; i < NLAM; ++i) {
                float z = zl[i];
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) z += __shfl_xor_sync(0xffffffffu, z, d);
                if (lane == 0) sWk[256 + rb * 16 + i] = z;
            }
        }
        bar_compute();
        if (tid < 2 * (NLAM - 7)) {
            // tid -> (chunk of the pair, level index i >= 7): Z[c][lv] for readers, Y[c][0] for the level inside the pair
            const int cpart = tid / (NLAM - 7), i = 7 + tid % (NLAM - 7);
            const float z = sWk[256 + (cpart * 2) * 16 + i] + sWk[256 + (cpart * 2 + 1) * 16 + i];
            const long cidx = ((long)b * p.H + h) * p.NT + (r * SEGP + pl) * 2 + cpart;
            if (i == 7) {
                if (cpart == 1) {
                    p.Zc[cidx * p.LZ + 0] = z;                         // chunk level 0: reader is the second chunk
                    p.Yc[(cidx - 1) * (MLOW + 1) + 0] = z;             // ... and its contributor total, same block pair
                }
            } else if ((pl >> (i - 8)) & 1) {
                p.Zc[cidx * p.LZ + (i - 7)] = z;                       // pair level i-8 = chunk level i-7
            }
        }
        STAMP();   // 7 dl / Z out

        umma::mbar_wait(barB, gs & 1, abort_flag);
        umma::fence_after_sync();
        STAMP();   // 8 batch B complete
        // columns 64..127 (boxes 2, 3) into the k tile: one box per warp of a lane quarter, so that this step on the critical
        // path (the k tile's reload waits for the reduce-add of these boxes) takes half as long
        dk_box(2 + ch, 2 + ch, true);
        umma::fence_async_smem();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(dk_ready1)) : "memory");
        STAMP();   // 9 dk staged
        // ---- dq tile -> fp32 staging (dS + scaled do space) -> TMA reduce-add
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tcb::TB_DQ, warp, ch * 64 + hb * 32), t);
            unsigned char* box = sStage + (ch * 2 + hb) * 16384;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<float4*>(box + box_offset(row, c * 4)) = make_float4(t[c * 4], t[c * 4 + 1], t[c * 4 + 2], t[c * 4 + 3]);
        }
        STAMP();   // 10 dq staged
        umma::fence_async_smem();
        bar_compute();
        if (tid == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(dq_ready)) : "memory");
        if (ch == 1) {
            const float w = wq_row - ((sWk[row] + sWk[128 + row]) + (sWk[256 + row] + sWk[384 + row]));
            red_add_f32(p.wq + ((long)b * p.T + t0 + row) * p.H + h, w);
        }
        STAMP();   // 11 reduces issued
        // ---- pair summary and the Fenwick carry over pair levels
        if (MP > 0 && pl + 1 < npairs) {
            const int j = __ffs(~pl) - 1;
            if (j < MP) {
                float kv[32];
                umma::tmem_ld32(umma::tmem_addr(tbase + tcb::TB_KV, warp, ch * 32), kv);
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
        STAMP();   // 12 states merged
        if (have_next) store_lam();
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();                                  // barrier 3
        STAMP();   // 13 after barrier 3
        umma::fence_after_sync();
        if (*abort_flag) { alive = false; break; }
      }
    }
    umma::fence_before_sync();
    bar_work();
}

// ------------------------------------------------------------------------------------------
// reverse-order pass: dv, the level part of dk, adjoint level states
// ------------------------------------------------------------------------------------------
namespace tcr {
constexpr int TR_S = 0;                                              // first batch
constexpr int TR_DVA = 128, TR_DVB = 192, TR_DK = 256, TR_KVA = 384, TR_KVB = 448, TR_DH0 = 0, TR_DH1 = 64;   // second batch
}  // namespace tcr

template <int MLOW>
struct Bwd2TcSmem {
    static constexpr int MP = MLOW - 1;
    static constexpr uint32_t q_off = 0;
    static constexpr uint32_t k_off = q_off + tc::Q_BYTES;
    static constexpr uint32_t v_off = k_off + tc::Q_BYTES;
    static constexpr uint32_t do_off = v_off + tc::V_BYTES;
    static constexpr uint32_t p_off = do_off + tc::V_BYTES;                // P tile (32 KB) ...
    static constexpr uint32_t dos_off = p_off + tc::PT * tc::PT * 2;       // ... + 2 scaled do tiles: also the 64 KB fp32 staging
    static constexpr uint32_t vs_off = dos_off + 2 * tc::V_BYTES;
    static constexpr uint32_t dkv_off = vs_off + tc::V_BYTES;              // bf16 [128 features][64]
    static constexpr uint32_t gp_off = dkv_off + tc::H_BYTES;              // float [2][3][128]: decay tables of this pair and the next
    static constexpr uint32_t lam_off = gp_off + 2 * 3 * 128 * 4;
    static constexpr uint32_t misc_off = lam_off + 128 * tc::LAM_LD * 2;   // float [512]
    static constexpr uint32_t bar_off = misc_off + 2048;
    static constexpr uint32_t total = bar_off + 128 + 1024;
};

template <int MLOW>
__global__ void __launch_bounds__(tc::NTHREADS, 1) m2_bwd_revorder_tc_kernel(const __grid_constant__ Mamba2Params p) {
    using SM = Bwd2TcSmem<MLOW>;
    constexpr int MP = SM::MP;
    constexpr int SEGP = 1 << MP;
    constexpr int NLAM = 8 + (MP > 0 ? MP : 1);
    static_assert(MP <= 2, "tensor memory layout");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = smem + SM::q_off;
    unsigned char* sK = smem + SM::k_off;
    unsigned char* sV = smem + SM::v_off;
    unsigned char* sDO = smem + SM::do_off;
    unsigned char* sP = smem + SM::p_off;
    unsigned char* sDOs = smem + SM::dos_off;
    unsigned char* sStage = smem + SM::p_off;
    unsigned char* sVs = smem + SM::vs_off;
    unsigned char* sDKV = smem + SM::dkv_off;
    float* sTab = reinterpret_cast<float*>(smem + SM::gp_off);           // [2][3][128]: per pair G | Cf | Vf
    bf16* sLam = reinterpret_cast<bf16*>(smem + SM::lam_off);
    float* sMisc = reinterpret_cast<float*>(smem + SM::misc_off);        // [2][128] k.dk halves ; [8][8] Y partials at +256
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* barA = bars + 0;
    uint64_t* barB = bars + 1;
    uint64_t* full_qk = bars + 2;
    uint64_t* full_vd = bars + 3;
    uint64_t* empty_qvd = bars + 4;    // the second batch is complete: q, v and do may be overwritten
    uint64_t* empty_k = bars + 5;      // ... and the compute warps have taken their k row sums
    uint64_t* dk_ready = bars + 6;     // the dk tile of the pair is staged (fp32) for the store agent
    uint64_t* stage_free = bars + 7;   // the store agent's reduce-add has read the staging area
    uint64_t* barB1 = bars + 8;        // the part of the second batch that does not need P is complete
    uint64_t* early_ready = bars + 9;  // every element-wise thread has written its part of dKV, Vs and the scaled do (256 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 104);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % p.H;
    const int r = (blockIdx.x / p.H) % p.NS;
    const int b = blockIdx.x / (p.H * p.NS);
    const int grp = h / (p.H / p.G);
    const int L = p.L;
    const int npairs = min(SEGP, p.NT / 2 - r * SEGP);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 9; ++i) umma::mbar_init(&bars[i], i == 5 ? 256 : 1);   // empty_k: one arrival per element-wise thread
        umma::mbar_init(early_ready, 256);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    constexpr uint32_t ID_KK128 = umma::idesc_bf16(128, 128, false, false);
    constexpr uint32_t ID_KM64 = umma::idesc_bf16(128, 64, false, true);
    constexpr uint32_t ID_MM64 = umma::idesc_bf16(128, 64, true, true);

    if (warp >= tc::MMA_WARP) {
        RegisterSplit<56, 224>::release();
        if (warp == tc::MMA_WARP + 1) {
            if (lane == 0) {
                const int brow = b * p.T + r * SEGP * tc::PT;
                for (int it = 0; it < npairs; ++it) {
                    const int row0 = brow + (npairs - 1 - it) * tc::PT;
                    // k is free once the element-wise threads have taken its row sums (its products belong to the early part of
                    // the second batch); q, v, do once the whole second batch is done: the loads overlap the read-out of that
                    // pair's results
                    if (it >= 1 && !umma::mbar_wait(empty_k, (it - 1) & 1, abort_flag)) break;
                    tma::expect_tx(full_qk, 2 * tc::Q_BYTES);
                    tma::load_panel(sK, &p.tm_k, 0, grp, row0, full_qk);
                    tma::load_panel(sK + tc::Q_BYTES / 2, &p.tm_k, 64, grp, row0, full_qk);
                    if (it >= 1 && !umma::mbar_wait(empty_qvd, (it - 1) & 1, abort_flag)) break;
                    tma::load_panel(sQ, &p.tm_q, 0, grp, row0, full_qk);
                    tma::load_panel(sQ + tc::Q_BYTES / 2, &p.tm_q, 64, grp, row0, full_qk);
                    tma::expect_tx(full_vd, 2 * tc::V_BYTES);
                    tma::load_panel(sV, &p.tm_v, 0, h, row0, full_vd);
                    tma::load_panel(sDO, &p.tm_do, 0, h, row0, full_vd);
                }
            }
            return;
        }
        if (warp == tc::MMA_WARP + 2) {
            // ---- store agent: issues the fp32 TMA reduce-add of the staged dk tile and waits for it, so that no
            //      element-wise thread stalls on a bulk-group wait
            if (lane == 0) {
                for (int it = 0; it < npairs; ++it) {
                    const int grow = b * p.T + (r * SEGP + (npairs - 1 - it)) * tc::PT;
                    if (!umma::mbar_wait(dk_ready, it & 1, abort_flag)) break;
#pragma unroll
                    for (int bx = 0; bx < 4; ++bx) tma::reduce_add_box(&p.tm_dk, bx * 32, grp, grow, sStage + bx * 16384);
                    tma::commit_group();
                    tma::wait_group_read0();
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(stage_free)) : "memory");
                }
                tma::wait_group0();
            }
            return;
        }
        if (warp > tc::MMA_WARP) return;
        umma::tmem_alloc(tmem_slot, tc::TM_COLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        const uint32_t aQ = umma::smem_addr(sQ), aK = umma::smem_addr(sK), aDO = umma::smem_addr(sDO);
        const uint32_t aP = umma::smem_addr(sP), aDOs = umma::smem_addr(sDOs), aVs = umma::smem_addr(sVs), aDKV = umma::smem_addr(sDKV);
        for (int it = 0; it < npairs; ++it) {
            const int pl = npairs - 1 - it;
            // (no barrier here: the end-of-pair barrier of the previous pair is all the tensor core needs)
            if (lane == 0) {
                umma::mbar_wait(full_qk, it & 1, abort_flag);
                umma::gemm_kk<tc::PT, tc::PT, tc::KD>(tbase + tcr::TR_S, aQ, aK, ID_KK128, false);
                umma::commit(barA);
                // the products that do not need P run while the element-wise warps turn S into P
                umma::mbar_wait(early_ready, it & 1, abort_flag);
                umma::fence_after_sync();
                umma::gemm_km<tc::PT, tc::KD, tc::KD>(tbase + tcr::TR_DVB, aK, aDKV, ID_KM64, false);         // k dKV
                umma::gemm_kk<tc::PT, tc::KD, tc::VD>(tbase + tcr::TR_DK, aVs, aDKV, ID_KK128, false);        // Vs dKV^T
                umma::gemm_mm<tc::PT, tc::PT, 64>(tbase + tcr::TR_KVA, aK, aVs, ID_MM64, false);              // first chunk of the pair
                umma::gemm_mm<tc::PT, tc::PT, 64>(tbase + tcr::TR_KVB, aK + 64 * umma::ROW_BYTES, aVs + 64 * umma::ROW_BYTES, ID_MM64, false);
                umma::commit(barB1);
            }
            __syncwarp();
            umma::fence_before_sync();
            bar_work();                              // barrier 2: P is written
            umma::fence_after_sync();
            if (lane == 0) {
                umma::mbar_wait(full_vd, it & 1, abort_flag);
                umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase + tcr::TR_DVA, aP, aDO, ID_MM64, false);          // P^T do
                int slot = 0;
#pragma unroll
                for (int lv = 0; lv < MP; ++lv)
                    if ((pl >> lv) & 1) {
                        umma::gemm_mm<tc::PT, tc::PT, tc::PT>(tbase + (slot == 0 ? tcr::TR_DH0 : tcr::TR_DH1), aQ,
                                                              aDOs + slot * tc::V_BYTES, ID_MM64, false);       // q^T (do * scale)
                        ++slot;
                    }
                umma::commit(barB);
                umma::mbar_wait(barB, it & 1, abort_flag);
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(empty_qvd)) : "memory");
            }
            __syncwarp();
            umma::fence_before_sync();
            bar_work();                              // barrier 3
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
    RegisterSplit<56, 224>::acquire();
    const int rb = warp & 3;
    const int row = rb * 32 + lane;
    const int ch = warp >> 2;

    float g_n[4];
    constexpr int LAMR = (tc::PT * tc::MAX_L_TC) / 256;   // (every column: fetching only the NLAM columns read here made this kernel spill)
    uint32_t lam_r[LAMR];
    uint32_t lam_rc[LAMR];
    const int NC = L;
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
    // Decay tables of a pair from the g values in g_n, by one full warp: G (pair-wide inclusive cumulative sum),
    // Cf = exp(G[end of 32-block] - G[j]), Vf = exp(G[127] - G[j]).  Built ahead of the pair that reads them, so that
    // a pair starts without a barrier of its own.
    auto decay_tables = [&](float* tG) {
        float gq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) gq[i] = g_n[i];
        gq[1] += gq[0];
        gq[2] += gq[1];
        gq[3] += gq[2];
        float tot = gq[3];
#pragma unroll
        for (int d = 1; d < 16; d <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, tot, d);
            if ((lane & 15) >= d) tot += t;
        }
        const float gla = __shfl_sync(0xffffffffu, tot, 15);
        const float glb = __shfl_sync(0xffffffffu, tot, 31);
        const float glp = gla + glb;
        const float pbase = tot - gq[3] + (lane >= 16 ? gla : 0.f);
        const float gend = __shfl_sync(0xffffffffu, tot, (lane & ~7) + 7) + (lane >= 16 ? gla : 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float G = pbase + gq[i];
            tG[4 * lane + i] = G;
            tG[128 + 4 * lane + i] = fexp(gend - G);
            tG[256 + 4 * lane + i] = fexp(glp - G);
        }
    };
    constexpr int TABLE_WARP = 4;                    // lane quarter 0, column half 1: the warp with the most slack
    auto store_lam = [&]() {
#pragma unroll
        for (int i = 0; i < LAMR; ++i)
            if (lam_rc[i] != 0xffffffffu)
                sLam[(lam_rc[i] >> 8) * tc::LAM_LD + (lam_rc[i] & 255)] = __ushort_as_bfloat16((unsigned short)lam_r[i]);
    };
    fetch_small(npairs - 1);
    store_lam();
    if (warp == TABLE_WARP) {
        fetch_g(npairs - 1);
        decay_tables(sTab);
        if (npairs > 1) fetch_g(npairs - 2);
    }

    // adjoint states: thread = state row `row`, 32 columns; index MP = adjoint of the segment summary
    float RM[MP + 1][32];
#pragma unroll
    for (int lv = 0; lv <= MP; ++lv)
#pragma unroll
        for (int e = 0; e < 32; ++e) RM[lv][e] = 0.f;
    if (p.NS > 1 && r < p.NS - 1) {
        const float* dH = p.seg_dHf + (((long)b * p.H + h) * p.NS + r) * tc::KD * tc::VD + row * tc::VD + ch * 32;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 x = *reinterpret_cast<const float4*>(dH + c * 4);
            RM[MP][c * 4] = x.x; RM[MP][c * 4 + 1] = x.y; RM[MP][c * 4 + 2] = x.z; RM[MP][c * 4 + 3] = x.w;
        }
    }
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;

    for (int it = 0; it < npairs; ++it) {
#ifdef LLATTN_STAMPS
        int nstamp = 0;
        const int stamp_slot = (blockIdx.x == 300 && it == 2) ? (tid == 0 ? 0 : (tid == 200 ? 1 : (tid == 96 ? 2 : -1))) : -1;
#endif
        STAMPR();   // 0 top
        const int pl = npairs - 1 - it;
        const long t0 = (long)(r * SEGP + pl) * tc::PT;
        const float* sGp = sTab + (it & 1) * 384;    // tables of this pair (written while the previous one ran)
        const float* sCf = sGp + 128;
        const float* sVf = sGp + 256;
        if (it + 1 < npairs) fetch_small(pl - 1);
        STAMPR();   // 1 small fetches issued
        const float Gi = sGp[row];
        const float glp = sGp[tc::PT - 1];
        float lam[NLAM];
#pragma unroll
        for (int i = 0; i < NLAM; ++i) lam[i] = (i < L) ? __bfloat162float(sLam[row * tc::LAM_LD + i]) : 0.f;

        // ---- adjoint of the pair summary: segment adjoint + pair levels whose bit is clear -> bf16 tile
        {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                float x0 = RM[MP][e], x1 = RM[MP][e + 1];
#pragma unroll
                for (int lv = 0; lv < MP; ++lv)
                    if (!((pl >> lv) & 1)) {
                        x0 += RM[lv][e];
                        x1 += RM[lv][e + 1];
                    }
                pk[e >> 1] = pack_bf16(x0, x1);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(sDKV + umma::tile_offset(row, ch * 32 + c * 8, tc::KD)) =
                    make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
        }
        STAMPR();   // 2 dKV tile written
        umma::mbar_wait(full_vd, it & 1, abort_flag);
        if (it >= 1) umma::mbar_wait(stage_free, (it - 1) & 1, abort_flag);   // P / scaled-do space was the dk staging area
        // ---- Vs and the scaled copies of do for the reader insertions
        {
#pragma unroll
            for (int i = tid; i < tc::PT * (tc::VD / 8); i += 256) {
                const int j = i / (tc::VD / 8), c = (i % (tc::VD / 8)) * 8;
                const float sc = sVf[j];
                const uint32_t off = umma::tile_offset(j, c, tc::PT);
                uint4 x = *reinterpret_cast<const uint4*>(sV + off);
                uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v2 = *reinterpret_cast<__nv_bfloat162*>(&xw[e]);
                    xw[e] = pack_bf16(__bfloat162float(v2.x) * sc, __bfloat162float(v2.y) * sc);
                }
                *reinterpret_cast<uint4*>(sVs + off) = x;
            }
            uint4 dox[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) dox[c] = *reinterpret_cast<const uint4*>(sDO + umma::tile_offset(row, ch * 32 + c * 8, tc::PT));
            int slot = 0;
#pragma unroll
            for (int lv = 0; lv < MP; ++lv)
                if ((pl >> lv) & 1) {
                    const float rs = lam[8 + lv] * fexp(Gi);
                    unsigned char* dst = sDOs + slot * tc::V_BYTES;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t* xw = reinterpret_cast<const uint32_t*>(&dox[c]);
                        uint32_t outw[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[e]);
                            outw[e] = pack_bf16(__bfloat162float(v2.x) * rs, __bfloat162float(v2.y) * rs);
                        }
                        *reinterpret_cast<uint4*>(dst + umma::tile_offset(row, ch * 32 + c * 8, tc::PT)) =
                            make_uint4(outw[0], outw[1], outw[2], outw[3]);
                    }
                    ++slot;
                }
        }
        STAMPR();   // 3 Vs / scaled do written
        umma::fence_async_smem();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(early_ready)) : "memory");
        // ---- S -> P (bf16 tile)
        umma::mbar_wait(barA, it & 1, abort_flag);
        umma::fence_after_sync();
        STAMPR();   // 4 S complete
        // blocks above the diagonal: zeros
#pragma unroll 1
        for (int jb = rb + 1; jb < 4; ++jb) {
            const int j0 = jb * 32 + ch * 16;
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(sP + umma::tile_offset(row, j0 + c * 8, tc::PT)) = make_uint4(0u, 0u, 0u, 0u);
        }
        // blocks below the diagonal (run-time loop: one copy of the body keeps the loop inside the instruction cache)
#pragma unroll 1
        for (int jb = 0; jb < rb; ++jb) {
            const int j0 = jb * 32 + ch * 16;
            uint32_t packed[8];
            float s[16];
            umma::tmem_ld16(umma::tmem_addr(tbase + tcr::TR_S, warp, j0), s);
            // one level per block, decay factorised through the block end
            const float lm = ((rb ^ jb) == 1) ? lam[6] : lam[7];
            const float rf = lm * fexp(Gi - sGp[jb * 32 + 31]);
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
                const float4 cf = *reinterpret_cast<const float4*>(sCf + j0 + e);
                packed[e >> 1] = pack_bf16(s[e] * rf * cf.x, s[e + 1] * rf * cf.y);
                packed[(e >> 1) + 1] = pack_bf16(s[e + 2] * rf * cf.z, s[e + 3] * rf * cf.w);
            }
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(sP + umma::tile_offset(row, j0 + c * 8, tc::PT)) =
                    make_uint4(packed[c * 4], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
        }
        // diagonal block: levels 0..5, causal mask folded into the exponent
        {
            const int j0 = rb * 32 + ch * 16;
            uint32_t packed[8];
            float s[16];
            umma::tmem_ld16(umma::tmem_addr(tbase + tcr::TR_S, warp, j0), s);
            const int li = lane;
#pragma unroll
            for (int e = 0; e < 16; e += 4) {
                const float4 gj = *reinterpret_cast<const float4*>(sGp + j0 + e);
                const float gjv[4] = {gj.x, gj.y, gj.z, gj.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int jj = ch * 16 + e + u;
                    const int x = li ^ jj;
                    float lm = lam[0];
                    lm = (x >= 1) ? lam[1] : lm;
                    lm = (x >= 2) ? lam[2] : lm;
                    lm = (x >= 4) ? lam[3] : lm;
                    lm = (x >= 8) ? lam[4] : lm;
                    lm = (x >= 16) ? lam[5] : lm;
                    const float d = (jj <= li) ? (Gi - gjv[u]) : -INFINITY;
                    s[e + u] = s[e + u] * fexp(d) * lm;
                }
                packed[e >> 1] = pack_bf16(s[e], s[e + 1]);
                packed[(e >> 1) + 1] = pack_bf16(s[e + 2], s[e + 3]);
            }
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(sP + umma::tile_offset(row, j0 + c * 8, tc::PT)) =
                    make_uint4(packed[c * 4], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
        }
        STAMPR();   // 5 P written
        if (warp == TABLE_WARP && it + 1 < npairs) {
            decay_tables(sTab + ((it + 1) & 1) * 384);
            if (it + 2 < npairs) fetch_g(pl - 2);
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();                                  // barrier 2
        umma::fence_after_sync();

        // ---- first the results that do not depend on P (they complete while P^T do and the reader insertions run)
        umma::mbar_wait(barB1, it & 1, abort_flag);
        umma::fence_after_sync();
        STAMPR();   // 6 early part of batch B complete
        // contributor totals Y = <KV of each chunk of the pair, adjoint state>, then the decay / reset of the adjoint states
        const float dec = fexp(glp);
        {
            float kva[32], kvb[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tcr::TR_KVA, warp, ch * 32), kva);
            umma::tmem_ld32(umma::tmem_addr(tbase + tcr::TR_KVB, warp, ch * 32), kvb);
#pragma unroll
            for (int lv = 0; lv <= MP; ++lv) {
                float ya = 0.f, yb = 0.f;
                if (lv == MP || !((pl >> lv) & 1)) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        ya += kva[e] * RM[lv][e];
                        yb += kvb[e] * RM[lv][e];
                    }
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) {
                    ya += __shfl_xor_sync(0xffffffffu, ya, d);
                    yb += __shfl_xor_sync(0xffffffffu, yb, d);
                }
                if (lane == 0) {
                    sMisc[256 + warp * 8 + lv * 2] = ya;
                    sMisc[256 + warp * 8 + lv * 2 + 1] = yb;
                }
            }
#pragma unroll
            for (int lv = 0; lv <= MP; ++lv) {
                const bool reset = (lv < MP) && ((pl & ((2 << lv) - 1)) == 0);
                const float f = reset ? 0.f : dec;
#pragma unroll
                for (int e = 0; e < 32; ++e) RM[lv][e] *= f;
            }
        }
        // level part of dk: the row sums k_j . dk_j (the tile itself is staged below, once its staging area is free)
        float wk_part = 0.f;
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tcr::TR_DK, warp, ch * 64 + hb * 32), t);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint4 kx = *reinterpret_cast<const uint4*>(sK + umma::tile_offset(row, ch * 64 + hb * 32 + c * 8, tc::PT));
                const uint32_t* xw = reinterpret_cast<const uint32_t*>(&kx);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[e]);
                    wk_part += __bfloat162float(v2.x) * t[c * 8 + e * 2] + __bfloat162float(v2.y) * t[c * 8 + e * 2 + 1];
                }
            }
        }
        sMisc[ch * 128 + row] = wk_part;
        // the k tile has no reader left (its products completed with barB1): released here, not at the end of the pair, so that
        // the next pair's k is in flight while dv, the dk staging and the state updates run.  The store of wk_part above needs
        // every k word this thread loaded, so the loads have returned before the arrive is issued.
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(empty_k)) : "memory");
        STAMPR();   // 7 Y, decay, k row sums
        // ---- then what needs the whole batch: P (staging area of dk) and the scaled do are free, dv and the insertions are there
        umma::mbar_wait(barB, it & 1, abort_flag);
        umma::fence_after_sync();
        // dv = P^T do + decay_j (k dKV) : stage bf16 rows, coalesced copy-out
        {
            float ta[32], tb[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tcr::TR_DVA, warp, ch * 32), ta);
            umma::tmem_ld32(umma::tmem_addr(tbase + tcr::TR_DVB, warp, ch * 32), tb);
            const float sc = sVf[row];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 x;
                uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    xw[e] = pack_bf16(ta[c * 8 + e * 2] + sc * tb[c * 8 + e * 2], ta[c * 8 + e * 2 + 1] + sc * tb[c * 8 + e * 2 + 1]);
                *reinterpret_cast<uint4*>(sVs + umma::tile_offset(row, ch * 32 + c * 8, tc::PT)) = x;   // Vs is free: second batch done
            }
        }
        // dk tile -> fp32 staging (P / scaled-do space)
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
            float t[32];
            umma::tmem_ld32(umma::tmem_addr(tbase + tcr::TR_DK, warp, ch * 64 + hb * 32), t);
            unsigned char* box = sStage + (ch * 2 + hb) * 16384;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<float4*>(box + box_offset(row, c * 4)) = make_float4(t[c * 4], t[c * 4 + 1], t[c * 4 + 2], t[c * 4 + 3]);
        }
        STAMPR();   // 8 dv, dk staged
        // reader insertions into the adjoint states
        {
            int slot = 0;
#pragma unroll
            for (int lv = 0; lv < MP; ++lv) {
                if ((pl >> lv) & 1) {
                    float t[32];
                    umma::tmem_ld32(umma::tmem_addr(tbase + (slot == 0 ? tcr::TR_DH0 : tcr::TR_DH1), warp, ch * 32), t);
#pragma unroll
                    for (int e = 0; e < 32; ++e) RM[lv][e] += t[e];
                    ++slot;
                }
            }
        }
        STAMPR();   // 9 states updated
        umma::fence_async_smem();
        bar_compute();
        if (tid == 0) {
            // every compute thread has staged its part of dk
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(dk_ready)) : "memory");
        }
        {
            bf16* gdv = p.dv + (((long)b * p.T + t0) * p.H + h) * tc::VD;
#pragma unroll
            for (int i = tid; i < tc::PT * 8; i += 256) {
                const int rr = i >> 3, c = (i & 7) * 8;
                *reinterpret_cast<uint4*>(gdv + (long)rr * p.H * tc::VD + c) =
                    *reinterpret_cast<const uint4*>(sVs + umma::tile_offset(rr, c, tc::PT));
            }
        }
        if (ch == 0) red_add_f32(p.wq + ((long)b * p.T + t0 + row) * p.H + h, -(sMisc[row] + sMisc[128 + row]));
        if (tid < 2 * (MP + 1)) {
            // Y of chunk (2*pair + cpart): pair level lv -> chunk level lv + 1 ; index MP -> combined high levels (slot MLOW)
            const int lv = tid >> 1, cpart = tid & 1;
            float y = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) y += sMisc[256 + w * 8 + lv * 2 + cpart];
            const long cidx = ((long)b * p.H + h) * p.NT + (r * SEGP + pl) * 2 + cpart;
            p.Yc[cidx * (MLOW + 1) + (lv == MP ? MLOW : lv + 1)] = y;
        }
        STAMPR();   // 10 dv out
        if (it + 1 < npairs) store_lam();
        umma::fence_async_smem();
        umma::fence_before_sync();
        bar_work();                                  // barrier 3
        STAMPR();   // 11 after barrier 3
        umma::fence_after_sync();
        if (*abort_flag) break;
    }
    umma::fence_before_sync();
    bar_work();
}

int mamba2_bwd2_tc_launch(const Mamba2Params& p_in, cudaStream_t stream) {
    Mamba2Params p = p_in;
    int rc;
    const long BT = (long)p.B * p.T;
    if ((rc = tma::make_panel_map(&p.tm_q, p.q, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_k, p.k, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_v, p.v, BT, p.H, p.V, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_do, p.d_o, BT, p.H, p.V, tc::PT)) != 0) return rc;
    if ((rc = tma::make_f32_box_map(&p.tm_dk, p.dk_acc, BT, p.G, p.K, tc::PT)) != 0) return rc;
    auto kern = m2_bwd_revorder_tc_kernel<M2_MLOW>;
    const size_t sm = Bwd2TcSmem<M2_MLOW>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    kern<<<p.B * p.H * p.NS, tc::NTHREADS, sm, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

int mamba2_bwd1_tc_launch(const Mamba2Params& p_in, cudaStream_t stream) {
    Mamba2Params p = p_in;
    int rc;
    const long BT = (long)p.B * p.T;
    if ((rc = tma::make_panel_map(&p.tm_q, p.q, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_k, p.k, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_v, p.v, BT, p.H, p.V, tc::PT)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_do, p.d_o, BT, p.H, p.V, tc::PT)) != 0) return rc;
    if ((rc = tma::make_f32_box_map(&p.tm_dq, p.dq_acc, BT, p.G, p.K, tc::PT)) != 0) return rc;
    if ((rc = tma::make_f32_box_map(&p.tm_dk, p.dk_acc, BT, p.G, p.K, tc::PT)) != 0) return rc;
    auto kern = m2_bwd_fwdorder_tc_kernel<M2_MLOW>;
    const size_t sm = Bwd1TcSmem<M2_MLOW>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    const int nitems = p.B * p.H * p.NS;
    kern<<<nitems < sms ? nitems : sms, tc::NTHREADS, sm, stream>>>(p); LLATTN_LAUNCHED();      // persistent: one CTA per SM
    return (int)cudaGetLastError();
}

}  // namespace llattn

#ifdef LLATTN_STAMPS
extern "C" int llattn_debug_read_stamps_bwd(long long* host_dst) {
    return (int)cudaMemcpyFromSymbol(host_dst, llattn::g_stamps, sizeof(long long) * 3 * 32);
}
#endif
