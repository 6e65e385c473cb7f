// Log-linear Gated DeltaNet: the sequential scans over chunks on tcgen05 / TMEM / TMA (K = 128).
//
// Same mathematics as gdn_scan_kernel (gdn_fwd.cu) and gdn_scan_bwd_kernel (gdn_bwd.cu); reference being
// replaced: hattention/chunkwise_hgdn.py:718-788 with fla_future/chunk_delta_h.py:34-186 (forward state
// recurrence per level) and :206-368 (its adjoint).  One CTA per (batch, head, 32-column slice of V) walks the
// chunks in order.  The transition of a level state is used in the form
//     H' = H + Wd H  (+ kd^T u for the level that receives the chunk's own writes),
//     Wd = (exp(gl) - 1) I - kd^T wd,
// with the K x K matrix Wd of every chunk prepared by the chunk-parallel kernel.  The fp32 master of every level
// state lives in TENSOR MEMORY and the transition is one accumulating tcgen05.mma chain onto it, so the dependent
// chain of a chunk is: bf16 copies (shared memory) --MMA--> masters --element-wise warps--> new bf16 copies.  The
// element-wise step only converts (and, where a carry merges levels, adds a few slots); its loops over levels
// are run-time loops over tensor-memory addresses (a version with the masters in registers, every level loop
// unrolled and one chain of products per level took twice as long per chunk).
// The reader products qd H_lv (output) use the same bf16 copies; they are issued behind the transition products
// and consumed one chunk later.  The bf16 copies are kept transposed ([V column][K]) so that they are K-major B
// operands whose rows continue from level to level: a range of levels is read by ONE chain with N = 32 x (number
// of levels) (an instruction costs the same for N = 32 as for N = 128; slots of levels inside the range that are
// not live receive products of stale copies and are never read).
#include "tc_common.cuh"
#include "llattn_gdn.h"

namespace llattn {

namespace gtc {
constexpr int KD = 128, VS = GDN_VS, MAXLEV = GDN_MAXLEV;
constexpr int NTHREADS = 384, MMA_WARP = 8;
constexpr uint32_t QD_BYTES = CH * KD * 2;               // qd / kd tile: two panels of 64 rows
constexpr uint32_t WK_BYTES = KD * KD * 2;               // Wd: two panels of 128 rows
constexpr uint32_t ST_ROWS = MAXLEV * VS;                // rows of the transposed state tile: level * 32 + column
constexpr uint32_t ST_BYTES = ST_ROWS * KD * 2;          // two panels of 256 rows
constexpr uint32_t LV_BYTES = VS * 128;                  // one level's rows inside a panel
constexpr int TM_M = 0, TM_R = 256, TM_COLS = 512;       // masters / reader products: slot of level lv at lv * 32
}  // namespace gtc

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(bar)) : "memory");
}

// What a thread of the element-wise warps needs to write its 16 values (row k or token t of a transposed tile,
// columns ch * 16 ..) as bf16 into a [column][row] tile: two neighbouring lanes hold rows r, r + 1; they exchange
// halves so that each writes 32-bit words (rows r, r + 1 of one column): the even lane the even columns, the odd
// lane the odd ones.  The address pieces that do not change are computed once.
struct TransposedStore {
    uint32_t base;        // byte offset of (column ch*16 + parity, row & ~1) inside a 32-row block of the first panel
    uint32_t xo[4];       // swizzled 16-byte chunk position for columns 2i + parity (mod 8)
    uint32_t sel;
    __device__ __forceinline__ void init(int r, int ch, int lane, uint32_t panel_bytes) {
        const int par = lane & 1;
        base = (uint32_t)((r >> 6) * panel_bytes + (ch * 16 + par) * 128 + (r & 6) * 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) xo[i] = (uint32_t)((((r & 63) >> 3) ^ ((2 * i + par) & 7)) << 4);
        sel = par ? 0x3276u : 0x5410u;
    }
    // mine[m] = bf16 pair (columns 2m, 2m + 1) of this thread's row; block = shared-memory address of the 32-row block
    __device__ __forceinline__ void store(uint32_t block, const uint32_t (&mine)[8]) const {
        uint32_t word[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) word[m] = __byte_perm(mine[m], __shfl_xor_sync(0xffffffffu, mine[m], 1), sel);
#pragma unroll
        for (int m = 0; m < 8; ++m)
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(block + base + (uint32_t)(m * 256) + xo[m & 3]), "r"(word[m]) : "memory");
    }
};

__device__ __forceinline__ float lambda_of_level(uint64_t l0123, uint64_t l4567, int lv) {
    const uint64_t w = (lv < 4) ? l0123 : l4567;
    return __uint_as_float((uint32_t)((w >> ((lv & 3) * 16)) & 0xFFFFull) << 16);
}

struct ScanTcSmem {
    static constexpr uint32_t STAGE = 2 * gtc::QD_BYTES + gtc::WK_BYTES;        // qd | kd | Wd
    static constexpr uint32_t stage_off = 0;                                    // [2]
    static constexpr uint32_t st_off = stage_off + 2 * STAGE;
    static constexpr uint32_t ut_off = st_off + gtc::ST_BYTES;                  // [2] u^T: one panel of 32 rows ([column][token])
    static constexpr uint32_t bar_off = ut_off + 2 * gtc::LV_BYTES;
    static constexpr uint32_t total = bar_off + 128 + 1024;                     // + slack for the 1024-byte alignment
};

// SAVE also writes, for every chunk, the bf16 level states that the chunk reads:
// hs[((b*H + h)*(V/64) + vs/2)*NT + c][level][K][64] (the backward's recomputation, or a forward whose caller keeps
// the workspace for the backward; V a multiple of 64); OUT = false skips the output (recomputation only).
template <bool SAVE, bool OUT>
__global__ void __launch_bounds__(gtc::NTHREADS, 1) gdn_scan_tc_kernel(const __grid_constant__ GdnParams p) {
    using SM = ScanTcSmem;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sStage = smem + SM::stage_off;
    unsigned char* sSt = smem + SM::st_off;
    unsigned char* sUT = smem + SM::ut_off;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* full = bars + 0;       // [2] tiles of a chunk landed
    uint64_t* empty = bars + 2;      // [2] every product of the chunk that used the stage is complete
    uint64_t* barT = bars + 4;       // transition products of a chunk complete
    uint64_t* barR = bars + 5;       // reader products of a chunk complete
    uint64_t* barS = bars + 6;       // bf16 state copies of the next chunk written (256 arrivals)
    // One barrier per u^T buffer: the staging of chunk c + 1 may finish before the MMA thread has looked at the
    // barrier of chunk c, and a parity wait cannot tell a phase from the one two completions later.
    uint64_t* barU = bars + 7;       // [2] u^T of a chunk written (128 arrivals: warps of lane quarters 2, 3)
    uint64_t* barO = bars + 9;       // reader products of a chunk consumed (128 arrivals: lane quarters 0, 1)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 88);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 96);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nvs = p.V / gtc::VS;
    const int vs = blockIdx.x % nvs;
    const int h = (blockIdx.x / nvs) % p.H;
    const int b = blockIdx.x / (nvs * p.H);
    const int nlev = p.NLEV, NT = p.NT;
    const uint32_t lev_mask = (1u << nlev) - 1u;
    // level-state tiles for the backward are [K][64]: one tile per pair of 32-column slices, this CTA's slice in its half
    auto pair_tile = [&](int c, int lv) -> size_t { return ((((size_t)(blockIdx.x >> 1)) * NT + c) * nlev + lv) * (size_t)(gtc::KD * 64); };

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 6; ++i) umma::mbar_init(&bars[i], 1);
        umma::mbar_init(barS, 256);
        umma::mbar_init(&barU[0], 128);
        umma::mbar_init(&barU[1], 128);
        umma::mbar_init(barO, 128);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    if (warp >= gtc::MMA_WARP) {
        if (warp == gtc::MMA_WARP + 1) {
            if (lane == 0) {
                for (int c = 0; c < NT; ++c) {
                    const int st = c & 1;
                    if (c >= 2 && !umma::mbar_wait(&empty[st], ((c >> 1) - 1) & 1, abort_flag)) break;
                    const int row0 = b * p.T + c * CH;
                    unsigned char* qd = sStage + st * SM::STAGE;
                    unsigned char* kd = qd + gtc::QD_BYTES;
                    unsigned char* wk = kd + gtc::QD_BYTES;
                    tma::expect_tx(&full[st], (OUT ? gtc::QD_BYTES : 0u) + gtc::QD_BYTES + gtc::WK_BYTES);
                    if (OUT) {
                        tma::load_panel(qd, &p.tm_qd, 0, h, row0, &full[st]);
                        tma::load_panel(qd + CH * 128, &p.tm_qd, 64, h, row0, &full[st]);
                    }
                    tma::load_panel(kd, &p.tm_kd, 0, h, row0, &full[st]);
                    tma::load_panel(kd + CH * 128, &p.tm_kd, 64, h, row0, &full[st]);
                    const int wrow0 = (b * NT + c) * gtc::KD;
                    tma::load_panel(wk, &p.tm_wk, 0, h, wrow0, &full[st]);
                    tma::load_panel(wk + gtc::KD * 128, &p.tm_wk, 64, h, wrow0, &full[st]);
                }
            }
            return;
        }
        if (warp > gtc::MMA_WARP) return;
        umma::tmem_alloc(tmem_slot, gtc::TM_COLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        const uint32_t aSt = umma::smem_addr(sSt);
        constexpr uint32_t ID_MK32 = umma::idesc_bf16(128, gtc::VS, true, false);
        bool ok = true;
        for (int c = 0; c < NT && ok; ++c) {
            const int st = c & 1;
            const uint32_t aQd = umma::smem_addr(sStage + st * SM::STAGE);
            const uint32_t aKd = aQd + gtc::QD_BYTES, aWk = aKd + gtc::QD_BYTES;
            const uint32_t aUT = umma::smem_addr(sUT + st * gtc::LV_BYTES);
            const uint32_t live = (uint32_t)c & lev_mask;
            const bool trans = (c + 1 < NT);
            const int jc = __ffs(~c) - 1;
#ifdef LLATTN_STAMPS
            int nstamp = 0;
            const int stamp_slot = (blockIdx.x == 5 && c == 37 && lane == 0) ? 2 : -1;
#endif
            if (lane == 0) {
                STAMP();
                ok = umma::mbar_wait(&full[st], (c >> 1) & 1, abort_flag);
                if (ok && c > 0) ok = umma::mbar_wait(barS, (c - 1) & 1, abort_flag);
                STAMP();
                if (ok && trans) ok = umma::mbar_wait(&barU[st], (c >> 1) & 1, abort_flag);
                if (ok) {
                    umma::fence_after_sync();
                    if (trans) {
                        // the level that receives this chunk's writes starts from kd^T u (its slot held a dead level); the
                        // levels below the carry (all live; the element-wise warps add them into that level afterwards) and the
                        // live levels above it advance in place: master += Wd H_lv
                        umma::gemm_mk<CH, gtc::VS, CH>(tbase + gtc::TM_M + jc * gtc::VS, aKd, aUT, ID_MK32, false);
                        if (jc > 0)
                            umma::gemm_kk<gtc::KD, gtc::ST_ROWS, gtc::KD>(tbase + gtc::TM_M, aWk, aSt, umma::idesc_bf16(128, gtc::VS * jc, false, false), true);
                        const uint32_t above = live & ~((2u << jc) - 1u);
                        if (above) {
                            const int lo = __ffs(above) - 1, hi = 31 - __clz(above);
                            umma::gemm_kk<gtc::KD, gtc::ST_ROWS, gtc::KD>(tbase + gtc::TM_M + lo * gtc::VS, aWk, aSt + lo * gtc::LV_BYTES,
                                                                          umma::idesc_bf16(128, gtc::VS * (hi - lo + 1), false, false), true);
                        }
                        umma::commit(barT);
                    }
                    STAMP();
                    if (OUT) {
                        if (c > 0) ok = umma::mbar_wait(barO, (c - 1) & 1, abort_flag);
                        STAMP();
                        if (ok && live) {
                            umma::fence_after_sync();
                            // readers: qd H_lv in rows 0..63 (rows 64..127 of the M = 128 product are not used), one chain from
                            // the lowest to the highest live level
                            const int lo = __ffs(live) - 1, hi = 31 - __clz(live);
                            umma::gemm_kk<CH, gtc::ST_ROWS, gtc::KD>(tbase + gtc::TM_R + lo * gtc::VS, aQd, aSt + lo * gtc::LV_BYTES,
                                                                     umma::idesc_bf16(128, gtc::VS * (hi - lo + 1), false, false), false);
                            umma::commit(barR);
                        }
                    }
                    if (ok) umma::commit(&empty[st]);
                    STAMP();
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (lane == 0 && ok) {
            // every product has completed before tensor memory is released
            const int last = NT - 1;
            umma::mbar_wait(&empty[last & 1], (last >> 1) & 1, abort_flag);
        }
        __syncwarp();
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();
        umma::tmem_dealloc(tbase, gtc::TM_COLS);
        return;
    }

    // ================= warps 0..7 =================

    const int rb = warp & 3, ch = warp >> 2;
    const int row = rb * 32 + lane;            // tensor-memory lane: token (reader products), state row k (masters)
    const bool qrow = rb < 2;                  // warp-uniform: lane quarters 0, 1 write the output, 2, 3 stage u^T
    const int tok = row & 63;
    const int col0 = vs * gtc::VS + ch * 16;   // this thread's 16 V columns
    TransposedStore ts_state, ts_tok;
    ts_state.init(row, ch, lane, gtc::ST_ROWS * 128);
    ts_tok.init(tok, ch, lane, 0);
    const uint32_t aSt = umma::smem_addr(sSt), aUT = umma::smem_addr(sUT);

    // Per-chunk inputs are fetched ahead of their use: for the output warps the lambda row and 16 columns of the
    // intra-chunk output of the chunk whose reader products are in flight; for the others 16 columns of u two
    // chunks ahead (staged transposed one chunk ahead).
    uint4 in_n[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    unsigned short lam_raw[gtc::MAXLEV] = {0, 0, 0, 0, 0, 0, 0, 0};   // lambda of levels 0..7 (bf16 bits)
    auto token_row = [&](int c) -> long { return ((long)b * p.T + (long)c * CH + tok) * p.H + h; };
    auto fetch_u = [&](int c) {
        const uint4* src = reinterpret_cast<const uint4*>(p.u + token_row(c) * p.V + col0);
        in_n[0] = src[0];
        in_n[1] = src[1];
    };
    auto fetch_o = [&](int c) {
        const long r = token_row(c);
        const uint4* src = reinterpret_cast<const uint4*>(p.o + r * p.V + col0);
        in_n[0] = src[0];
        in_n[1] = src[1];
        // the lambda row is only requested here; it is packed when it is used, one iteration later (packing at once would
        // wait for the loads)
        const unsigned short* lp = reinterpret_cast<const unsigned short*>(p.l + r * p.L + INTRA_LEVELS);
#pragma unroll
        for (int i = 0; i < gtc::MAXLEV; ++i) lam_raw[i] = (i < nlev) ? lp[i] : (unsigned short)0;
    };
    // 16 columns of u of one token into the transposed tile [column][token]
    auto stage_ut = [&](int buf) {
        const uint32_t* xin = reinterpret_cast<const uint32_t*>(in_n);
        uint32_t mine[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) mine[j] = xin[j];
        ts_tok.store(aUT + buf * gtc::LV_BYTES, mine);
        umma::fence_async_smem();
        mbar_arrive(&barU[buf]);
    };

    if (!qrow) {
        fetch_u(0);
        if (NT > 1) stage_ut(0);
        if (NT > 1) fetch_u(1);
    }
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;
    const uint32_t tR = umma::tmem_addr(tbase + gtc::TM_R, warp, ch * 16), tM = umma::tmem_addr(tbase + gtc::TM_M, warp, ch * 16);
    uint32_t phT = 0, phR = 0;
    bool alive = true;

    // output rows of chunk c: lambda-weighted reader products plus the intra-chunk part
    auto write_output = [&](int c) {
        const uint32_t live = (uint32_t)c & lev_mask;
        uint64_t lam_a = 0, lam_b = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lam_a |= (uint64_t)lam_raw[i] << (16 * i);
            lam_b |= (uint64_t)lam_raw[4 + i] << (16 * i);
        }
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
        uint32_t m = live;
#pragma unroll 1
        while (m) {
            const int l0 = __ffs(m) - 1;
            m &= m - 1;
            const bool two = (m != 0);
            const int l1 = two ? __ffs(m) - 1 : l0;
            m &= m - 1;
            float r0[16], r1[16];
            umma::tmem_ld16x2(tR + l0 * gtc::VS, r0, tR + l1 * gtc::VS, r1);
            const float w0 = lambda_of_level(lam_a, lam_b, l0), w1 = two ? lambda_of_level(lam_a, lam_b, l1) : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] += w0 * r0[j] + w1 * r1[j];
        }
        umma::fence_before_sync();
        mbar_arrive(barO);
        const uint32_t* xin = reinterpret_cast<const uint32_t*>(in_n);
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xin[j]);
            w[j] = pack_bf16(__bfloat162float(v2.x) + acc[2 * j], __bfloat162float(v2.y) + acc[2 * j + 1]);
        }
        st_global_32B(p.o + token_row(c) * p.V + col0, w);
    };
    // bf16 copy of one level's master for the next chunk (and, with SAVE, for the backward)
    auto publish_level = [&](int lv, const float (&v)[16], int c_next) {
        uint32_t mine[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) mine[j] = pack_bf16(v[2 * j], v[2 * j + 1]);
        if (SAVE) {
            st_global_32B(p.hs + pair_tile(c_next, lv) + (size_t)row * 64 + (vs & 1) * gtc::VS + ch * 16, mine);
        }
        ts_state.store(aSt + lv * gtc::LV_BYTES, mine);
    };

    for (int c = 0; c < NT; ++c) {
        const uint32_t live = (uint32_t)c & lev_mask;
        const bool trans = (c + 1 < NT);
        const int jc = __ffs(~c) - 1;
#ifdef LLATTN_STAMPS
        int nstamp = 0;
        const int stamp_slot = (blockIdx.x == 5 && c == 37) ? (tid == 0 ? 0 : (tid == 64 ? 1 : -1)) : -1;
#endif
        STAMP();
        // ---- off the chain, while the products of this chunk run
        if (qrow) {
            if (OUT) {
                if (c > 0) write_output(c - 1);                      // its reader products were waited for at the end of the last iteration
                fetch_o(c);                                          // consumed in the next iteration
            }
        } else if (c + 2 < NT) {
            stage_ut((c + 1) & 1);                                   // u of chunk c + 1 (needed only if that chunk has a transition)
            fetch_u(c + 2);
        }
        if (OUT && c == NT - 1 && p.final_states != nullptr) {
            // prefill hand-off: the level states every token of the last chunk starts from.  Level 7 + lv holds the block
            // of 2^lv chunks for each set bit lv of c (the binary-indexed tree as it stands before this chunk); the
            // caller steps the last chunk's tokens through the decode kernel, which fills levels 0..6.
            float* dst = p.final_states + (((long)b * p.H + h) * gtc::KD + row) * (long)p.V * p.L;
#pragma unroll 1
            for (uint32_t m = live; m; m &= m - 1) {
                const int lv = __ffs(m) - 1;
                float v[16];
                umma::tmem_ld16(tM + lv * gtc::VS, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) dst[(long)(col0 + j) * p.L + INTRA_LEVELS + lv] = v[j];
            }
        }
        STAMP();
        if (!trans) break;

        // ---- the chain: transition products -> masters -> bf16 copies for the next chunk
        {
            const bool ok = umma::mbar_wait(barT, phT, abort_flag);
            phT ^= 1;
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        }
        umma::fence_after_sync();
        STAMP();
        if (jc > 0) {
            // the levels below the carry merge into the carry level
            float acc[16];
            umma::tmem_ld16(tM + jc * gtc::VS, acc);
#pragma unroll 1
            for (int lv = 0; lv < jc; ++lv) {
                float t[16];
                umma::tmem_ld16(tM + lv * gtc::VS, t);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] += t[j];
            }
            umma::tmem_st16(tM + jc * gtc::VS, acc);
            umma::tmem_wait_st();
        }
        STAMP();
        // the reader products of this chunk (issued behind the transition products) still read the bf16 copies:
        // they must be complete before the copies are replaced
        if (OUT && live) {
            const bool ok = umma::mbar_wait(barR, phR, abort_flag);
            phR ^= 1;
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
            umma::fence_after_sync();
        }
        STAMP();
        {
            uint32_t m = (uint32_t)(c + 1) & lev_mask;               // the carry level and the live levels above it
#pragma unroll 1
            while (m) {
                const int l0 = __ffs(m) - 1;
                m &= m - 1;
                const bool two = (m != 0);
                const int l1 = two ? __ffs(m) - 1 : l0;
                m &= m - 1;
                float v0[16], v1[16];
                umma::tmem_ld16x2(tM + l0 * gtc::VS, v0, tM + l1 * gtc::VS, v1);
                publish_level(l0, v0, c + 1);
                if (two) publish_level(l1, v1, c + 1);
            }
        }
        STAMP();
        umma::fence_async_smem();
        umma::fence_before_sync();
        mbar_arrive(barS);
        STAMP();
    }
    if (OUT && qrow && alive) {
        // reader products of the last chunk
        const uint32_t live = (uint32_t)(NT - 1) & lev_mask;
        bool ok = true;
        if (live) {
            ok = umma::mbar_wait(barR, phR, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            umma::fence_after_sync();
        }
        if (ok) write_output(NT - 1);
    }
    umma::fence_before_sync();
    bar_work();
}

// ------------------------------------------------------------------------------------------
// reverse scan: adjoints of the level states.  With Wd as above the adjoint recurrence of a state is
//     E (adjoint after chunk c)  ->  E + Wd^T E  (+ qd^T (lambda_lv * do) for the levels the chunk reads)
// Wd^T is the same shared-memory tile read MN-major, and the masters of the adjoints live in tensor memory like
// the forward's.  The reader terms do not depend on E: their operands (lambda_lv * do, transposed, one 32-row
// block per level) are staged one chunk ahead and their products are issued in the same batch, accumulating
// onto the masters.  d_u = kd E_jc is left to the chunk-parallel gradient kernel, which holds the same tiles.
// ------------------------------------------------------------------------------------------
struct ScanBwdTcSmem {
    static constexpr uint32_t STAGE = gtc::QD_BYTES + gtc::WK_BYTES;            // qd | Wd
    static constexpr uint32_t stage_off = 0;                                    // [2]
    static constexpr uint32_t e_off = stage_off + 2 * STAGE;                    // transposed adjoint copies
    static constexpr uint32_t dl_off = e_off + gtc::ST_BYTES;                   // [2] (lambda_lv * do)^T: [level * 32 + column][token]
    static constexpr uint32_t DL_BYTES = gtc::ST_ROWS * 128;
    static constexpr uint32_t bar_off = dl_off + 2 * DL_BYTES;
    static constexpr uint32_t total = bar_off + 128 + 1024;
};

__global__ void __launch_bounds__(gtc::NTHREADS, 1) gdn_scan_bwd_tc_kernel(const __grid_constant__ GdnParams p) {
    using SM = ScanBwdTcSmem;
    constexpr int TCOLS = 256;                 // one 32-column slot per level
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sStage = smem + SM::stage_off;
    unsigned char* sE = smem + SM::e_off;
    unsigned char* sDL = smem + SM::dl_off;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::bar_off);
    uint64_t* full = bars + 0;       // [2]
    uint64_t* empty = bars + 2;      // [2]
    uint64_t* barT = bars + 4;       // products of a chunk complete
    uint64_t* barS = bars + 5;       // bf16 adjoint copies of the next (earlier) chunk written (256 arrivals)
    uint64_t* barD = bars + 6;       // [2] (lambda * do)^T of a chunk staged (256 arrivals); one barrier per buffer, see barU above
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::bar_off + 64);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::bar_off + 72);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nvs = p.V / gtc::VS;
    const int vs = blockIdx.x % nvs;
    const int h = (blockIdx.x / nvs) % p.H;
    const int b = blockIdx.x / (nvs * p.H);
    const int nlev = p.NLEV, NT = p.NT;
    const uint32_t lev_mask = (1u << nlev) - 1u;
    auto pair_tile = [&](int c, int lv) -> size_t { return ((((size_t)(blockIdx.x >> 1)) * NT + c) * nlev + lv) * (size_t)(gtc::KD * 64); };

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 5; ++i) umma::mbar_init(&bars[i], 1);
        umma::mbar_init(barS, 256);
        umma::mbar_init(&barD[0], 256);
        umma::mbar_init(&barD[1], 256);
        umma::fence_mbar_init();
        *abort_flag = *p.err;
    }
    __syncthreads();
    if (*abort_flag) return;

    if (warp >= gtc::MMA_WARP) {
        if (warp == gtc::MMA_WARP + 1) {
            if (lane == 0) {
                for (int it = 0; it < NT - 1; ++it) {                      // chunk 0 reads no state: nothing to propagate there
                    const int c = NT - 1 - it, st = it & 1;
                    if (it >= 2 && !umma::mbar_wait(&empty[st], ((it >> 1) - 1) & 1, abort_flag)) break;
                    unsigned char* qd = sStage + st * SM::STAGE;
                    unsigned char* wk = qd + gtc::QD_BYTES;
                    const int row0 = b * p.T + c * CH, wrow0 = (b * NT + c) * gtc::KD;
                    tma::expect_tx(&full[st], SM::STAGE);
                    tma::load_panel(qd, &p.tm_qd, 0, h, row0, &full[st]);
                    tma::load_panel(qd + CH * 128, &p.tm_qd, 64, h, row0, &full[st]);
                    tma::load_panel(wk, &p.tm_wk, 0, h, wrow0, &full[st]);
                    tma::load_panel(wk + gtc::KD * 128, &p.tm_wk, 64, h, wrow0, &full[st]);
                }
            }
            return;
        }
        if (warp > gtc::MMA_WARP) return;
        umma::tmem_alloc(tmem_slot, TCOLS);
        umma::fence_before_sync();
        bar_work();
        umma::fence_after_sync();
        const uint32_t tbase = *tmem_slot;
        const uint32_t aE = umma::smem_addr(sE);
        bool ok = true;
        for (int it = 0; it < NT - 1 && ok; ++it) {
            const int c = NT - 1 - it, st = it & 1;
            const uint32_t aQd = umma::smem_addr(sStage + st * SM::STAGE), aWk = aQd + gtc::QD_BYTES;
            const uint32_t aDL = umma::smem_addr(sDL + st * SM::DL_BYTES);
            const uint32_t readers = (uint32_t)c & lev_mask;             // levels whose states this chunk reads (never empty for c >= 1)
            const bool trans = (c + 1 < NT);
            const uint32_t written = trans ? ((uint32_t)(c + 1) & lev_mask) : 0u;   // levels that hold a state after this chunk
            const int jc = __ffs(~c) - 1;
            if (lane == 0) {
                ok = umma::mbar_wait(&full[st], (it >> 1) & 1, abort_flag);
                if (ok && it > 0) ok = umma::mbar_wait(barS, (it - 1) & 1, abort_flag);
                if (ok) ok = umma::mbar_wait(&barD[st], (it >> 1) & 1, abort_flag);
                if (ok) {
                    umma::fence_after_sync();
                    // master += Wd^T E_lv for every level written by this chunk: ONE chain from the carry level (whose
                    // result is shared by all levels below it) to the highest such level
                    if (written) {
                        const int hi = 31 - __clz(written);
                        umma::gemm_mk<gtc::KD, gtc::ST_ROWS, gtc::KD>(tbase + jc * gtc::VS, aWk, aE + jc * gtc::LV_BYTES,
                                                                      umma::idesc_bf16(128, gtc::VS * (hi - jc + 1), true, false), true);
                    }
                    // qd^T (lambda_lv * do): below the carry into fresh slots (those levels held no state after this chunk),
                    // above it onto the masters
                    const uint32_t above = readers & ~((2u << jc) - 1u);
                    if (jc > 0)
                        umma::gemm_mk<CH, gtc::ST_ROWS, CH>(tbase, aQd, aDL, umma::idesc_bf16(128, gtc::VS * jc, true, false), false);
                    if (above) {
                        const int lo = __ffs(above) - 1, hi = 31 - __clz(above);
                        umma::gemm_mk<CH, gtc::ST_ROWS, CH>(tbase + lo * gtc::VS, aQd, aDL + lo * gtc::LV_BYTES,
                                                            umma::idesc_bf16(128, gtc::VS * (hi - lo + 1), true, false), trans);
                    }
                    umma::commit(barT);
                    umma::commit(&empty[st]);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (lane == 0 && ok && NT > 1) umma::mbar_wait(&empty[(NT - 2) & 1], ((NT - 2) >> 1) & 1, abort_flag);
        __syncwarp();
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();
        umma::tmem_dealloc(tbase, TCOLS);
        return;
    }

    // ================= warps 0..7 =================

    const int rb = warp & 3, ch = warp >> 2;
    const int row = rb * 32 + lane;            // state row k
    const int tok = row & 63;                  // token whose do / lambda row this thread stages
    const int lpar = rb >> 1;                  // ... for the live levels of this parity (in order of appearance)
    const int col0 = vs * gtc::VS + ch * 16;
    TransposedStore ts_state, ts_tok;
    ts_state.init(row, ch, lane, gtc::ST_ROWS * 128);
    ts_tok.init(tok, ch, lane, 0);
    const uint32_t aE = umma::smem_addr(sE), aDLbase = umma::smem_addr(sDL);

    uint4 do_n[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    unsigned short lam_raw[gtc::MAXLEV] = {0, 0, 0, 0, 0, 0, 0, 0};
    auto fetch_do = [&](int c) {
        const long r = ((long)b * p.T + (long)c * CH + tok) * p.H + h;
        const uint4* src = reinterpret_cast<const uint4*>(p.d_o + r * p.V + col0);
        do_n[0] = src[0];
        do_n[1] = src[1];
        const unsigned short* lp = reinterpret_cast<const unsigned short*>(p.l + r * p.L + INTRA_LEVELS);
#pragma unroll
        for (int i = 0; i < gtc::MAXLEV; ++i) lam_raw[i] = (i < nlev) ? lp[i] : (unsigned short)0;   // packed when used (see the forward kernel)
    };
    // (lambda_lv * do)^T of chunk c for every level the chunk reads; the two halves of the CTA take alternate levels
    auto stage_dl = [&](int c, int buf) {
        const uint32_t* xin = reinterpret_cast<const uint32_t*>(do_n);
        uint64_t lam_a = 0, lam_b = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            lam_a |= (uint64_t)lam_raw[i] << (16 * i);
            lam_b |= (uint64_t)lam_raw[4 + i] << (16 * i);
        }
        int seen = 0;
#pragma unroll 1
        for (uint32_t m = (uint32_t)c & lev_mask; m; m &= m - 1, ++seen) {
            if ((seen & 1) != lpar) continue;
            const int lv = __ffs(m) - 1;
            const float lm = lambda_of_level(lam_a, lam_b, lv);
            uint32_t mine[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xin[j]);
                mine[j] = pack_bf16(lm * __bfloat162float(v2.x), lm * __bfloat162float(v2.y));
            }
            // both lanes of a pair take the same levels (same lane quarter), so the exchange inside store() is uniform
            ts_tok.store(aDLbase + buf * SM::DL_BYTES + lv * gtc::LV_BYTES, mine);
        }
        umma::fence_async_smem();
        mbar_arrive(&barD[buf]);
    };

    fetch_do(NT - 1);
    if (NT > 1) stage_dl(NT - 1, 0);
    if (NT > 2) fetch_do(NT - 2);
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;
    const uint32_t tM = umma::tmem_addr(tbase, warp, ch * 16);
    uint32_t phT = 0;

    for (int it = 0; it < NT - 1; ++it) {
        const int c = NT - 1 - it;                          // c >= 1
        const bool trans = (c + 1 < NT);
        const int jc = __ffs(~c) - 1;

        // ---- off the chain, while the products of this chunk run: operands of the next (earlier) chunk
        if (c >= 2) {
            stage_dl(c - 1, (it + 1) & 1);                  // rows of chunk c - 1, fetched one iteration ago
            if (c >= 3) fetch_do(c - 2);
        }

        // ---- the chain: products -> masters -> bf16 copies for the next (earlier) chunk
        {
            const bool ok = umma::mbar_wait(barT, phT, abort_flag);
            phT ^= 1;
            if (!__all_sync(0xffffffffu, ok)) break;
        }
        umma::fence_after_sync();
        if (jc > 0 && trans) {
            // below the carry every level receives the carry level's new adjoint on top of its own reader term
            float ej[16];
            umma::tmem_ld16(tM + jc * gtc::VS, ej);
#pragma unroll 1
            for (int lv = 0; lv < jc; ++lv) {
                float t[16];
                umma::tmem_ld16(tM + lv * gtc::VS, t);
#pragma unroll
                for (int j = 0; j < 16; ++j) t[j] += ej[j];
                umma::tmem_st16(tM + lv * gtc::VS, t);
            }
            umma::tmem_wait_st();
        }
        {
            // adjoints of the states that chunk c reads = of the states written by chunk c - 1: bf16 copies for the next
            // iteration and, in the [K][32] layout, for the chunk-parallel gradient kernel
            uint32_t m = (uint32_t)c & lev_mask;
#pragma unroll 1
            while (m) {
                const int lv = __ffs(m) - 1;
                m &= m - 1;
                float v[16];
                umma::tmem_ld16(tM + lv * gtc::VS, v);
                uint32_t mine[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) mine[j] = pack_bf16(v[2 * j], v[2 * j + 1]);
                st_global_32B(p.dhs + pair_tile(c - 1, lv) + (size_t)row * 64 + (vs & 1) * gtc::VS + ch * 16, mine);
                ts_state.store(aE + lv * gtc::LV_BYTES, mine);
            }
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        mbar_arrive(barS);
    }
    umma::fence_before_sync();
    bar_work();
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static int gdn_tc_maps(GdnParams& p) {
    const long BT = (long)p.B * p.T;
    int rc;
    if ((rc = tma::make_panel_map(&p.tm_qd, p.qd, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_kd, p.kd, BT, p.H, p.K, CH)) != 0) return rc;
    if ((rc = tma::make_panel_map(&p.tm_wk, p.wk, (long)p.B * p.NT * p.K, p.H, p.K, p.K)) != 0) return rc;
    return 0;
}

template <bool SAVE, bool OUT>
static int launch_scan_tc(GdnParams& p, cudaStream_t stream) {
    int rc = gdn_tc_maps(p);
    if (rc != 0) return rc;
    auto kern = gdn_scan_tc_kernel<SAVE, OUT>;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ScanTcSmem::total)) != cudaSuccess) return (int)e;
    kern<<<p.B * p.H * (p.V / gtc::VS), gtc::NTHREADS, ScanTcSmem::total, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

// mode 0: forward (output), 1: forward that keeps the level states, 2: recomputation for the backward (states only)
int gdn_scan_tc_dispatch(const GdnParams& p0, int mode, cudaStream_t stream) {
    if (p0.K != gtc::KD || p0.V % 64 != 0 || p0.NLEV > gtc::MAXLEV) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    GdnParams p = p0;
    if (mode == 0) return launch_scan_tc<false, true>(p, stream);
    if (mode == 1) return launch_scan_tc<true, true>(p, stream);
    return launch_scan_tc<true, false>(p, stream);
}

int gdn_scan_bwd_tc_dispatch(const GdnParams& p0, cudaStream_t stream) {
    if (p0.K != gtc::KD || p0.V % 64 != 0 || p0.NLEV > gtc::MAXLEV) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    GdnParams p = p0;
    int rc = gdn_tc_maps(p);
    if (rc != 0) return rc;
    auto kern = gdn_scan_bwd_tc_kernel;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ScanBwdTcSmem::total)) != cudaSuccess) return (int)e;
    kern<<<p.B * p.H * (p.V / gtc::VS), gtc::NTHREADS, ScanBwdTcSmem::total, stream>>>(p); LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

}  // namespace llattn

#ifdef LLATTN_STAMPS
extern "C" int llattn_debug_read_stamps_gdn(long long* host_dst) {
    return (int)cudaMemcpyFromSymbol(host_dst, llattn::g_stamps, sizeof(llattn::g_stamps));
}
#endif
