// Log-linear Gated DeltaNet: the sequential scans over chunks on tcgen05 / TMEM / TMA (K = 128).
//
// Same mathematics as gdn_scan_kernel (gdn_fwd.cu) and gdn_scan_bwd_kernel (gdn_bwd.cu); reference being
// replaced: hattention/chunkwise_hgdn.py:718-788 with fla_future/chunk_delta_h.py:34-186 (forward state
// recurrence per level) and :206-368 (its adjoint).  One CTA per (batch, head, 32-column slice of V) walks the
// chunks in order.  The transition of a level state is used in the form
//     H' = exp(gl) H - (kd^T wd) H  (+ kd^T u for the level that receives the chunk's own writes)
// with the K x K matrix -kd^T wd of every chunk prepared by the chunk-parallel kernel, so that the dependent
// chain of a chunk is ONE batch of tensor-core products followed by ONE element-wise step:
//     level states (bf16, shared memory) --MMA--> -W H_lv (+ kd^T u)  --> fp32 masters (registers) --> bf16 copies
// The reader products qd H_lv (output) use the same bf16 copies but are off the chain: they are issued after the
// transition products and consumed one chunk later.  Every product is a tcgen05.mma chain issued by one thread
// with M = 128.  The level states are kept transposed ([V column][K]) so that they are K-major B operands whose
// rows continue from level to level: a range of levels is read by ONE chain with N = 32 x (number of levels).  Accumulators sit in tensor memory (one 32-column slot per level and kind of product); eight
// element-wise warps (two per lane quarter, 16 columns each) hold the fp32 masters.
#include "tc_common.cuh"
#include "llattn_gdn.h"

namespace llattn {

namespace gtc {
constexpr int KD = 128, VS = GDN_VS, MAXLEV = GDN_MAXLEV;
constexpr int NTHREADS = 384, MMA_WARP = 8;
constexpr uint32_t QD_BYTES = CH * KD * 2;               // qd / kd / wd tile: two panels of 64 rows
constexpr uint32_t WK_BYTES = KD * KD * 2;               // -kd^T wd: two panels of 128 rows
constexpr uint32_t STAGE_BYTES = 2 * QD_BYTES + WK_BYTES;   // qd | kd | wk  (forward)   /   kd | qd | wk  (reverse)
constexpr uint32_t ST_ROWS = MAXLEV * VS;                // rows of the transposed state tile: level * 32 + column
constexpr uint32_t ST_BYTES = ST_ROWS * KD * 2;          // two panels of 256 rows
constexpr uint32_t UT_BYTES = VS * 128;                  // u^T: one panel of 32 rows ([column][token])
constexpr int TM_R = 0, TM_T = 256, TM_COLS = 512;       // reader / transition products: slot of level lv at lv * 32
}  // namespace gtc

struct ScanTcSmem {
    static constexpr uint32_t stage_off = 0;                                    // [2]
    static constexpr uint32_t st_off = stage_off + 2 * gtc::STAGE_BYTES;
    static constexpr uint32_t ut_off = st_off + gtc::ST_BYTES;                  // [2]
    static constexpr uint32_t bar_off = ut_off + 2 * gtc::UT_BYTES;
    static constexpr uint32_t total = bar_off + 128 + 1024;                     // + slack for the 1024-byte alignment
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(bar)) : "memory");
}

// SAVE also writes, for every chunk, the bf16 level states that the chunk reads:
// hs[((b*H + h)*nvs + vs)*NT + c][level][K][32] (the backward's recomputation, or a forward whose caller keeps
// the workspace for the backward); OUT = false skips the output (recomputation only).
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
        RegisterSplit<56, 224>::release();
        if (warp == gtc::MMA_WARP + 1) {
            if (lane == 0) {
                for (int c = 0; c < NT; ++c) {
                    const int st = c & 1;
                    if (c >= 2 && !umma::mbar_wait(&empty[st], ((c >> 1) - 1) & 1, abort_flag)) break;
                    const int row0 = b * p.T + c * CH;
                    unsigned char* qd = sStage + st * gtc::STAGE_BYTES;
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
            const uint32_t aQd = umma::smem_addr(sStage + st * gtc::STAGE_BYTES);
            const uint32_t aKd = aQd + gtc::QD_BYTES, aWk = aKd + gtc::QD_BYTES;
            const uint32_t aUT = umma::smem_addr(sUT + st * gtc::UT_BYTES);
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
                STAMP();
                if (ok && c > 0) ok = umma::mbar_wait(barS, (c - 1) & 1, abort_flag);
                STAMP();
                if (ok && trans) ok = umma::mbar_wait(&barU[st], (c >> 1) & 1, abort_flag);
                STAMP();
                if (ok) {
                    umma::fence_after_sync();
                    if (trans) {
                        // level that receives this chunk's writes and everything below the carry: kd^T u - W (sum of those states)
                        // An instruction costs about the same for N = 32 as for N = 128, so the -W H_lv products are issued as
                        // at most two chains: the levels below the carry (all live; the element-wise warps add their slots into
                        // the carry level), and ONE chain that spans the live levels above the carry (slots of levels in
                        // between that are not live receive products of stale copies and are ignored).
                        umma::gemm_mk<CH, gtc::VS, CH>(tbase + gtc::TM_T + jc * gtc::VS, aKd, aUT, ID_MK32, false);
                        if (jc > 0)
                            umma::gemm_kk<gtc::KD, gtc::ST_ROWS, gtc::KD>(tbase + gtc::TM_T, aWk, aSt, umma::idesc_bf16(128, gtc::VS * jc, false, false), false);
                        const uint32_t above = live & ~((2u << jc) - 1u);
                        if (above) {
                            const int lo = __ffs(above) - 1, hi = 31 - __clz(above);
                            umma::gemm_kk<gtc::KD, gtc::ST_ROWS, gtc::KD>(tbase + gtc::TM_T + lo * gtc::VS, aWk, aSt + lo * gtc::VS * 128,
                                                                          umma::idesc_bf16(128, gtc::VS * (hi - lo + 1), false, false), false);
                        }
                        umma::commit(barT);
                    }
                    STAMP();
                    if (OUT) {
                        if (c > 0) ok = umma::mbar_wait(barO, (c - 1) & 1, abort_flag);
                        STAMP();
                        if (ok && live) {
                            umma::fence_after_sync();
                            // readers: qd H_lv in rows 0..63 (rows 64..127 of the M = 128 product are not used)
                            // one chain from the lowest to the highest live level
                            const int lo = __ffs(live) - 1, hi = 31 - __clz(live);
                            umma::gemm_kk<CH, gtc::ST_ROWS, gtc::KD>(tbase + gtc::TM_R + lo * gtc::VS, aQd, aSt + lo * gtc::VS * 128,
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
    RegisterSplit<56, 224>::acquire();
    const int rb = warp & 3, ch = warp >> 2;
    const int row = rb * 32 + lane;            // tensor-memory lane: token (reader products), state row k (transition products)
    const bool qrow = rb < 2;                  // warp-uniform: lane quarters 0, 1 write the output, 2, 3 stage u^T
    const int tok = row & 63;
    const int col0 = vs * gtc::VS + ch * 16;   // this thread's 16 V columns

    float M[gtc::MAXLEV][16];                  // fp32 masters: state row `row`, 16 columns, every level
#pragma unroll
    for (int lv = 0; lv < gtc::MAXLEV; ++lv)
#pragma unroll
        for (int j = 0; j < 16; ++j) M[lv][j] = 0.f;

    // Per-chunk inputs are fetched ahead of their use: the chunk's total log decay (one chunk ahead); for the
    // output warps the lambda row and 16 columns of the intra-chunk output of the chunk whose reader products
    // are in flight; for the others 16 columns of u two chunks ahead (staged transposed one chunk ahead).
    float gl_n = 0.f;
    uint4 in_n[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    uint32_t lam_n[gtc::MAXLEV / 2] = {0, 0, 0, 0};
    auto token_row = [&](int c) -> long { return ((long)b * p.T + (long)c * CH + tok) * p.H + h; };
    auto fetch_gl = [&](int c) { gl_n = p.g_cum[((long)b * p.T + (long)c * CH + (CH - 1)) * p.H + h]; };
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
        const unsigned short* lp = reinterpret_cast<const unsigned short*>(p.l + r * p.L + INTRA_LEVELS);
#pragma unroll
        for (int i = 0; i < gtc::MAXLEV / 2; ++i) {
            const uint32_t a = (2 * i < nlev) ? lp[2 * i] : 0u, bb = (2 * i + 1 < nlev) ? lp[2 * i + 1] : 0u;
            lam_n[i] = a | (bb << 16);
        }
    };
    // 16 columns of u of one token into the transposed tile [column][token]
    auto stage_ut = [&](const uint4 (&x)[2], int buf) {
        unsigned char* dst = sUT + buf * gtc::UT_BYTES;
        const uint32_t* xin = reinterpret_cast<const uint32_t*>(x);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            *reinterpret_cast<unsigned short*>(dst + umma::tile_offset(ch * 16 + 2 * j, tok, gtc::VS)) = (unsigned short)(xin[j] & 0xFFFFu);
            *reinterpret_cast<unsigned short*>(dst + umma::tile_offset(ch * 16 + 2 * j + 1, tok, gtc::VS)) = (unsigned short)(xin[j] >> 16);
        }
        umma::fence_async_smem();
        mbar_arrive(&barU[buf]);
    };
    // output rows of chunk c: lambda-weighted reader products plus the intra-chunk part
    uint32_t phR = 0;
    auto write_output = [&](int c, const uint4 (&x)[2], const uint32_t (&lam)[gtc::MAXLEV / 2], uint32_t tR, bool wait_products) -> bool {
        const uint32_t live = (uint32_t)c & lev_mask;
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
        if (live) {
            if (wait_products) {
                const bool ok = umma::mbar_wait(barR, phR, abort_flag);
                phR ^= 1;
                if (!__all_sync(0xffffffffu, ok)) return false;
                umma::fence_after_sync();
            }
            // two level slots per wait (a slot of a level that is not live holds stale values and is ignored)
#pragma unroll
            for (int g = 0; g < gtc::MAXLEV / 2; ++g) {
                if ((live >> (2 * g)) & 0x3u) {
                    float r[2][16];
                    umma::tmem_ld16x2(tR + (2 * g) * gtc::VS, r[0], tR + (2 * g + 1) * gtc::VS, r[1]);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int lv = 2 * g + i;
                        if ((live >> lv) & 1) {
                            const float lm = __uint_as_float(((lam[lv >> 1] >> ((lv & 1) * 16)) & 0xFFFFu) << 16);
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[j] += lm * r[i][j];
                        }
                    }
                }
            }
            umma::fence_before_sync();
        }
        mbar_arrive(barO);
        const uint32_t* xin = reinterpret_cast<const uint32_t*>(x);
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xin[j]);
            w[j] = pack_bf16(__bfloat162float(v2.x) + acc[2 * j], __bfloat162float(v2.y) + acc[2 * j + 1]);
        }
        uint4* d4 = reinterpret_cast<uint4*>(p.o + token_row(c) * p.V + col0);
        d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
        d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
        return true;
    };

    fetch_gl(0);
    if (!qrow) {
        fetch_u(0);
        if (NT > 1) stage_ut(in_n, 0);
        if (NT > 1) fetch_u(1);
    }
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;
    const uint32_t tR = umma::tmem_addr(tbase + gtc::TM_R, warp, ch * 16), tT = umma::tmem_addr(tbase + gtc::TM_T, warp, ch * 16);
    uint32_t phT = 0;
    bool alive = true;
    // Transposed bf16 copy of one level: element (column n, row k) of the [32 x 128] block.  Two neighbouring lanes hold rows
    // k, k + 1; they exchange halves so that each writes 32-bit words (rows k, k+1 of one column): the even lane the even
    // columns, the odd lane the odd ones.  Address pieces that do not change are computed once.
    const int par = lane & 1;
    const uint32_t st_base = umma::smem_addr(sSt) + (uint32_t)((row >> 6) * gtc::ST_ROWS * 128 + (ch * 16 + par) * 128 + (row & 6) * 2);
    uint32_t st_xo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) st_xo[i] = (uint32_t)((((row & 63) >> 3) ^ ((2 * i + par) & 7)) << 4);
    const uint32_t st_sel = par ? 0x3276u : 0x5410u;
    auto store_state_transposed = [&](uint32_t level_base, const float (&v)[16]) {
        uint32_t word[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const uint32_t mine = pack_bf16(v[2 * m], v[2 * m + 1]);
            word[m] = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 1), st_sel);
        }
#pragma unroll
        for (int m = 0; m < 8; ++m)
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(level_base + (uint32_t)(m * 256) + st_xo[m & 3]), "r"(word[m]) : "memory");
    };

    for (int c = 0; c < NT; ++c) {
        const uint32_t live = (uint32_t)c & lev_mask;
        const bool trans = (c + 1 < NT);
        const int jc = __ffs(~c) - 1;
        const float dec = fexp(gl_n);
#ifdef LLATTN_STAMPS
        int nstamp = 0;
        const int stamp_slot = (blockIdx.x == 5 && c == 37) ? (tid == 0 ? 0 : (tid == 64 ? 1 : -1)) : -1;
#endif
        STAMP();
        if (c + 1 < NT) fetch_gl(c + 1);

        // ---- off the chain, while the products of this chunk run
        if (qrow) {
            if (OUT) {
                if (c > 0 && !write_output(c - 1, in_n, lam_n, tR, false)) { alive = false; break; }
                fetch_o(c);                                          // consumed in the next iteration
            }
        } else if (c + 2 < NT) {
            stage_ut(in_n, (c + 1) & 1);                             // u of chunk c + 1 (needed only if that chunk has a transition)
            fetch_u(c + 2);
        }
        if (SAVE) {
            bf16* dst = p.hs + ((size_t)blockIdx.x * NT + c) * nlev * (gtc::KD * gtc::VS) + (size_t)row * gtc::VS + ch * 16;
#pragma unroll
            for (int lv = 0; lv < gtc::MAXLEV; ++lv) {
                if ((live >> lv) & 1) {
                    uint32_t w[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) w[j] = pack_bf16(M[lv][2 * j], M[lv][2 * j + 1]);
                    uint4* d4 = reinterpret_cast<uint4*>(dst + (size_t)lv * gtc::KD * gtc::VS);
                    d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
        if (OUT && c == NT - 1 && p.final_states != nullptr) {
            // prefill hand-off: the level states every token of the last chunk starts from.  Level 7 + lv holds the block
            // of 2^lv chunks for each set bit lv of c (the binary-indexed tree as it stands before this chunk); the
            // caller steps the last chunk's tokens through the decode kernel, which fills levels 0..6.
            float* dst = p.final_states + (((long)b * p.H + h) * gtc::KD + row) * (long)p.V * p.L;
#pragma unroll
            for (int lv = 0; lv < gtc::MAXLEV; ++lv) {
                if ((live >> lv) & 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) dst[(long)(col0 + j) * p.L + INTRA_LEVELS + lv] = M[lv][j];
                }
            }
        }
        if (!trans) break;
        STAMP();

        // ---- the chain: transition products -> fp32 masters -> bf16 copies for the next chunk
        {
            const bool ok = umma::mbar_wait_backoff(barT, phT, abort_flag, 32);
            phT ^= 1;
            if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        }
        STAMP();
        umma::fence_after_sync();
        {
            // the states below the carry merge into the carry level (whose master is zero until now)
#pragma unroll
            for (int tgt = 1; tgt < gtc::MAXLEV; ++tgt) {
                if (tgt == jc) {
#pragma unroll
                    for (int lv = 0; lv < tgt; ++lv)
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            M[tgt][j] += M[lv][j];
                            M[lv][j] = 0.f;
                        }
                }
            }
            const uint32_t dest = (uint32_t)(c + 1) & lev_mask;       // the carry level and the live levels above it
            const uint32_t below = (1u << jc) - 1u;                   // their -W H_lv products go to the carry level
            // the carry level first (its slot may sit in a later group than the slots added to it)
#pragma unroll
            for (int g = gtc::MAXLEV / 4 - 1; g >= 0; --g) {
                if (((dest | below) >> (4 * g)) & 0xFu) {
                    uint32_t t[4][16];
#pragma unroll
                    for (int i = 0; i < 4; ++i) umma::tmem_ld16_issue(tT + (4 * g + i) * gtc::VS, t[i]);
                    umma::tmem_ld_wait4(t[0], t[1], t[2], t[3]);
#pragma unroll
                    for (int i = 3; i >= 0; --i) {
                        const int lv = 4 * g + i;
                        if ((dest >> lv) & 1) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) M[lv][j] = dec * M[lv][j] + __uint_as_float(t[i][j]);
                        } else if (lv < jc) {
#pragma unroll
                            for (int tgt = 1; tgt < gtc::MAXLEV; ++tgt) {
                                if (tgt > lv && tgt == jc) {
#pragma unroll
                                    for (int j = 0; j < 16; ++j) M[tgt][j] += __uint_as_float(t[i][j]);
                                }
                            }
                        }
                    }
                }
            }
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
#pragma unroll
        for (int lv = 0; lv < gtc::MAXLEV; ++lv) {
            if ((((uint32_t)(c + 1) & lev_mask) >> lv) & 1) store_state_transposed(st_base + lv * gtc::VS * 128, M[lv]);
        }
        STAMP();
        umma::fence_async_smem();
        umma::fence_before_sync();
        mbar_arrive(barS);
        STAMP();
    }
    if (OUT && qrow && alive) {
        // reader products of the last chunk
        write_output(NT - 1, in_n, lam_n, tR, true);
    }
    umma::fence_before_sync();
    bar_work();
}

// ------------------------------------------------------------------------------------------
// reverse scan: adjoints of the level states.  With W = -kd^T wd the adjoint recurrence of a state is
//     E (adjoint after chunk c)  ->  exp(gl) E + W^T E  (+ qd^T (lambda_lv * do) for the levels the chunk reads)
// W^T is the same shared-memory tile read MN-major.  The reader terms do not depend on E: their operands
// (lambda_lv * do, transposed, one 32-row block per level) are staged one chunk ahead and their products are
// issued in the same batch, accumulating onto W^T E_lv where both go to the same level.  d_u = kd E_jc is left
// to the chunk-parallel gradient kernel, which holds the same adjoint tiles.
// ------------------------------------------------------------------------------------------
struct ScanBwdTcSmem {
    static constexpr uint32_t STAGE = gtc::QD_BYTES + gtc::WK_BYTES;            // qd | wk
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
        RegisterSplit<56, 224>::release();
        if (warp == gtc::MMA_WARP + 1) {
            if (lane == 0) {
                for (int it = 0; it < NT; ++it) {
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
        for (int it = 0; it < NT && ok; ++it) {
            const int c = NT - 1 - it, st = it & 1;
            const uint32_t aQd = umma::smem_addr(sStage + st * SM::STAGE), aWk = aQd + gtc::QD_BYTES;
            const uint32_t aDL = umma::smem_addr(sDL + st * SM::DL_BYTES);
            const uint32_t readers = (uint32_t)c & lev_mask;             // levels whose states this chunk reads
            const bool trans = (c + 1 < NT);
            const uint32_t written = trans ? ((uint32_t)(c + 1) & lev_mask) : 0u;   // levels that hold a state after this chunk
            const int jc = __ffs(~c) - 1;
            if (lane == 0) {
                ok = umma::mbar_wait(&full[st], (it >> 1) & 1, abort_flag);
                if (ok && it > 0) ok = umma::mbar_wait(barS, (it - 1) & 1, abort_flag);
                if (ok && readers) ok = umma::mbar_wait(&barD[st], (it >> 1) & 1, abort_flag);
                if (ok) {
                    umma::fence_after_sync();
                    // W^T E_lv for every level written by this chunk (the carry level's product is shared by all levels below
                    // it): ONE chain from the carry level to the highest such level (an instruction costs about the same for
                    // N = 32 as for N = 128; slots of levels in between receive products of stale copies and are ignored)
                    if (written) {
                        const int hi = 31 - __clz(written);
                        umma::gemm_mk<gtc::KD, gtc::ST_ROWS, gtc::KD>(tbase + jc * gtc::VS, aWk, aE + jc * gtc::VS * 128,
                                                                      umma::idesc_bf16(128, gtc::VS * (hi - jc + 1), true, false), false);
                    }
                    // qd^T (lambda_lv * do): below the carry into fresh slots, above it onto W^T E_lv
                    const uint32_t above = readers & ~((2u << jc) - 1u);
                    if (jc > 0)
                        umma::gemm_mk<CH, gtc::ST_ROWS, CH>(tbase, aQd, aDL, umma::idesc_bf16(128, gtc::VS * jc, true, false), false);
                    if (above) {
                        const int lo = __ffs(above) - 1, hi = 31 - __clz(above);
                        umma::gemm_mk<CH, gtc::ST_ROWS, CH>(tbase + lo * gtc::VS, aQd, aDL + lo * gtc::VS * 128,
                                                            umma::idesc_bf16(128, gtc::VS * (hi - lo + 1), true, false), trans);
                    }
                    umma::commit(barT);
                    umma::commit(&empty[st]);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (lane == 0 && ok) umma::mbar_wait(&empty[(NT - 1) & 1], ((NT - 1) >> 1) & 1, abort_flag);
        __syncwarp();
        if (*abort_flag && lane == 0) atomicExch(p.err, 1);
        umma::fence_before_sync();
        bar_work();
        umma::tmem_dealloc(tbase, TCOLS);
        return;
    }

    // ================= warps 0..7 =================
    RegisterSplit<56, 224>::acquire();
    const int rb = warp & 3, ch = warp >> 2;
    const int row = rb * 32 + lane;            // state row k
    const int tok = row & 63;                  // token whose do / lambda row this thread stages
    const int lpar = rb >> 1;                  // ... for the live levels of this parity (in order of appearance)
    const int col0 = vs * gtc::VS + ch * 16;

    float E[gtc::MAXLEV][16];                  // fp32 masters of the adjoints
#pragma unroll
    for (int lv = 0; lv < gtc::MAXLEV; ++lv)
#pragma unroll
        for (int j = 0; j < 16; ++j) E[lv][j] = 0.f;

    float gl_n = 0.f;
    uint4 do_n[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    uint32_t lam_n[gtc::MAXLEV / 2] = {0, 0, 0, 0};
    auto fetch_gl = [&](int c) { gl_n = p.g_cum[((long)b * p.T + (long)c * CH + (CH - 1)) * p.H + h]; };
    auto fetch_do = [&](int c) {
        const long r = ((long)b * p.T + (long)c * CH + tok) * p.H + h;
        const uint4* src = reinterpret_cast<const uint4*>(p.d_o + r * p.V + col0);
        do_n[0] = src[0];
        do_n[1] = src[1];
        const unsigned short* lp = reinterpret_cast<const unsigned short*>(p.l + r * p.L + INTRA_LEVELS);
#pragma unroll
        for (int i = 0; i < gtc::MAXLEV / 2; ++i) {
            const uint32_t a = (2 * i < nlev) ? lp[2 * i] : 0u, bb = (2 * i + 1 < nlev) ? lp[2 * i + 1] : 0u;
            lam_n[i] = a | (bb << 16);
        }
    };
    // (lambda_lv * do)^T of chunk c for every level the chunk reads; the two halves of the CTA take alternate levels
    auto stage_dl = [&](int c, const uint4 (&x)[2], const uint32_t (&lam)[gtc::MAXLEV / 2], int buf) {
        const uint32_t readers = (uint32_t)c & lev_mask;
        if (!readers) return;
        unsigned char* dst = sDL + buf * SM::DL_BYTES;
        const uint32_t* xin = reinterpret_cast<const uint32_t*>(x);
        int seen = 0;
#pragma unroll
        for (int lv = 0; lv < gtc::MAXLEV; ++lv) {
            if ((readers >> lv) & 1) {
                if ((seen & 1) == lpar) {
                    const float lm = __uint_as_float(((lam[lv >> 1] >> ((lv & 1) * 16)) & 0xFFFFu) << 16);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(&xin[j]);
                        *reinterpret_cast<bf16*>(dst + umma::tile_offset(lv * gtc::VS + ch * 16 + 2 * j, tok, gtc::ST_ROWS)) =
                            __float2bfloat16(lm * __bfloat162float(v2.x));
                        *reinterpret_cast<bf16*>(dst + umma::tile_offset(lv * gtc::VS + ch * 16 + 2 * j + 1, tok, gtc::ST_ROWS)) =
                            __float2bfloat16(lm * __bfloat162float(v2.y));
                    }
                }
                ++seen;
            }
        }
        umma::fence_async_smem();
        mbar_arrive(&barD[buf]);
    };

    fetch_gl(NT - 1);
    fetch_do(NT - 1);
    stage_dl(NT - 1, do_n, lam_n, 0);
    if (NT > 1) fetch_do(NT - 2);
    umma::fence_before_sync();
    bar_work();
    umma::fence_after_sync();
    const uint32_t tbase = *tmem_slot;
    const uint32_t tT = umma::tmem_addr(tbase, warp, ch * 16);
    uint32_t phT = 0;
    // transposed bf16 copy of one level, written as 32-bit words by pairs of lanes (see the forward kernel)
    const int par = lane & 1;
    const uint32_t e_base = umma::smem_addr(sE) + (uint32_t)((row >> 6) * gtc::ST_ROWS * 128 + (ch * 16 + par) * 128 + (row & 6) * 2);
    uint32_t st_xo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) st_xo[i] = (uint32_t)((((row & 63) >> 3) ^ ((2 * i + par) & 7)) << 4);
    const uint32_t st_sel = par ? 0x3276u : 0x5410u;
    auto store_state_transposed = [&](uint32_t level_base, const float (&v)[16]) {
        uint32_t word[8];
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const uint32_t mine = pack_bf16(v[2 * m], v[2 * m + 1]);
            word[m] = __byte_perm(mine, __shfl_xor_sync(0xffffffffu, mine, 1), st_sel);
        }
#pragma unroll
        for (int m = 0; m < 8; ++m)
            asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(level_base + (uint32_t)(m * 256) + st_xo[m & 3]), "r"(word[m]) : "memory");
    };

    for (int it = 0; it < NT; ++it) {
        const int c = NT - 1 - it;
        const uint32_t readers = (uint32_t)c & lev_mask;
        const bool trans = (c + 1 < NT);
        const uint32_t written = trans ? ((uint32_t)(c + 1) & lev_mask) : 0u;
        const int jc = __ffs(~c) - 1;
        const float dec = fexp(gl_n);
        if (c >= 1) fetch_gl(c - 1);

        // ---- off the chain, while the products of this chunk run
        if (c >= 1) stage_dl(c - 1, do_n, lam_n, (it + 1) & 1);   // rows of chunk c - 1, fetched one iteration ago
        if (c >= 2) fetch_do(c - 2);
        if (trans) {
            // adjoints of the states written by this chunk, for the chunk-parallel gradient kernel
            bf16* dst = p.dhs + ((size_t)blockIdx.x * NT + c) * nlev * (gtc::KD * gtc::VS) + (size_t)row * gtc::VS + ch * 16;
#pragma unroll
            for (int lv = 0; lv < gtc::MAXLEV; ++lv) {
                if ((written >> lv) & 1) {
                    uint32_t w[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) w[j] = pack_bf16(E[lv][2 * j], E[lv][2 * j + 1]);
                    uint4* d4 = reinterpret_cast<uint4*>(dst + (size_t)lv * gtc::KD * gtc::VS);
                    d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
        if (c == 0) break;                                  // no state exists before the first chunk

        // ---- the chain: products -> fp32 masters -> bf16 copies for the next (earlier) chunk
        {
            const bool ok = umma::mbar_wait_backoff(barT, phT, abort_flag, 32);
            phT ^= 1;
            if (!__all_sync(0xffffffffu, ok)) break;
        }
        umma::fence_after_sync();
        {
            // Below the carry every level receives the same transition term  exp(gl) E_jc + W^T E_jc: it is formed in
            // place in the carry level's master (which is cleared at the end, that level is not read by this chunk).
            uint32_t tj[16];
            if (trans) umma::tmem_ld16_issue(tT + jc * gtc::VS, tj);           // completes with the first pair below
            bool have_common = !trans;
#pragma unroll
            for (int g = 0; g < gtc::MAXLEV / 2; ++g) {
                if ((readers >> (2 * g)) & 0x3u) {
                    float t[2][16];
                    umma::tmem_ld16x2(tT + (2 * g) * gtc::VS, t[0], tT + (2 * g + 1) * gtc::VS, t[1]);
                    if (!have_common) {
                        umma::tmem_ld_wait1(tj);
#pragma unroll
                        for (int lv = 0; lv < gtc::MAXLEV; ++lv) {
                            if (lv == jc) {
#pragma unroll
                                for (int j = 0; j < 16; ++j) E[lv][j] = dec * E[lv][j] + __uint_as_float(tj[j]);
                            }
                        }
                        have_common = true;
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int lv = 2 * g + i;
                        if ((readers >> lv) & 1) {
                            if (lv < jc) {
#pragma unroll
                                for (int tgt = 1; tgt < gtc::MAXLEV; ++tgt) {
                                    if (tgt > lv && tgt == jc) {
#pragma unroll
                                        for (int j = 0; j < 16; ++j) E[lv][j] = (trans ? E[tgt][j] : 0.f) + t[i][j];
                                    }
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 16; ++j) E[lv][j] = dec * E[lv][j] + t[i][j];
                            }
                        }
                    }
                }
            }
            if (!have_common) umma::tmem_ld_wait1(tj);                          // not reached (a chunk c >= 1 reads at least one level)
#pragma unroll
            for (int lv = 0; lv < gtc::MAXLEV; ++lv) {
                if ((readers >> lv) & 1) {
                    store_state_transposed(e_base + lv * gtc::VS * 128, E[lv]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) E[lv][j] = 0.f;
                }
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
    if ((rc = tma::make_panel_map(&p.tm_wd, p.wd, BT, p.H, p.K, CH)) != 0) return rc;
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
    if (p0.K != gtc::KD || p0.V % gtc::VS != 0 || p0.NLEV > gtc::MAXLEV) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    GdnParams p = p0;
    if (mode == 0) return launch_scan_tc<false, true>(p, stream);
    if (mode == 1) return launch_scan_tc<true, true>(p, stream);
    return launch_scan_tc<true, false>(p, stream);
}

int gdn_scan_bwd_tc_dispatch(const GdnParams& p0, cudaStream_t stream) {
    if (p0.K != gtc::KD || p0.V % gtc::VS != 0 || p0.NLEV > gtc::MAXLEV) return LLATTN_ERR_UNSUPPORTED_SHAPE;
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
