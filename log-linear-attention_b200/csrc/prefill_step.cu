// Prefill hand-off and single-token decode step of log-linear Mamba-2 for sm_100a.
//
// Reference being replaced: the level-state side of hattention_prefill (hattention/kernel.py:470-560:
// chunk_fwd_kernel_h's final states `ht` for the inter-chunk levels plus postprocess_prefill_hstate_,
// :378-466, for the levels inside the last chunk) and hattention_step (kernel.py:563-633 with
// HState.cascade_weak / insert / step_output, hattention/recurrent.py:42-54, 79-98, 134-166).
//
// After m + 1 = T tokens the state of level 0 is k_m v_m^T, and for every set bit j of m, level j + 1
// holds the 2^j tokens that follow the buckets of the higher set bits (oldest tokens in the highest
// level):   S_l = sum_{s in bucket l} exp(sum_{r = s+1 .. m} g_r) k_s v_s^T .
//   mamba2_final_state_kernel : one CTA per (batch, head, level) sums its bucket with warp-level MMA
//       (decay folded into v), 64 tokens at a time from the end of the bucket backwards.
//   mamba2_step_kernel : one CTA per (batch, head); the host passes the carry level j of the cascade
//       (levels 0..j are summed into level j); then every level is decayed by exp(g), level 0 becomes
//       k v^T, and o = q . sum_l lambda_l S_l.  HBM-bound: reads and writes L*K*V floats per head.
#include "llattn_common.cuh"
#include "../../include/llattn.h"

namespace llattn {

template <int KD, int VD>
__global__ void __launch_bounds__(256, 1) mamba2_final_state_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                                    const float* __restrict__ g, float* __restrict__ states,
                                                                    int B, int T, int H, int G, int L) {
    constexpr int LDK = KD + PAD, LDV = VD + PAD;
    constexpr int MT = KD / 128;                         // 16-row tiles of the K x V result per warp (8 warps)
    static_assert(KD % 128 == 0 || KD == 64, "K rows are split over the warps");
    __shared__ __align__(16) bf16 sK[CH * LDK];
    __shared__ __align__(16) bf16 sVs[CH * LDV];
    __shared__ float sDec[CH];
    __shared__ float sRed[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int lev = blockIdx.y;
    const int h = blockIdx.x % H, b = blockIdx.x / H;
    const int grp = h / (H / G);
    const int m = T - 1;
    // bucket of this level
    int s0 = 0, s1 = 0;
    if (lev == 0) {
        s0 = m;
        s1 = m + 1;
    } else if (lev - 1 < 31 && ((m >> (lev - 1)) & 1)) {
        s0 = (m >> lev) << lev;                          // tokens taken by the higher set bits
        s1 = s0 + (1 << (lev - 1));
    }
    float* out = states + ((long)(b * H + h) * KD * VD) * L + lev;
    if (s1 == s0) {
        for (int e = tid; e < KD * VD; e += 256) out[(long)e * L] = 0.f;
        return;
    }
    // decay from the end of the bucket to the last token: sum_{r = s1 .. m} g_r
    float part = 0.f;
    for (int r = s1 + tid; r <= m; r += 256) part += g[((long)b * T + r) * H + h];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
    if (lane == 0) sRed[warp] = part;
    __syncthreads();
    float after = 0.f;
    for (int w = 0; w < 8; ++w) after += sRed[w];

    // warps split the K rows: K = 128 -> 16 rows each; K = 64 -> warps 0..3 take 16 rows each
    const bool active = (KD >= 128) || warp < 4;
    constexpr int MTW = (KD >= 128) ? MT : 1;
    float acc[MTW][VD / 8][4];
    zero_acc(acc);
    const int lr = lane >> 2, lc2 = (lane & 3) * 2;
    for (int e1 = s1; e1 > s0; e1 -= CH) {
        const int a = max(e1 - CH, s0);                  // tile [a, e1), up to 64 tokens, rows beyond are zero
        const int n = e1 - a;
        __syncthreads();                                 // previous tile consumed
        // in-tile decay: token a + i gets exp(after + sum_{r = a+i+1 .. e1-1} g_r)
        if (warp == 0) {
            const int i0 = CH - 1 - 2 * lane, i1 = CH - 2 - 2 * lane;      // reversed order
            float x0 = (i0 + 1 < n) ? g[((long)b * T + a + i0 + 1) * H + h] : 0.f;
            float x1 = (i1 + 1 < n) ? g[((long)b * T + a + i1 + 1) * H + h] : 0.f;
            warp_cumsum64(x0, x1, lane);
            sDec[i0] = (i0 < n) ? fexp(after + x0) : 0.f;
            sDec[i1] = (i1 < n) ? fexp(after + x1) : 0.f;
        }
        for (int e = tid; e < CH * (KD / 8); e += 256) {
            const int i = e / (KD / 8), c8 = (e % (KD / 8)) * 8;
            uint4 x = make_uint4(0, 0, 0, 0);
            if (i < n) x = *reinterpret_cast<const uint4*>(k + (((long)b * T + a + i) * G + grp) * KD + c8);
            *reinterpret_cast<uint4*>(sK + i * LDK + c8) = x;
        }
        __syncthreads();
        for (int e = tid; e < CH * (VD / 8); e += 256) {
            const int i = e / (VD / 8), c8 = (e % (VD / 8)) * 8;
            uint4 x = make_uint4(0, 0, 0, 0);
            if (i < n) {
                x = *reinterpret_cast<const uint4*>(v + (((long)b * T + a + i) * H + h) * VD + c8);
                const float d = sDec[i];
                uint32_t* xw = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&xw[q4]);
                    xw[q4] = pack_bf16(__bfloat162float(t2.x) * d, __bfloat162float(t2.y) * d);
                }
            }
            *reinterpret_cast<uint4*>(sVs + i * LDV + c8) = x;
        }
        __syncthreads();
        if (active) warp_gemm<MTW, VD / 16, true, true>(acc, sK, LDK, warp * 16 * MTW, sVs, LDV, 0, CH, lane);
        // decay accumulated over this tile for the next (earlier) tile: sum_{r = a .. e1-1} g_r
        float tile = 0.f;
        if (warp == 0) {
            float x = 0.f;
            for (int i = lane; i < n; i += 32) x += g[((long)b * T + a + i) * H + h];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
            if (lane == 0) sRed[0] = x;
        }
        __syncthreads();
        tile = sRed[0];
        after += tile;
    }
    if (active) {
#pragma unroll
        for (int mt = 0; mt < MTW; ++mt)
#pragma unroll
            for (int nt = 0; nt < VD / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int row = warp * 16 * MTW + mt * 16 + lr + (e >> 1) * 8, col = nt * 8 + lc2 + (e & 1);
                    out[((long)row * VD + col) * L] = acc[mt][nt][e];
                }
    }
}

// one decode step for one (batch, head) per CTA; thread t owns column t % VD and rows t / VD, + 256 / VD, ...
template <int MAXL>
__global__ void __launch_bounds__(256) mamba2_step_kernel(float* __restrict__ states, const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                          const bf16* __restrict__ v, const float* __restrict__ g, const bf16* __restrict__ lam,
                                                          bf16* __restrict__ o, int H, int G, int K, int V, int L, int carry) {
    extern __shared__ float sh[];                        // q[K] | k[K] | partial outputs [256]
    float* sQ = sh;
    float* sKk = sh + K;
    float* sO = sh + 2 * K;
    const int tid = threadIdx.x;
    const int h = blockIdx.x % H, b = blockIdx.x / H;
    const int grp = h / (H / G);
    for (int i = tid; i < K; i += 256) {
        sQ[i] = __bfloat162float(q[((long)b * G + grp) * K + i]);
        sKk[i] = __bfloat162float(k[((long)b * G + grp) * K + i]);
    }
    float lm[MAXL];
#pragma unroll
    for (int l = 0; l < MAXL; ++l) lm[l] = (l < L) ? __bfloat162float(lam[((long)b * H + h) * L + l]) : 0.f;
    const float dec = __expf(g[(long)b * H + h]);
    __syncthreads();
    const int col = tid % V, rstep = 256 / V;
    const float vv = __bfloat162float(v[((long)b * H + h) * V + col]);
    float* S = states + (long)(b * H + h) * K * V * L;
    float osum = 0.f;
    for (int row = tid / V; row < K; row += rstep) {
        float* p = S + ((long)row * V + col) * L;
        float s[MAXL];
#pragma unroll
        for (int l = 0; l < MAXL; ++l) s[l] = (l < L) ? p[l] : 0.f;
        // cascade: levels 0 .. carry are summed into level carry
        float merged = 0.f;
#pragma unroll
        for (int l = 0; l < MAXL; ++l)
            if (l <= carry) {
                merged += s[l];
                s[l] = 0.f;
            }
#pragma unroll
        for (int l = 0; l < MAXL; ++l)
            if (l == carry) s[l] = merged;
        float acc = 0.f;
#pragma unroll
        for (int l = 0; l < MAXL; ++l) {
            s[l] *= dec;
            if (l == 0) s[l] = sKk[row] * vv;
            acc += lm[l] * s[l];
            if (l < L) p[l] = s[l];
        }
        osum += sQ[row] * acc;
    }
    sO[tid] = osum;
    __syncthreads();
    if (tid < V) {
        float t = 0.f;
        for (int r = 0; r < rstep; ++r) t += sO[r * V + tid];
        o[((long)b * H + h) * V + tid] = __float2bfloat16(t);
    }
}

}  // namespace llattn

extern "C" {

int llattn_mamba2_final_state(const void* k, const void* v, const float* g, float* states,
                              int B, int T, int H, int G, int K, int V, int L, void* stream) {
    if (B <= 0 || T <= 0 || H <= 0 || G <= 0 || H % G != 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (!((K == 64 || K == 128) && V == 64) || L <= 0 || L > 32) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (L < 1 + (32 - __builtin_clz((unsigned)(T - 1) | 1u)) && T > 1) return LLATTN_ERR_TOO_FEW_LEVELS;
    if (!k || !v || !g || !states) return LLATTN_ERR_NULL;
    using bf = __nv_bfloat16;
    dim3 grid(B * H, L);
    cudaStream_t st = (cudaStream_t)stream;
    if (K == 128) { llattn::mamba2_final_state_kernel<128, 64><<<grid, 256, 0, st>>>((const bf*)k, (const bf*)v, g, states, B, T, H, G, L); LLATTN_LAUNCHED(); }
    else { llattn::mamba2_final_state_kernel<64, 64><<<grid, 256, 0, st>>>((const bf*)k, (const bf*)v, g, states, B, T, H, G, L); LLATTN_LAUNCHED(); }
    return (int)cudaGetLastError();
}

int llattn_mamba2_step(float* states, const void* q, const void* k, const void* v, const float* g, const void* lambda, void* o,
                       int B, int H, int G, int K, int V, int L, int carry_level, void* stream) {
    if (B <= 0 || H <= 0 || G <= 0 || H % G != 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (K <= 0 || K > 1024 || V <= 0 || V > 256 || 256 % V != 0 || L <= 0 || L > 32) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (carry_level < 0 || carry_level >= L) return LLATTN_ERR_TOO_FEW_LEVELS;
    if (!states || !q || !k || !v || !g || !lambda || !o) return LLATTN_ERR_NULL;
    using bf = __nv_bfloat16;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sm = (size_t)(2 * K + 256) * sizeof(float);
    if (L <= 16)
        llattn::mamba2_step_kernel<16><<<B * H, 256, sm, st>>>(states, (const bf*)q, (const bf*)k, (const bf*)v, g, (const bf*)lambda, (bf*)o, H, G, K, V, L, carry_level);
    else
        llattn::mamba2_step_kernel<32><<<B * H, 256, sm, st>>>(states, (const bf*)q, (const bf*)k, (const bf*)v, g, (const bf*)lambda, (bf*)o, H, G, K, V, L, carry_level);
    LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

}  // extern "C"
