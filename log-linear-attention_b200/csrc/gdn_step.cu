// One decode step of the log-linear Gated DeltaNet layer (delta-rule transition on every level state).
//
// Reference being replaced: hattention_step with hstruct = GDELTA (hattention/kernel.py:563-633), i.e.
// HState.cascade_weak / insert and step_output (hattention/recurrent.py:42-54, 79-98, 134-166):
//   cascade      levels 0 .. carry are summed into level carry (the caller runs the cascade on the token counts)
//   transition   S_l <- exp(g) (S_l - beta k (k^T S_l))          for every level l
//   write        S_0 <- beta k v^T
//   output       o = q . sum_l lambda_l S_l
// The states are fp32 (B,H,K,V,L), level innermost, updated in place in ONE pass over HBM: a CTA owns 8 value
// columns of one (batch, head); its 256 threads hold the K x 8 x L slice in registers (thread = one column, K/32
// rows), so k^T S_l is a reduction over threads (warp shuffles, then shared memory) between the load and the store.
#include "llattn_common.cuh"
#include "../../include/llattn.h"

namespace llattn {

constexpr int GS_VC = 8;      // value columns per CTA

template <int MAXL, int RPT>   // RPT = K / 32 rows per thread
__global__ void __launch_bounds__(256) gdn_step_kernel(float* __restrict__ states, const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                       const bf16* __restrict__ v, const bf16* __restrict__ beta, const float* __restrict__ g,
                                                       const bf16* __restrict__ lam, bf16* __restrict__ o, int H, int K, int V, int L, int carry) {
    __shared__ float sQ[256], sK[256];
    __shared__ float sRed[8][GS_VC][MAXL];
    __shared__ float sO[8][GS_VC];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nvc = V / GS_VC;
    const int vc = blockIdx.x % nvc;
    const int h = (blockIdx.x / nvc) % H;
    const int b = blockIdx.x / (nvc * H);
    const long bh = (long)b * H + h;
    for (int i = tid; i < K; i += 256) {
        sQ[i] = __bfloat162float(q[bh * K + i]);
        sK[i] = __bfloat162float(k[bh * K + i]);
    }
    float lm[MAXL];
#pragma unroll
    for (int l = 0; l < MAXL; ++l) lm[l] = (l < L) ? __bfloat162float(lam[bh * L + l]) : 0.f;
    const float dec = __expf(g[bh]);
    const float be = __bfloat162float(beta[bh]);
    const int colc = lane & 7;                     // column inside the CTA's slice
    const int rg = warp * 4 + (lane >> 3);         // row group 0..31: rows rg, rg + 32, ...
    const int col = vc * GS_VC + colc;
    const float vv = __bfloat162float(v[bh * V + col]);
    __syncthreads();

    float s[RPT][MAXL];
    float* S = states + bh * (long)K * V * L;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
        const float* pp = S + ((long)(rg + 32 * r) * V + col) * L;
#pragma unroll
        for (int l = 0; l < MAXL; ++l) s[r][l] = (l < L) ? pp[l] : 0.f;
        // cascade: levels 0 .. carry are summed into level carry
        float merged = 0.f;
#pragma unroll
        for (int l = 0; l < MAXL; ++l)
            if (l <= carry) {
                merged += s[r][l];
                s[r][l] = 0.f;
            }
#pragma unroll
        for (int l = 0; l < MAXL; ++l)
            if (l == carry) s[r][l] = merged;
    }
    // k^T S_l for this column: this thread's rows, then the 4 row groups of the warp, then the 8 warps
    float ks[MAXL];
#pragma unroll
    for (int l = 0; l < MAXL; ++l) {
        float x = 0.f;
#pragma unroll
        for (int r = 0; r < RPT; ++r) x += sK[rg + 32 * r] * s[r][l];
        x += __shfl_xor_sync(0xffffffffu, x, 8);
        x += __shfl_xor_sync(0xffffffffu, x, 16);
        ks[l] = x;
    }
    if (lane < 8) {
#pragma unroll
        for (int l = 0; l < MAXL; ++l) sRed[warp][lane][l] = ks[l];
    }
    __syncthreads();
#pragma unroll
    for (int l = 0; l < MAXL; ++l) {
        float x = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) x += sRed[w][colc][l];
        ks[l] = x;
    }
    // transition, write of the new token, output
    float osum = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
        const int row = rg + 32 * r;
        const float bk = be * sK[row];
        float* pp = S + ((long)row * V + col) * L;
        float acc = 0.f;
#pragma unroll
        for (int l = 0; l < MAXL; ++l) {
            float x = dec * (s[r][l] - bk * ks[l]);
            if (l == 0) x = bk * vv;
            acc += lm[l] * x;
            if (l < L) pp[l] = x;
        }
        osum += sQ[row] * acc;
    }
    osum += __shfl_xor_sync(0xffffffffu, osum, 8);
    osum += __shfl_xor_sync(0xffffffffu, osum, 16);
    if (lane < 8) sO[warp][lane] = osum;
    __syncthreads();
    if (tid < GS_VC) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += sO[w][tid];
        o[bh * V + vc * GS_VC + tid] = __float2bfloat16(t);
    }
}

}  // namespace llattn

extern "C" int llattn_gdn_step(float* states, const void* q, const void* k, const void* v, const void* beta, const float* g,
                               const void* lambda, void* o, int B, int H, int K, int V, int L, int carry_level, void* stream) {
    if (B <= 0 || H <= 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (K <= 0 || K > 256 || K % 32 != 0 || V <= 0 || V % llattn::GS_VC != 0 || L <= 0 || L > 32) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (carry_level < 0 || carry_level >= L) return LLATTN_ERR_TOO_FEW_LEVELS;
    if (!states || !q || !k || !v || !beta || !g || !lambda || !o) return LLATTN_ERR_NULL;
    using bf = __nv_bfloat16;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)(B * H * (V / llattn::GS_VC));
#define LLATTN_GDN_STEP(MAXL, RPT)                                                                                          \
    llattn::gdn_step_kernel<MAXL, RPT><<<grid, 256, 0, st>>>(states, (const bf*)q, (const bf*)k, (const bf*)v, (const bf*)beta, g, \
                                                             (const bf*)lambda, (bf*)o, H, K, V, L, carry_level)
    const int rpt = K / 32;
    if (L <= 16) {
        switch (rpt) {
            case 1: LLATTN_GDN_STEP(16, 1); break;
            case 2: LLATTN_GDN_STEP(16, 2); break;
            case 3: LLATTN_GDN_STEP(16, 3); break;
            case 4: LLATTN_GDN_STEP(16, 4); break;
            case 6: LLATTN_GDN_STEP(16, 6); break;
            case 8: LLATTN_GDN_STEP(16, 8); break;
            default: return LLATTN_ERR_UNSUPPORTED_SHAPE;
        }
    } else {
        switch (rpt) {
            case 2: LLATTN_GDN_STEP(32, 2); break;
            case 4: LLATTN_GDN_STEP(32, 4); break;
            default: return LLATTN_ERR_UNSUPPORTED_SHAPE;
        }
    }
#undef LLATTN_GDN_STEP
    LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}
