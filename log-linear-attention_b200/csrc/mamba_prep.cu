// Element-wise preparation of the log-linear Mamba-2 layer call and its backward for sm_100a (HBM-bound;
// one pass over the (B,T,H,.) tensors per direction instead of about six).
//
// Reference being replaced: the torch ops around the kernel in hmamba_chunk_scan_combined
// (hattention/mamba_apis.py:346-366, 401-402) and compute_lambda (:70-85):
//     dt  = softplus(dt_raw + dt_bias)          v = x * dt           g = A * dt
//     lam = softplus(L * dl) | exp(-exp(L) softplus(dl)) | L * dl    y = o + D * x
// Rounding points follow torch's type promotion for bf16 activations with fp32 parameters (the
// products are fp32 there): dt and g stay fp32, v and lam are rounded once to bf16 (the cast at the
// kernel boundary, hattention/kernel.py), y = o + D x is fp32 or bf16 as the caller asks.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/llattn.h"
#include "launch_count.h"

namespace llattn {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// LPR lanes share one (b,t,h) row; each lane owns 8 consecutive elements of the P-wide row and the
// lambda columns lane, lane + LPR, ...
template <int LPR, int MODE>
__global__ void __launch_bounds__(256) m2_prep_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dt_raw,
                                                          const float* __restrict__ dt_bias, const float* __restrict__ A,
                                                          const __nv_bfloat16* __restrict__ dl, const float* __restrict__ Lp,
                                                          __nv_bfloat16* __restrict__ v, float* __restrict__ g, __nv_bfloat16* __restrict__ lam,
                                                          long rows, int H, int P, int L) {
    const int lane = threadIdx.x % LPR;
    const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    if (row >= rows) return;
    const int h = (int)(row % H);
    float t = __bfloat162float(dt_raw[row]);
    if (dt_bias) t += dt_bias[h];
    const float dt = softplus_f(t);
    if (lane == 0) g[row] = A[h] * dt;
    if (lane * 8 < P) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + row * P + lane * 8);
        const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint4 out;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(__bfloat162float(hx[i].x) * dt, __bfloat162float(hx[i].y) * dt);
        *reinterpret_cast<uint4*>(v + row * P + lane * 8) = out;
    }
    for (int j = lane; j < L; j += LPR) {
        const float lp = Lp[h * L + j], d = __bfloat162float(dl[row * L + j]);
        float r;
        if (MODE == 0) r = softplus_f(lp * d);
        else if (MODE == 1) r = __expf(-__expf(lp) * softplus_f(d));
        else r = lp * d;
        lam[row * L + j] = __float2bfloat16(r);
    }
}

// gradients: dx = dv * dt (+ D * dy), d dt_raw = (sum_p dv x + A dg) sigmoid(dt_raw + bias), d dl, and the
// parameter sums dA, d dt_bias, dD (H) and dL (H,L) through shared-memory partials and one global atomic
// per CTA and entry.
template <int LPR, int MODE>
__global__ void __launch_bounds__(256) m2_prep_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dt_raw,
                                                          const float* __restrict__ dt_bias, const float* __restrict__ A,
                                                          const __nv_bfloat16* __restrict__ dl, const float* __restrict__ Lp,
                                                          const float* __restrict__ D, const __nv_bfloat16* __restrict__ dv,
                                                          const float* __restrict__ dg, const float* __restrict__ dlam,
                                                          const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                                                          __nv_bfloat16* __restrict__ ddt, __nv_bfloat16* __restrict__ ddl,
                                                          float* __restrict__ dA, float* __restrict__ dbias, float* __restrict__ dLp,
                                                          float* __restrict__ dD, long rows, int H, int P, int L) {
    extern __shared__ float sacc[];            // [H] dA | [H] dbias | [H] dD | [H*L] dL
    float* sA = sacc;
    float* sB = sA + H;
    float* sD = sB + H;
    float* sL = sD + H;
    for (int i = threadIdx.x; i < 3 * H + H * L; i += blockDim.x) sacc[i] = 0.f;
    __syncthreads();
    const int lane = threadIdx.x % LPR;
    const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    const bool act = row < rows;
    const int h = act ? (int)(row % H) : 0;
    float t = 0.f, dt = 0.f, dot = 0.f, dsum = 0.f;
    if (act) {
        t = __bfloat162float(dt_raw[row]);
        if (dt_bias) t += dt_bias[h];
        dt = softplus_f(t);
        if (lane * 8 < P) {
            const uint4 rx = *reinterpret_cast<const uint4*>(x + row * P + lane * 8);
            const uint4 rv = *reinterpret_cast<const uint4*>(dv + row * P + lane * 8);
            uint4 ry = make_uint4(0, 0, 0, 0);
            const float dcoef = D ? D[h] : 0.f;
            if (D) ry = *reinterpret_cast<const uint4*>(dy + row * P + lane * 8);
            const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx);
            const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&rv);
            const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&ry);
            uint4 out;
            __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x0 = __bfloat162float(hx[i].x), x1 = __bfloat162float(hx[i].y);
                const float v0 = __bfloat162float(hv[i].x), v1 = __bfloat162float(hv[i].y);
                const float y0 = __bfloat162float(hy[i].x), y1 = __bfloat162float(hy[i].y);
                dot += v0 * x0 + v1 * x1;
                dsum += y0 * x0 + y1 * x1;
                o[i] = __floats2bfloat162_rn(v0 * dt + dcoef * y0, v1 * dt + dcoef * y1);
            }
            *reinterpret_cast<uint4*>(dx + row * P + lane * 8) = out;
        }
    }
#pragma unroll
    for (int d = LPR / 2; d > 0; d >>= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, d);
        dsum += __shfl_xor_sync(0xffffffffu, dsum, d);
    }
    if (act) {
        if (lane == 0) {
            const float dgv = dg[row];
            const float d_dt = dot + A[h] * dgv;
            const float d_raw = d_dt * (t > 20.f ? 1.f : sigmoid_f(t));
            ddt[row] = __float2bfloat16(d_raw);
            atomicAdd(&sA[h], dgv * dt);
            atomicAdd(&sB[h], d_raw);
            if (D) atomicAdd(&sD[h], dsum);
        }
        for (int j = lane; j < L; j += LPR) {
            const float lp = Lp[h * L + j], d = __bfloat162float(dl[row * L + j]);
            const float gl = dlam[row * L + j];
            float g_dl, g_lp;
            if (MODE == 0) {
                const float a = lp * d;
                const float s = a > 20.f ? 1.f : sigmoid_f(a);
                g_dl = gl * s * lp;
                g_lp = gl * s * d;
            } else if (MODE == 1) {
                const float el = __expf(lp), sp = softplus_f(d);
                const float r = __expf(-el * sp);
                g_dl = -gl * r * el * (d > 20.f ? 1.f : sigmoid_f(d));
                g_lp = -gl * r * el * sp;
            } else {
                g_dl = gl * lp;
                g_lp = gl * d;
            }
            ddl[row * L + j] = __float2bfloat16(g_dl);
            atomicAdd(&sL[h * L + j], g_lp);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        atomicAdd(&dA[i], sA[i]);
        if (dbias) atomicAdd(&dbias[i], sB[i]);
        if (D) atomicAdd(&dD[i], sD[i]);
    }
    for (int i = threadIdx.x; i < H * L; i += blockDim.x) atomicAdd(&dLp[i], sL[i]);
}

template <int LPR, bool F32OUT>
__global__ void __launch_bounds__(256) m2_residual_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ D, void* __restrict__ y, long rows, int H, int P) {
    const int lane = threadIdx.x % LPR;
    const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    if (row >= rows || lane * 8 >= P) return;
    const float d = D[row % H];
    const uint4 ro = *reinterpret_cast<const uint4*>(o + row * P + lane * 8);
    const uint4 rx = *reinterpret_cast<const uint4*>(x + row * P + lane * 8);
    const __nv_bfloat162* ho = reinterpret_cast<const __nv_bfloat162*>(&ro);
    const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx);
    float r[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        r[2 * i] = __bfloat162float(ho[i].x) + __bfloat162float(hx[i].x) * d;
        r[2 * i + 1] = __bfloat162float(ho[i].y) + __bfloat162float(hx[i].y) * d;
    }
    if (F32OUT) {
        float* yo = reinterpret_cast<float*>(y) + row * P + lane * 8;
        *reinterpret_cast<float4*>(yo) = make_float4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<float4*>(yo + 4) = make_float4(r[4], r[5], r[6], r[7]);
    } else {
        uint4 out;
        __nv_bfloat162* w = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = __floats2bfloat162_rn(r[2 * i], r[2 * i + 1]);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(y) + row * P + lane * 8) = out;
    }
}

static int lanes_per_row(int P) { return P <= 32 ? 4 : (P <= 64 ? 8 : (P <= 128 ? 16 : 32)); }

}  // namespace llattn

extern "C" {

static int prep_check(long rows, int H, int P, int L, int mode) {
    if (rows <= 0 || H <= 0 || rows % H != 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (P <= 0 || P > 256 || P % 8 != 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (L <= 0 || L > 64 || mode < 0 || mode > 2) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    return 0;
}

#define LLATTN_PREP_DISPATCH(KERN, LPRV, MODEV, ...)                                              \
    do {                                                                                          \
        if (MODEV == 0) KERN<LPRV, 0> __VA_ARGS__;                                                \
        else if (MODEV == 1) KERN<LPRV, 1> __VA_ARGS__;                                           \
        else KERN<LPRV, 2> __VA_ARGS__;                                                           \
    } while (0)

int llattn_mamba2_prep_fwd(const void* x, const void* dt_raw, const float* dt_bias, const float* A, const void* dl, const float* Lp,
                           void* v, float* g, void* lambda, long rows, int H, int P, int L, int lambda_mode, void* stream) {
    int rc = prep_check(rows, H, P, L, lambda_mode);
    if (rc != 0) return rc;
    if (!x || !dt_raw || !A || !dl || !Lp || !v || !g || !lambda) return LLATTN_ERR_NULL;
    using bf = __nv_bfloat16;
    cudaStream_t st = (cudaStream_t)stream;
    const int lpr = llattn::lanes_per_row(P);
    const unsigned blocks = (unsigned)((rows * lpr + 255) / 256);
#define ARGS_F <<<blocks, 256, 0, st>>>((const bf*)x, (const bf*)dt_raw, dt_bias, A, (const bf*)dl, Lp, (bf*)v, g, (bf*)lambda, rows, H, P, L)
    if (lpr == 4) LLATTN_PREP_DISPATCH(llattn::m2_prep_fwd_kernel, 4, lambda_mode, ARGS_F);
    else if (lpr == 8) LLATTN_PREP_DISPATCH(llattn::m2_prep_fwd_kernel, 8, lambda_mode, ARGS_F);
    else if (lpr == 16) LLATTN_PREP_DISPATCH(llattn::m2_prep_fwd_kernel, 16, lambda_mode, ARGS_F);
    else LLATTN_PREP_DISPATCH(llattn::m2_prep_fwd_kernel, 32, lambda_mode, ARGS_F);
#undef ARGS_F
    LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

int llattn_mamba2_prep_bwd(const void* x, const void* dt_raw, const float* dt_bias, const float* A, const void* dl, const float* Lp,
                           const float* D, const void* dv, const float* dg, const float* dlambda, const void* dy,
                           void* dx, void* ddt, void* ddl, float* dA, float* dbias, float* dLp, float* dD,
                           long rows, int H, int P, int L, int lambda_mode, void* stream) {
    int rc = prep_check(rows, H, P, L, lambda_mode);
    if (rc != 0) return rc;
    if (!x || !dt_raw || !A || !dl || !Lp || !dv || !dg || !dlambda || !dx || !ddt || !ddl || !dA || !dLp) return LLATTN_ERR_NULL;
    if (D && (!dy || !dD)) return LLATTN_ERR_NULL;
    if (dt_bias && !dbias) return LLATTN_ERR_NULL;
    using bf = __nv_bfloat16;
    cudaStream_t st = (cudaStream_t)stream;
    const int lpr = llattn::lanes_per_row(P);
    const unsigned blocks = (unsigned)((rows * lpr + 255) / 256);
    const size_t sm = (size_t)(3 * H + H * L) * sizeof(float);
    if (sm > 48 * 1024) return LLATTN_ERR_UNSUPPORTED_SHAPE;
#define ARGS_B <<<blocks, 256, sm, st>>>((const bf*)x, (const bf*)dt_raw, dt_bias, A, (const bf*)dl, Lp, D, (const bf*)dv, dg, dlambda, \
                                         (const bf*)dy, (bf*)dx, (bf*)ddt, (bf*)ddl, dA, dt_bias ? dbias : nullptr, dLp, dD, rows, H, P, L)
    if (lpr == 4) LLATTN_PREP_DISPATCH(llattn::m2_prep_bwd_kernel, 4, lambda_mode, ARGS_B);
    else if (lpr == 8) LLATTN_PREP_DISPATCH(llattn::m2_prep_bwd_kernel, 8, lambda_mode, ARGS_B);
    else if (lpr == 16) LLATTN_PREP_DISPATCH(llattn::m2_prep_bwd_kernel, 16, lambda_mode, ARGS_B);
    else LLATTN_PREP_DISPATCH(llattn::m2_prep_bwd_kernel, 32, lambda_mode, ARGS_B);
#undef ARGS_B
    LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

int llattn_mamba2_residual(const void* o, const void* x, const float* D, void* y, int y_is_f32, long rows, int H, int P, void* stream) {
    int rc = prep_check(rows, H, P, 1, 0);
    if (rc != 0) return rc;
    if (!o || !x || !D || !y) return LLATTN_ERR_NULL;
    using bf = __nv_bfloat16;
    cudaStream_t st = (cudaStream_t)stream;
    const int lpr = llattn::lanes_per_row(P);
    const unsigned blocks = (unsigned)((rows * lpr + 255) / 256);
#define RES(LPRV)                                                                                                          \
    do {                                                                                                                   \
        if (y_is_f32) llattn::m2_residual_kernel<LPRV, true><<<blocks, 256, 0, st>>>((const bf*)o, (const bf*)x, D, y, rows, H, P);   \
        else llattn::m2_residual_kernel<LPRV, false><<<blocks, 256, 0, st>>>((const bf*)o, (const bf*)x, D, y, rows, H, P);           \
    } while (0)
    if (lpr == 4) RES(4);
    else if (lpr == 8) RES(8);
    else if (lpr == 16) RES(16);
    else RES(32);
#undef RES
    LLATTN_LAUNCHED();
    return (int)cudaGetLastError();
}

}  // extern "C"
