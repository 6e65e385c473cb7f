// Row-wise L2 normalisation of q / k and its backward for sm_100a (HBM-bound, one pass each).
//
// Reference being replaced: fla.modules.l2norm.l2norm_fwd / l2norm_bwd as called around the Gated
// DeltaNet drivers (hattention/kernel.py:20-29, 110-111, 224-225):
//     y  = bf16(bf16(x * rsqrt(sum x^2 + eps)) * scale)
//     dx = bf16(((dy * scale) - yhat (yhat . (dy * scale))) * rstd),   yhat = x * rstd in fp32
// A row (D <= 256 elements, D % 8 == 0) is handled by LPR lanes holding eight elements each.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/llattn.h"
#include "launch_count.h"

namespace llattn {

template <int LPR>
__global__ void __launch_bounds__(256) l2norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                         long rows, int D, float scale, float eps) {
    const int lane = threadIdx.x % LPR;
    const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    const bool active = row < rows && lane * 8 < D;
    float f[8];
    float ss = 0.f;
    if (active) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + row * D + lane * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __bfloat162float(h[i].x);
            f[2 * i + 1] = __bfloat162float(h[i].y);
            ss += f[2 * i] * f[2 * i] + f[2 * i + 1] * f[2 * i + 1];
        }
    }
#pragma unroll
    for (int d = LPR / 2; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if (active) {
        const float rstd = rsqrtf(ss + eps);
        uint4 out;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 n = __floats2bfloat162_rn(f[2 * i] * rstd, f[2 * i + 1] * rstd);
            o[i] = __floats2bfloat162_rn(__bfloat162float(n.x) * scale, __bfloat162float(n.y) * scale);
        }
        *reinterpret_cast<uint4*>(y + row * D + lane * 8) = out;
    }
}

template <int LPR>
__global__ void __launch_bounds__(256) l2norm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ dy,
                                                         __nv_bfloat16* __restrict__ dx, long rows, int D, float scale, float eps) {
    const int lane = threadIdx.x % LPR;
    const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    const bool active = row < rows && lane * 8 < D;
    float f[8], g[8];
    float ss = 0.f, dot = 0.f;
    if (active) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + row * D + lane * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float4 g0 = *reinterpret_cast<const float4*>(dy + row * D + lane * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(dy + row * D + lane * 8 + 4);
        g[0] = g0.x * scale; g[1] = g0.y * scale; g[2] = g0.z * scale; g[3] = g0.w * scale;
        g[4] = g1.x * scale; g[5] = g1.y * scale; g[6] = g1.z * scale; g[7] = g1.w * scale;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __bfloat162float(h[i].x);
            f[2 * i + 1] = __bfloat162float(h[i].y);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            ss += f[i] * f[i];
            dot += f[i] * g[i];
        }
    }
#pragma unroll
    for (int d = LPR / 2; d > 0; d >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, d);
        dot += __shfl_xor_sync(0xffffffffu, dot, d);
    }
    if (active) {
        const float rstd = rsqrtf(ss + eps);
        const float yd = dot * rstd * rstd;          // (yhat . g) * rstd, with yhat = x rstd
        uint4 out;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            o[i] = __floats2bfloat162_rn((g[2 * i] - f[2 * i] * yd) * rstd, (g[2 * i + 1] - f[2 * i + 1] * yd) * rstd);
        *reinterpret_cast<uint4*>(dx + row * D + lane * 8) = out;
    }
}

}  // namespace llattn

extern "C" {

static int l2norm_check(const void* a, const void* b, long rows, int D) {
    if (rows <= 0 || D <= 0 || D > 256 || D % 8 != 0) return LLATTN_ERR_UNSUPPORTED_SHAPE;
    if (!a || !b) return LLATTN_ERR_NULL;
    return 0;
}

int llattn_l2norm_fwd(const void* x, void* y, long rows, int D, float scale, void* stream) {
    int rc = l2norm_check(x, y, rows, D);
    if (rc != 0) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const __nv_bfloat16* xi = (const __nv_bfloat16*)x;
    __nv_bfloat16* yo = (__nv_bfloat16*)y;
    const int lpr = D <= 64 ? 8 : (D <= 128 ? 16 : 32);
    const long blocks = (rows * lpr + 255) / 256;
    if (lpr == 8) { llattn::l2norm_fwd_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(xi, yo, rows, D, scale, 1e-6f); LLATTN_LAUNCHED(); }
    else if (lpr == 16) { llattn::l2norm_fwd_kernel<16><<<(unsigned)blocks, 256, 0, st>>>(xi, yo, rows, D, scale, 1e-6f); LLATTN_LAUNCHED(); }
    else { llattn::l2norm_fwd_kernel<32><<<(unsigned)blocks, 256, 0, st>>>(xi, yo, rows, D, scale, 1e-6f); LLATTN_LAUNCHED(); }
    return (int)cudaGetLastError();
}

int llattn_l2norm_bwd(const void* x, const float* dy, void* dx, long rows, int D, float scale, void* stream) {
    int rc = l2norm_check(x, dx, rows, D);
    if (rc != 0) return rc;
    if (!dy) return LLATTN_ERR_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    const __nv_bfloat16* xi = (const __nv_bfloat16*)x;
    __nv_bfloat16* o = (__nv_bfloat16*)dx;
    const int lpr = D <= 64 ? 8 : (D <= 128 ? 16 : 32);
    const long blocks = (rows * lpr + 255) / 256;
    if (lpr == 8) { llattn::l2norm_bwd_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(xi, dy, o, rows, D, scale, 1e-6f); LLATTN_LAUNCHED(); }
    else if (lpr == 16) { llattn::l2norm_bwd_kernel<16><<<(unsigned)blocks, 256, 0, st>>>(xi, dy, o, rows, D, scale, 1e-6f); LLATTN_LAUNCHED(); }
    else { llattn::l2norm_bwd_kernel<32><<<(unsigned)blocks, 256, 0, st>>>(xi, dy, o, rows, D, scale, 1e-6f); LLATTN_LAUNCHED(); }
    return (int)cudaGetLastError();
}

}  // extern "C"
