// Internal launch parameters of the log-linear Gated DeltaNet kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/llattn.h"

namespace llattn {

struct GdnParams {
    // inputs (q, k already L2-normalised / scaled by the caller, one q/k per head)
    const __nv_bfloat16* q;      // (B,T,H,K)
    const __nv_bfloat16* k;      // (B,T,H,K)
    const __nv_bfloat16* v;      // (B,T,H,V)
    const __nv_bfloat16* beta;   // (B,T,H)
    const float* g;              // (B,T,H) raw log decay
    const __nv_bfloat16* l;      // (B,T,H,L)
    // outputs
    __nv_bfloat16* o;            // (B,T,H,V)
    float* g_cum;                // (B,T,H)
    __nv_bfloat16* Aw;           // (B,T,H,64)  (I + A)^-1 rows, saved for the backward
    __nv_bfloat16* Au;           // (B,T,H,64)  (I + A*Gamma)^-1 rows
    // scratch written by the chunk preparation, read by the scan
    __nv_bfloat16* kd;           // (B,T,H,K)  k exp(gl - G)
    __nv_bfloat16* wd;           // (B,T,H,K)  w exp(G)
    __nv_bfloat16* qd;           // (B,T,H,K)  exp(G) (q - tril(q k^T) w)
    __nv_bfloat16* u;            // (B,T,H,V)
    int B, T, H, K, V, L;
    int NT, NLEV;
};

int gdn_fwd_dispatch(const GdnParams& p, cudaStream_t stream);

}  // namespace llattn
