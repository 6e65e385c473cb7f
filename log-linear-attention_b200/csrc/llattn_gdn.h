// Internal launch parameters of the log-linear Gated DeltaNet kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/llattn.h"

namespace llattn {

constexpr int GDN_VS = 32;          // V columns per CTA of the sequential scans
constexpr int GDN_MAXLEV = 8;       // inter-chunk levels (T up to 64 * 2^8 = 16384)

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
    float* final_states;         // optional (B,H,K,V,L) fp32: level states as of the start of the last chunk (prefill hand-off)
    __nv_bfloat16* Aw;           // (B,T,H,64)  (I + A)^-1 rows, saved for the backward
    __nv_bfloat16* Au;           // (B,T,H,64)  (I + A*Gamma)^-1 rows
    // scratch written by the chunk preparation, read by the scan
    __nv_bfloat16* kd;           // (B,T,H,K)  k exp(gl - G)
    __nv_bfloat16* wd;           // (B,T,H,K)  w exp(G)
    __nv_bfloat16* qd;           // (B,T,H,K)  exp(G) (q - tril(q k^T) w)
    __nv_bfloat16* u;            // (B,T,H,V)
    __nv_bfloat16* wk;           // (B,NT*K,H,K)  (exp(gl) - 1) I - kd^T wd per chunk (tcgen05 scans; NULL: not produced)
    // backward
    const __nv_bfloat16* d_o;    // (B,T,H,V)
    __nv_bfloat16* hs;           // level states read by each chunk: [(b,h,slice)][chunk][level][K][32] (warp-MMA kernels) or
                                 // [(b,h,pair of slices)][chunk][level][K][64] (tcgen05 kernels); same size either way
    __nv_bfloat16* dhs;          // same layout: adjoints of the level states written by each chunk
    __nv_bfloat16* d_u;          // (B,T,H,V)
    __nv_bfloat16* dqd_neg;      // (B,T,H,K)  -(d_qd exp(G)) and
    float* d_grow;               // (B,T,H)    d_qd . qd + d_wd . wd - d_kd . kd, written by the tcgen05 level-gradient kernel for the
                                 //            chunk-local kernel (both null: that kernel derives them itself); d_gl then includes sum d_kd . kd
    float* d_qd;                 // (B,T,H,K)
    float* d_wd;                 // (B,T,H,K)
    float* d_kd;                 // (B,T,H,K)
    float* d_gl;                 // (B,NT,H)  gradient w.r.t. the chunk's total log decay, scan part
    float* dq;                   // (B,T,H,K) fp32 results
    float* dk;
    float* dv;                   // (B,T,H,V)
    __nv_bfloat16* dv_bf16;      // (B,T,H,V)  written instead of dv when not null
    float* dbeta;                // (B,T,H)
    float* dg;                   // (B,T,H)
    float* dl;                   // (B,T,H,L)
    int B, T, H, K, V, L;
    int NT, NLEV;
    int* err;                    // status word (first word of the call's workspace): set by a kernel whose bounded wait ran out
    // tensor maps of the chunk matrices (tcgen05 kernels; filled by their launchers)
    alignas(64) CUtensorMap tm_q, tm_k, tm_v, tm_qd, tm_wd, tm_kd, tm_wk, tm_u, tm_do, tm_hs, tm_dhs, tm_dqd, tm_dwd, tm_dkd;
};

bool gdn_bwd_levels_writes_row_terms(const GdnParams& p);
int gdn_fwd_dispatch(const GdnParams& p, cudaStream_t stream);
int gdn_fwd_keep_dispatch(const GdnParams& p, cudaStream_t stream);
int gdn_recompute_dispatch(const GdnParams& p, cudaStream_t stream);
int gdn_prep_tc_dispatch(const GdnParams& p, cudaStream_t stream);        // chunk preparation of the forward on tcgen05 (K = 128)
// tcgen05 scans (K = 128).  mode 0: forward, 1: forward that keeps the level states, 2: recomputation (states only)
int gdn_scan_tc_dispatch(const GdnParams& p, int mode, cudaStream_t stream);
int gdn_scan_bwd_tc_dispatch(const GdnParams& p, cudaStream_t stream);     // adjoint level states (d_u comes from the level-gradient kernel)
int gdn_bwd_scan_dispatch(const GdnParams& p, cudaStream_t stream);      // adjoint level states, d_u
int gdn_bwd_levels_dispatch(const GdnParams& p, cudaStream_t stream);    // d_qd, d_wd, d_kd, d_gl, dl (inter-chunk levels), d_u
int gdn_bwd_levels_tc_dispatch(const GdnParams& p, cudaStream_t stream); // the same on tcgen05 (reads the [K][64] tiles of the tcgen05 scans)
int gdn_bwd_chunk_dispatch(const GdnParams& p, cudaStream_t stream);     // dq, dk, dv, dbeta, dg, dl (intra-chunk levels)

}  // namespace llattn
