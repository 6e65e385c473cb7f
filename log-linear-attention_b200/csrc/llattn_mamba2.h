// Internal launch parameters shared by the log-linear Mamba-2 kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/llattn.h"

namespace llattn {

constexpr int M2_MLOW = 3;   // a segment is 2^M2_MLOW chunks (512 tokens)
constexpr int M2_MAX_LH = 10;   // segment levels held by the per-level scans over segments (T <= 512 * 2^10)

struct Mamba2Params {
    // tensor maps (64-column panels, 128 rows) for the tcgen05 kernels; valid only when those run
    alignas(64) CUtensorMap tm_q, tm_k, tm_v, tm_do;
    alignas(64) CUtensorMap tm_h0;             // level states of the segments as a (B*H*NS*LH*K, V) matrix
    alignas(64) CUtensorMap tm_dq, tm_dk;      // fp32 (B*T, G, K) accumulators, 32-column boxes (reduce-add)
    // inputs
    const __nv_bfloat16* q;      // (B,T,G,K)
    const __nv_bfloat16* k;      // (B,T,G,K)
    const __nv_bfloat16* v;      // (B,T,H,V)
    const float* g;              // (B,T,H) raw log decay
    const __nv_bfloat16* l;      // (B,T,H,L)
    const __nv_bfloat16* d_o;    // (B,T,H,V) upstream gradient (backward only)
    // outputs
    __nv_bfloat16* o;            // (B,T,H,V)
    float* g_cum;                // (B,T,H) in-chunk inclusive cumsum of g
    float* dq_acc;               // (B,T,G,K) fp32 accumulators (backward)
    float* dk_acc;               // (B,T,G,K)
    __nv_bfloat16* dv;           // (B,T,H,V)
    float* dl;                   // (B,T,H,L)
    float* wq;                   // (B,T,H)  accumulates q.dq - k.dk per token and head (backward)
    // segment-level scratch
    float* seg_F;                // (B,H,NS,K,V)
    float* seg_D;                // (B,H,NS)
    __nv_bfloat16* seg_H0;       // (B,H,NS,LH,K,V)
    __nv_bfloat16* o_hi;         // (B*H, NT/2, 8, 128, 8) high-level partial output, column-chunk major (tcgen05 chunk kernel)
    float* seg_dF;               // (B,H,NS,LH,K,V) reader summaries (backward)
    float* seg_dHf;              // (B,H,NS,K,V) gradient w.r.t. the segment summaries (backward)
    // per-chunk scalars from which the decay gradient across chunk boundaries is assembled
    float* Zc;                   // (B,H,NT,LZ)      reader side: sum_t lambda * dlambda per level
    float* Yc;                   // (B,H,NT,MLOW+1)  contributor side: <KV_c, adjoint state> per low level, + combined high
    float* Yseg;                 // (B,H,NS,LH)      contributor side per segment and high level
    int LZ;                      // MLOW + LH
    int* err;                    // device status word: set to 1 when a bounded wait on the tensor core gave up
    int B, T, H, G, K, V, L;
    int NT, NS, LH;
    int o_has_high;
    int lev_lo;                  // first segment level handled by one launch of the tensor-core high-level backward
    int reuse_states;            // backward: seg_D / seg_H0 come from the forward call, do not recompute them
};

int mamba2_fwd_dispatch(Mamba2Params p, cudaStream_t stream);
int mamba2_bwd_dispatch(Mamba2Params p, cudaStream_t stream);
// segment summaries and the per-level scan over segments only (needs NS > 1)
int mamba2_fwd_states_dispatch(Mamba2Params p, cudaStream_t stream);
// tcgen05 version of the chunk kernel (K = 128, V = 64, even number of chunks)
int mamba2_fwd_tc_launch(const Mamba2Params& p, cudaStream_t stream);
int mamba2_bwd1_tc_launch(const Mamba2Params& p, cudaStream_t stream);
int mamba2_bwd2_tc_launch(const Mamba2Params& p, cudaStream_t stream);
int mamba2_hi_bwd_tc_launch(const Mamba2Params& p, cudaStream_t stream);
int mamba2_seg_state_tc_launch(const Mamba2Params& p, cudaStream_t stream);
int mamba2_hi_out_tc_launch(const Mamba2Params& p, cudaStream_t stream);
extern std::atomic<int> g_use_tensor_core_path;   // test hook, see llattn_testing.h
void mamba2_uncumsum(const float* gc, float* g, long BT, int H, cudaStream_t stream);
int mamba2_dg(const Mamba2Params& p, float* dg, cudaStream_t stream);
void cast_f32_to_bf16(const float* src, void* dst, long n, cudaStream_t stream);

}  // namespace llattn
