/* C ABI of the B200 (sm_100a) chunkwise log-linear attention library, libllattn.so.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream (passed as void*), launches
 * asynchronously on that stream, never synchronises the device and never allocates: scratch
 * memory is provided by the caller (size from the matching *_workspace_bytes call; 256-byte
 * aligned).  Return value: 0 on success, a negative LLATTN_ERR_* code for rejected arguments,
 * or a positive cudaError_t value if a launch failed.
 *
 * Tensor layouts (all contiguous, "sequence first", as the reference passes them with
 * head_first=False): q,k (B,T,G,K) bf16; v,o,do,dv (B,T,H,V) bf16; g,dg (B,T,H) fp32;
 * lambda (B,T,H,L) bf16; dlambda (B,T,H,L) fp32; dq,dk (B,T,G,K) bf16.  Head h uses q/k group
 * h / (H/G).  Constraints: T % 64 == 0, T <= 524288 (the scans over 512-token segments hold ten segment
 * levels), K in {64,128}, V == 64, H % G == 0, L >= 7 + ceil(log2(T/64)), L <= 32 (the reference's
 * checks: hattention/chunkwise.py:1140-1153, 1211-1214).
 *
 * Status word.  The first 4 bytes of every workspace are a status word that the call clears and that a
 * kernel sets to 1 if one of its bounded waits (on a TMA transfer or on the tensor core) ran out; the
 * outputs of such a call are not valid.  A launch cannot report this through its return value (nothing
 * waits for the GPU), so callers that want to know read the word after synchronising:
 * llattn_workspace_status, or llattn_static_scratch_status for llattn_mamba2_fwd_static.
 */
#ifndef LLATTN_H_
#define LLATTN_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLATTN_ERR_UNSUPPORTED_SHAPE (-1)   /* K / V / L outside the compiled set            */
#define LLATTN_ERR_BAD_LENGTH (-2)          /* T not a multiple of the 64-token chunk        */
#define LLATTN_ERR_TOO_FEW_LEVELS (-3)      /* L < 7 + ceil(log2(T/64))                      */
#define LLATTN_ERR_BAD_GROUPS (-4)          /* H % G != 0                                    */
#define LLATTN_ERR_WORKSPACE (-5)           /* workspace NULL, misaligned or too small       */
#define LLATTN_ERR_NULL (-6)                /* a required pointer is NULL                    */
#define LLATTN_ERR_STATIC_SCRATCH (-7)      /* problem needs more than LLATTN_STATIC_SCRATCH_BYTES */
#define LLATTN_ERR_TENSOR_MAP (-8)          /* the driver refused a TMA tensor map for these pointers */

/* Size of the built-in scratch array used by llattn_mamba2_fwd_static (16 MiB). */
#define LLATTN_STATIC_SCRATCH_BYTES (16u << 20)

/* Library / ABI version, for the loader's sanity check. */
int llattn_version(void);
/* Number of kernels this library has launched in the process so far (all entry points, all threads). */
unsigned long long llattn_kernel_launches(void);
/* Copies the status word of `workspace` (a workspace that an earlier call on `stream` used) to *status_host
 * and returns after the stream has drained: unlike the compute entry points this one synchronises.
 * 0 = every wait completed, 1 = a kernel gave up and the call's outputs must be discarded.  (No counterpart
 * in the reference, whose Triton kernels have no bounded waits.) */
int llattn_workspace_status(const void* workspace, int* status_host, void* stream);
/* Chunk length the kernels are built for (64, as hattention/kernel.py:355-356 fixes it). */
int llattn_chunk(void);

/* Log-linear Mamba-2 forward.  Replaces hattention.chunkwise.chunkwise_fwd
 * (hattention/chunkwise.py:1118-1275) with output_final_state=False: writes o and the in-chunk
 * inclusive cumulative sum of g (the reference returns both). */
size_t llattn_mamba2_fwd_workspace_bytes(int B, int T, int H, int G, int K, int V, int L);
int llattn_mamba2_fwd(const void* q, const void* k, const void* v, const float* g, const void* lambda,
                      void* o, float* g_cum, void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int G, int K, int V, int L, void* stream);

/* Forward for callers that cannot hand the library a scratch buffer.  (No counterpart in the
 * reference: its drivers allocate with torch on every call.)
 *
 * Who needs it: code that must not call cudaMalloc / cudaFree or any allocator behind them at the
 * point where the operator runs - for instance a serving loop that has handed all device memory to
 * its own pool, a host that embeds this library without torch, or a latency-critical section where
 * the device-wide synchronisation of cudaMalloc is not acceptable - and that has no spare buffer
 * of its own to pass as `workspace`.
 *
 * Same computation and results as llattn_mamba2_fwd, but the segment-level scratch lives in an
 * array compiled into the library (LLATTN_STATIC_SCRATCH_BYTES = 16 MiB of device memory on every
 * GPU that loads the library, held until the process exits).  The call allocates and frees
 * nothing.  Shapes whose scratch need (llattn_mamba2_fwd_workspace_bytes) exceeds the array are
 * rejected with LLATTN_ERR_STATIC_SCRATCH; at T = 4096, K = 128, V = 64 the need is 1.125 MiB per
 * (batch, head), so the array serves B*H <= 14 there.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress) for
 * the device that is current at that moment and caches it; make that first call with the right
 * device current and before starting any stream capture.  All calls on one device share the one
 * array, and it keeps whatever the previous call left in it (the kernels overwrite every element
 * before reading it, so no clearing is needed): two calls whose kernels can overlap on the GPU
 * - different streams, or different host threads - race on it and must be serialised by the caller.
 * (Two host threads that make the FIRST call on a device at the same time both store the same looked-up
 * address into the cache; that is harmless, the race on the array itself is not.)
 * llattn_static_scratch_status reads the status word of the array on the current device (see "Status
 * word" above) after synchronising `stream`. */
size_t llattn_static_scratch_bytes(void);
int llattn_static_scratch_status(int* status_host, void* stream);
int llattn_mamba2_fwd_static(const void* q, const void* k, const void* v, const float* g, const void* lambda,
                             void* o, float* g_cum, int B, int T, int H, int G, int K, int V, int L, void* stream);

/* Log-linear Mamba-2 backward.  Replaces hattention.chunkwise.chunkwise_bwd
 * (hattention/chunkwise.py:1286-1597).  `g_cum` is the in-chunk cumulative sum that the forward
 * returned (the reference saves that tensor for backward, hattention/kernel.py:86,125); dg is the
 * gradient w.r.t. the raw per-token g.  dq and dk are already summed over the heads of each group
 * (chunkwise.py:1583-1591). */
size_t llattn_mamba2_bwd_workspace_bytes(int B, int T, int H, int G, int K, int V, int L);
int llattn_mamba2_bwd(const void* q, const void* k, const void* v, const float* g_cum, const void* lambda,
                      const void* d_o, void* dq, void* dk, void* dv, float* dg, float* dlambda,
                      void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int G, int K, int V, int L, void* stream);

/* Same as llattn_mamba2_bwd, but the segment-level states of the forward pass are read from the
 * workspace that the matching llattn_mamba2_fwd call used (unmodified since), instead of being
 * recomputed from k, v, g (two launches less).  fwd_workspace == NULL behaves exactly like
 * llattn_mamba2_bwd.  No counterpart in the reference, whose autograd function keeps only the inputs
 * (hattention/kernel.py:125) and recomputes the states per level (hattention/chunkwise.py:1464-1490). */
int llattn_mamba2_bwd_saved(const void* q, const void* k, const void* v, const float* g_cum, const void* lambda,
                            const void* d_o, void* dq, void* dk, void* dv, float* dg, float* dlambda,
                            void* workspace, size_t workspace_bytes, const void* fwd_workspace, size_t fwd_workspace_bytes,
                            int B, int T, int H, int G, int K, int V, int L, void* stream);

/* Element-wise preparation of the log-linear Mamba-2 layer call, its backward, and the D residual.
 * Replace the torch ops around the kernel in hmamba_chunk_scan_combined (hattention/mamba_apis.py:
 * 346-366, 401-402) and compute_lambda (hattention/mamba_apis.py:70-85).  rows = B*T*H; x, v, dv, dx, dy, o, y
 * are bf16 (rows, P); dt_raw, ddt bf16 (rows); dl, lambda, ddl bf16 (rows, L); g, dg fp32 (rows); dlambda fp32
 * (rows, L); A, dt_bias (may be NULL), D (may be NULL) fp32 (H); Lp fp32 (H, L).  lambda_mode: 0 "positive"
 * softplus(Lp dl), 1 "bounded" exp(-exp(Lp) softplus(dl)), 2 none Lp dl.
 *   fwd: dt = softplus(dt_raw + dt_bias); v = x dt; g = A dt; lambda = f(Lp, dl)
 *   bwd: dx = dv dt + D dy; ddt, ddl; dA, dbias, dD (H) and dLp (H, L) are ACCUMULATED with atomics into
 *        buffers the caller has cleared
 *   residual: y = o + D x, y fp32 (y_is_f32 != 0; what torch's promotion gives for fp32 D) or bf16
 * Constraints: P % 8 == 0, P <= 256, L <= 64. */
int llattn_mamba2_prep_fwd(const void* x, const void* dt_raw, const float* dt_bias, const float* A, const void* dl, const float* Lp,
                           void* v, float* g, void* lambda, long rows, int H, int P, int L, int lambda_mode, void* stream);
int llattn_mamba2_prep_bwd(const void* x, const void* dt_raw, const float* dt_bias, const float* A, const void* dl, const float* Lp,
                           const float* D, const void* dv, const float* dg, const float* dlambda, const void* dy,
                           void* dx, void* ddt, void* ddl, float* dA, float* dbias, float* dLp, float* dD,
                           long rows, int H, int P, int L, int lambda_mode, void* stream);
int llattn_mamba2_residual(const void* o, const void* x, const float* D, void* y, int y_is_f32, long rows, int H, int P, void* stream);

/* Prefill hand-off: the level states after T tokens, states fp32 (B,H,K,V,L), every level written.
 * Level 0 is k_m v_m^T for the last token m = T-1; for each set bit j of m, level j+1 holds the 2^j
 * tokens that follow the buckets of the higher set bits, each decayed to token m; other levels are zero.
 * Replaces the state side of hattention_prefill (hattention/kernel.py:470-560): the final states `ht` of
 * chunk_fwd_kernel_h (hattention/chunkwise.py:171-173, 278-280) for the inter-chunk levels together with
 * postprocess_prefill_hstate_ (hattention/kernel.py:378-466) for the levels inside the last chunk and its
 * clearing of unpopulated levels.  k (B,T,G,K), v (B,T,H,V) bf16, g (B,T,H) fp32 raw log decay.  Any T >= 1;
 * K in {64,128}, V == 64, bit_length(T-1) + 1 <= L <= 32. */
int llattn_mamba2_final_state(const void* k, const void* v, const float* g, float* states,
                              int B, int T, int H, int G, int K, int V, int L, void* stream);

/* One decode step (hattention_step, hattention/kernel.py:563-633, with HState.cascade_weak / insert and
 * step_output, hattention/recurrent.py:42-54, 79-98, 134-166) for every (batch, head): levels 0..carry_level
 * are summed into level carry_level (the caller runs the cascade on the token counts, which are the same
 * for every sequence: carry_level is the first level that is not full), every level is multiplied by
 * exp(g), level 0 becomes k v^T, and o = q . sum_l lambda_l S_l.  states fp32 (B,H,K,V,L) updated in place;
 * q, k (B,G,K), v (B,H,V), lambda (B,H,L), o (B,H,V) bf16; g (B,H) fp32.  256 % V == 0, L <= 32. */
int llattn_mamba2_step(float* states, const void* q, const void* k, const void* v, const float* g, const void* lambda, void* o,
                       int B, int H, int G, int K, int V, int L, int carry_level, void* stream);

/* Log-linear Gated DeltaNet forward.  Replaces hattention.chunkwise_hgdn.chunkwise_fwd
 * (hattention/chunkwise_hgdn.py:566-788) with output_final_state=False.  q and k are per head,
 * (B,T,H,K), and must already be L2-normalised (q also scaled) as the reference's autograd
 * function does before the call (hattention/kernel.py:110-111); beta is (B,T,H) bf16; g is the raw
 * log decay.  Writes o, the in-chunk cumulative g, and the two 64x64 UT-transform inverses per
 * chunk, Aw and Au, as (B,T,H,64) bf16 (the reference returns and saves them for the backward).
 * Constraints: T % 64 == 0, K == 128, V in {64,128}, 7 + ceil(log2(T/64)) <= L <= 32, T <= 16384. */
size_t llattn_gdn_fwd_workspace_bytes(int B, int T, int H, int K, int V, int L);
int llattn_gdn_fwd(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                   void* o, float* g_cum, void* Aw, void* Au, void* workspace, size_t workspace_bytes,
                   int B, int T, int H, int K, int V, int L, void* stream);

/* Prompt pass of the log-linear Gated DeltaNet layer: llattn_gdn_fwd plus the level states a decoder continues
 * from.  `states` is fp32 (B,H,K,V,L), level innermost (the layout of the reference's HState,
 * hattention/recurrent.py:9-40); it is cleared and then, for every set bit j of NT - 1 (NT = T / 64), level
 * 7 + j receives the state of the block of 2^j chunks that the LAST chunk reads, i.e. the states as they stand
 * before the last 64 tokens.  The caller feeds those 64 tokens (and any tokens beyond T) through
 * llattn_gdn_step, which builds the levels inside the chunk.  Together the two replace hattention_prefill with
 * hstruct = GDELTA (hattention/kernel.py:469-560: chunkwise_fwd with output_final_state=True, then
 * postprocess_prefill_hstate_, :378-466).  Other arguments and constraints as llattn_gdn_fwd. */
int llattn_gdn_prefill(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                       void* o, float* g_cum, void* Aw, void* Au, float* states, void* workspace, size_t workspace_bytes,
                       int B, int T, int H, int K, int V, int L, void* stream);

/* One decode step of the log-linear Gated DeltaNet layer for every (batch, head).  Replaces hattention_step with
 * hstruct = GDELTA (hattention/kernel.py:563-633) after its l2norm / scale of q and k, i.e. HState.cascade_weak /
 * insert with the delta-rule gate and step_output (hattention/recurrent.py:42-54, 79-98, 134-166): levels
 * 0..carry_level are summed into level carry_level (the caller runs the cascade on the token counts), every
 * level becomes exp(g) (S - beta k (k^T S)), level 0 becomes beta k v^T, and o = q . sum_l lambda_l S_l.
 * states fp32 (B,H,K,V,L) updated in place, one pass over HBM; q, k (B,H,K) already normalised (q also scaled),
 * v (B,H,V), beta (B,H), lambda (B,H,L), o (B,H,V) bf16; g (B,H) fp32 log decay.
 * K % 32 == 0, K <= 256, V % 8 == 0, L <= 32 (K / 32 in {1,2,3,4,6,8}; {2,4} when L > 16). */
int llattn_gdn_step(float* states, const void* q, const void* k, const void* v, const void* beta, const float* g,
                    const void* lambda, void* o, int B, int H, int K, int V, int L, int carry_level, void* stream);

/* Log-linear Gated DeltaNet backward, first stage: everything that involves the inter-chunk level
 * states.  Replaces, inside hattention.chunkwise_hgdn.chunkwise_bwd (hattention/chunkwise_hgdn.py:
 * 799-1010), the per-level loop over chunk_gated_delta_rule_fwd_h (state recomputation),
 * chunk_gated_delta_rule_bwd_dhu (adjoint states) and the state-dependent parts of chunk_bwd_dqkwg /
 * chunk_bwd_dv_local.  Inputs are those the reference saves for its backward: q, k (normalised, as in
 * the forward), v, beta, the in-chunk cumulative g, lambda, Aw, Au, and d_o.  Per chunk, with
 * kd = k exp(gl - G), wd = w exp(G), qd = exp(G)(q - tril(q k^T) w), u as in the forward, writes the
 * gradients with respect to those chunk matrices, fp32 (B,T,H,K): d_qd, d_wd, d_kd; bf16 (B,T,H,V):
 * d_u; the part of the gradient of each chunk's total log decay that comes from the state decay,
 * d_gl fp32 (B,T/64,H); and columns 7 .. 7+ceil(log2(T/64))-1 of dlambda, fp32 (B,T,H,L) (other
 * columns are left untouched).  Same shape constraints as llattn_gdn_fwd. */
size_t llattn_gdn_bwd_levels_workspace_bytes(int B, int T, int H, int K, int V, int L);
int llattn_gdn_bwd_levels(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                          const void* Aw, const void* Au, const void* d_o, float* d_qd, float* d_wd, float* d_kd, void* d_u,
                          float* d_gl, float* dlambda, void* workspace, size_t workspace_bytes,
                          int B, int T, int H, int K, int V, int L, void* stream);

/* Log-linear Gated DeltaNet backward, complete.  Replaces hattention.chunkwise_hgdn.chunkwise_bwd
 * (hattention/chunkwise_hgdn.py:799-1010): the stage above followed by the chunk-local part
 * (gradients through kd, wd, qd, u, the UT transform, tril(q k^T) and the intra-chunk output).
 * Inputs as saved by the reference's autograd function (hattention/kernel.py:113-120): normalised
 * q, k, then v, beta, the in-chunk cumulative g, lambda, Aw, Au, and d_o (bf16 (B,T,H,V)).
 * Outputs are fp32: dq, dk (B,T,H,K) with respect to the NORMALISED q, k (the caller applies the
 * l2norm / scale backward as hattention/kernel.py:208-221 does), dv (B,T,H,V), dbeta, dg (B,T,H)
 * with respect to the raw g, dlambda (B,T,H,L; every column is written).  Same shape constraints
 * as llattn_gdn_fwd. */
size_t llattn_gdn_bwd_workspace_bytes(int B, int T, int H, int K, int V, int L);
int llattn_gdn_bwd(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                   const void* Aw, const void* Au, const void* d_o, float* dq, float* dk, float* dv, float* dbeta, float* dg,
                   float* dlambda, void* workspace, size_t workspace_bytes,
                   int B, int T, int H, int K, int V, int L, void* stream);

/* The same forward and backward with the forward's intermediates kept between the two calls, so that
 * the backward does not recompute them (the reference recomputes w, u and the level states in its
 * backward, hattention/chunkwise_hgdn.py:820-870; keeping them trades memory for about a fifth of the
 * step).  llattn_gdn_fwd_keep is llattn_gdn_fwd with a larger workspace that, on return, holds the
 * chunk matrices and every chunk's level states; the caller leaves it untouched and hands it to
 * llattn_gdn_bwd_kept as fwd_workspace.  Results are those of llattn_gdn_fwd / llattn_gdn_bwd. */
size_t llattn_gdn_fwd_keep_workspace_bytes(int B, int T, int H, int K, int V, int L);
int llattn_gdn_fwd_keep(const void* q, const void* k, const void* v, const void* beta, const float* g, const void* lambda,
                        void* o, float* g_cum, void* Aw, void* Au, void* workspace, size_t workspace_bytes,
                        int B, int T, int H, int K, int V, int L, void* stream);
size_t llattn_gdn_bwd_kept_workspace_bytes(int B, int T, int H, int K, int V, int L);
int llattn_gdn_bwd_kept(const void* q, const void* k, const void* v, const void* beta, const float* g_cum, const void* lambda,
                        const void* Aw, const void* Au, const void* d_o, float* dq, float* dk, float* dv, float* dbeta,
                        float* dg, float* dlambda, const void* fwd_workspace, size_t fwd_workspace_bytes, void* workspace,
                        size_t workspace_bytes, int B, int T, int H, int K, int V, int L, void* stream);
/* llattn_gdn_bwd_kept with dv written in bf16 (B,T,H,V), the dtype the reference's autograd function returns for bf16 v
 * (hattention/kernel.py:226: dv.to(v)): saves the caller a conversion pass over dv.  Same workspace size. */
int llattn_gdn_bwd_kept_bf16dv(const void* q, const void* k, const void* v, const void* beta, const float* g_cum,
                               const void* lambda, const void* Aw, const void* Au, const void* d_o, float* dq, float* dk,
                               void* dv_bf16, float* dbeta, float* dg, float* dlambda, const void* fwd_workspace,
                               size_t fwd_workspace_bytes, void* workspace, size_t workspace_bytes,
                               int B, int T, int H, int K, int V, int L, void* stream);

/* Row-wise L2 normalisation of q / k and its backward, as applied around the Gated DeltaNet drivers
 * when use_qk_l2norm_in_kernel is set.  Replace fla.modules.l2norm.l2norm_fwd / l2norm_bwd with the
 * scale folded in (hattention/kernel.py:20-29: l2norm_and_scale_fwd / l2norm_and_scale_bwd).
 *   fwd: y = bf16(bf16(x rsqrt(sum x^2 + 1e-6)) * scale)        x, y bf16 (rows, D)
 *   bwd: dx = bf16((g - yhat (yhat . g)) rstd), g = dy * scale   dy fp32 (rows, D), dx bf16
 * Constraints: D % 8 == 0, D <= 256. */
int llattn_l2norm_fwd(const void* x, void* y, long rows, int D, float scale, void* stream);
int llattn_l2norm_bwd(const void* x, const float* dy, void* dx, long rows, int D, float scale, void* stream);

/* Diagnostic: one 128 x N x kred bf16 tensor-core product (tcgen05.mma, accumulator in tensor
 * memory) per operand-layout combination used by the kernels: mode 0: D = A B^T with A [128][kred],
 * B [N][kred]; mode 1: D = A B with B [kred][N]; mode 2: D = A^T B with A [kred][128], B [kred][N].
 * D is [128][N] fp32.  Modes 10, 11, 12 are the same three products issued through the compile-time shaped
 * loops that the kernels use.  *err_flag is set to 1 if the tensor core did not signal completion within
 * the kernel's bounded wait.  (No counterpart in the reference; used by the test-suite.) */
int llattn_selftest_umma(const void* A, const void* B, float* D, int N, int kred, int mode, int* err_flag, void* stream);

/* Diagnostic: SM clock cycles from the issue of `reps` back-to-back 128 x N x kred products of one layout
 * combination (modes as above, operands resident in shared memory, accumulator in tensor memory) to their
 * completion, written to *cycles (device memory); issuers = 2 lets two warps issue `reps` products each at the
 * same time into separate accumulators.  (No counterpart in the reference.) */
int llattn_selftest_umma_cycles(int N, int kred, int mode, int reps, int issuers, long long* cycles, int* err_flag, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LLATTN_H_ */
