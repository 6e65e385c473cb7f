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
 * h / (H/G).  Constraints: T % 64 == 0, K in {64,128}, V == 64, H % G == 0,
 * L >= 7 + ceil(log2(T/64)), L <= 32 (the reference's checks: hattention/chunkwise.py:1140-1153,
 * 1211-1214).
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

/* Library / ABI version, for the loader's sanity check. */
int llattn_version(void);
/* Chunk length the kernels are built for (64, as hattention/kernel.py:355-356 fixes it). */
int llattn_chunk(void);

/* Log-linear Mamba-2 forward.  Replaces hattention.chunkwise.chunkwise_fwd
 * (hattention/chunkwise.py:1118-1275) with output_final_state=False: writes o and the in-chunk
 * inclusive cumulative sum of g (the reference returns both). */
size_t llattn_mamba2_fwd_workspace_bytes(int B, int T, int H, int G, int K, int V, int L);
int llattn_mamba2_fwd(const void* q, const void* k, const void* v, const float* g, const void* lambda,
                      void* o, float* g_cum, void* workspace, size_t workspace_bytes,
                      int B, int T, int H, int G, int K, int V, int L, void* stream);

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

#ifdef __cplusplus
}
#endif
#endif /* LLATTN_H_ */
