/* Entry points of libllattn.so that exist for the test-suite only.  They are not part of the product ABI
 * (include/llattn.h does not declare them) and may change without notice. */
#ifndef LLATTN_TESTING_H_
#define LLATTN_TESTING_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Process-wide choice between the tcgen05 (tensor memory) kernels (1, default) and the warp-level mma.sync
 * kernels (0) where both exist, so that a test can compare the two generations on the same inputs.  The flag
 * is an atomic; calls that are already dispatched keep the kernels they were given. */
void llattn_testing_use_tensor_core_path(int enabled);

/* One CTA waits on an mbarrier that nothing ever completes, with `spin_limit` polls as the bound, and then
 * reports through the same path as the production kernels: *status_dev (device memory) is set to 1 and the
 * kernel returns.  Lets a test see the give-up path without a hung GPU.  spin_limit is clamped to [1, 2^20]. */
int llattn_selftest_wait_timeout(int spin_limit, int* status_dev, void* stream);

/* Cycles of `reps` executions of one element-wise phase of the kernels (the fp32 32 x 32 x 32 block product of the
 * triangular inverses, 256 threads, operands in shared memory, a 256-thread barrier after each).  `copies` (1 or 64) separate
 * copies of the phase's code (about 2.3 KB each) are executed per repetition, which sets the instruction footprint of the loop
 * body; `spin_warps` (0..4) further warps of the CTA poll meanwhile; `env` adds features of the production kernels' environment:
 * bit 0 operands inside a 160 KB dynamic shared-memory allocation, bit 1 all 512 tensor-memory columns held, bit 2 the polling
 * thread of warp 8 uses mbarrier.try_wait (needs spin_warps >= 1).  cycles[0] receives clock64() ticks for reps x copies
 * phases; sink takes 384 floats. */
int llattn_selftest_ew_cycles(int reps, int spin_warps, int copies, int env, long long* cycles, float* sink, void* stream);

#ifdef __cplusplus
}
#endif
#endif
