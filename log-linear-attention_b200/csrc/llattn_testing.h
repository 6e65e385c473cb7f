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

#ifdef __cplusplus
}
#endif
#endif
