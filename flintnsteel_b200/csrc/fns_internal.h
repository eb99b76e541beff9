/* fns_internal.h - entry points that the library exports for its own tests, its benchmark and its engine glue.
 * Not part of the ABI in include/fns_b200.h: nothing here is meant for a caller of the sampler. */
#ifndef FNS_B200_INTERNAL_H
#define FNS_B200_INTERNAL_H

#include "../../include/fns_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Launch geometry chosen for a call (slices per row, threads, dynamic shared memory of the select kernel),
 * for benchmarks and tests. */
int fns_b200_plan(const fns_b200_sampler * s, int dtype, int vocab, int rows, int history_bound, int * slices,
                  int * slice_len, int * smem_bytes);
/* Overrides the number of slices per row (0 = automatic).  For tests that must show that results do not depend
 * on the launch geometry. */
int fns_b200_set_slices(fns_b200_sampler * s, int slices);
/* Overrides the block size of the select kernel: 256 (sliced rows), 512 (one block per row when it fits), 0 =
 * automatic.  For the same tests. */
int fns_b200_set_threads(fns_b200_sampler * s, int threads);

/* The engine glue says that the logits of the handle's next calls lie in page-locked HOST memory (on = 1) or in
 * device memory (on = 0): host logits are read in place by the kernel that skips every vector the mask excludes,
 * never by the bulk-copy kernel, which would move whole chunks over PCIe. */
int fns_b200_hint_host_logits(fns_b200_sampler * s, int on);

#ifdef __cplusplus
}
#endif
#endif /* FNS_B200_INTERNAL_H */
