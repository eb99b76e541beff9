/* fns_internal.h - entry points that the library exports for its own tests, its benchmark and its engine glue.
 * Not part of the ABI in include/fns_b200.h: nothing here is meant for a caller of the sampler. */
#ifndef FNS_B200_INTERNAL_H
#define FNS_B200_INTERNAL_H

#include <stddef.h>

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
/* Calls of up to `rows` rows take the cluster kernel (0: never).  For the same tests. */
int fns_b200_set_cluster_rows(fns_b200_sampler * s, int rows);

/* One row with its parameters passed by value from the host (as fns_b200_sample_one) and a history in device memory
 * (history [history_stride] ids, history_len [1]): the engine glue's one-session step, which then uploads nothing
 * but the mask. */
int fns_b200_sample_one_with_history(fns_b200_sampler * s, const void * logits, int dtype, int vocab, const uint32_t * mask,
                                     const int32_t * history, int64_t history_stride, const int32_t * history_len,
                                     const fns_b200_params * params_host, int32_t * out_token, void * stream);

/* The engine glue says that the logits of the handle's next calls lie in page-locked HOST memory (on = 1) or in
 * device memory (on = 0): host logits are read in place by the kernel that skips every vector the mask excludes,
 * never by the bulk-copy kernel, which would move whole chunks over PCIe. */
int fns_b200_hint_host_logits(fns_b200_sampler * s, int on);

/* The dispatcher reaches its kernels, its collective and its allocator through this table.  The defaults are the CUDA
 * sampler, NCCL and cudaMalloc; a test fills in stand-ins that work on host memory, so that the dispatcher's own
 * logic (shard arithmetic, buffer layout, strides handed to the merge) runs on a machine without a GPU.  Every
 * function returns a status code; `user` is passed back as the first argument. */
typedef struct fns_b200_mg_ops {
    void * user;
    int (*alloc)(void * user, size_t bytes, void ** out);
    int (*release)(void * user, void * p);
    int (*copy)(void * user, void * dst, const void * src, size_t bytes, void * stream);
    int (*select_rows)(void * user, const void * logits, int dtype, int64_t row_stride, int vocab, int rows, int32_t id_base,
                       const uint32_t * masks, int64_t mask_stride_words, const int32_t * history, int64_t history_stride,
                       const int32_t * history_len, const fns_b200_params * params, fns_b200_cand * out_cands, void * stream);
    int (*finalize_rows)(void * user, const fns_b200_cand * cands, int lists, int list_len, int64_t list_stride,
                         int64_t row_stride, int rows, const fns_b200_params * params, int32_t * out_tokens, void * stream);
    int (*sample_rows)(void * user, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
                       const uint32_t * masks, int64_t mask_stride_words, const int32_t * history, int64_t history_stride,
                       const int32_t * history_len, const fns_b200_params * params, int32_t * out_tokens, void * stream);
    int (*allgather)(void * user, const void * send, void * recv, size_t bytes_per_rank, void * stream);
} fns_b200_mg_ops;
int fns_b200_mg_create_with_ops(int rank, int world, int mode, int max_rows, int vocab, int k_cap, int max_history,
                                const fns_b200_mg_ops * ops, fns_b200_mg ** out);

#ifdef __cplusplus
}
#endif
#endif /* FNS_B200_INTERNAL_H */
