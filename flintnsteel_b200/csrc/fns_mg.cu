// fns_mg.cu - the multi-GPU dispatcher behind the C ABI: one process per GPU, NCCL over NVLink for the one
// exchange step.  The reference (NomenAK/FlintNSteel) is single-GPU, one row per call (docs/ENGINE.md:132), so this
// layer has no counterpart there; it partitions the two kinds of work of the sampler:
//
//   rows         independent sessions.  Every rank samples the rows that its own LM head produced, with its own
//                workspace and stream: no collective on the data path.  (The tokens can be gathered afterwards,
//                4 bytes per row.)
//   vocabulary   one very large vocabulary split evenly over the ranks on 32-id boundaries (whole bitmask words).
//                Every rank selects the top-k_cap (value, id) candidates of its shard of every row (select_rows,
//                the first half of the path), ONE all-gather brings the lists of all shards into local memory
//                (k_cap * 8 bytes per row and rank), and every rank runs the same merge + draw on the gathered
//                lists (finalize_rows), so all ranks hold the same tokens without a broadcast.  Exact for the reason
//                the reference's 128 slices are (src/kernels.cu:594-597): the global top-k lies in the union of the
//                shards' top-k, and the merge orders by (value, id) alone.
//
// The three steps are enqueued on the caller's stream back to back; the host does nothing in between.  NCCL is
// loaded at run time (dlopen of libnccl.so.2) when a dispatcher spans more than one rank, so a single-GPU user needs
// no NCCL at all.  Kernels, collective and allocator are reached through a table of function pointers whose
// defaults are the CUDA sampler and NCCL; tests replace them to run the dispatcher's logic without a GPU.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "fns_internal.h"

namespace {

struct NcclApi {
    void * lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char * (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

NcclApi & nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.lib) api.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!api.lib) return;
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.lib, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.lib, "ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.lib, "ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.lib, "ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.lib, "ncclGetErrorString"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GetErrorString;
    });
    return api;
}

}  // namespace

struct fns_b200_mg {
    int device, rank, world, mode, max_rows, vocab, k_cap, max_history;
    int lo, hi;                 // VOCAB: the ids this rank owns
    fns_b200_mg_ops ops;
    bool default_ops;
    fns_b200_sampler * sampler; // default ops
    ncclComm_t comm;
    bool own_comm;
    fns_b200_cand * local;      // [max_rows][k_cap] this shard's lists
    fns_b200_cand * gathered;   // [world][max_rows][k_cap]
    int32_t * tok_pad;          // [ceil(max_rows)] ROWS: this rank's tokens padded to the widest shard
    int32_t * tok_all;          // [world][width]
    bool prof;
    std::vector<cudaEvent_t> ev;  // four per recorded call
    int prof_calls;
    char msg[256];
};

namespace {

int mfail(fns_b200_mg * m, int code, const char * what) {
    if (m) std::snprintf(m->msg, sizeof m->msg, "%s", what);
    return code;
}

void shard_range(int total, int rank, int world, int * lo, int * hi) {  // the first total % world ranks get one more
    const int base = total / world, extra = total % world;
    *lo = rank * base + (rank < extra ? rank : extra);
    *hi = *lo + base + (rank < extra ? 1 : 0);
}

// ---- default table: the CUDA sampler, cudaMalloc, NCCL ----------------------------------------------------------
int d_alloc(void *, size_t bytes, void ** out) { return cudaMalloc(out, bytes) == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA; }
int d_release(void *, void * p) { return cudaFree(p) == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA; }
int d_copy(void *, void * dst, const void * src, size_t bytes, void * stream) {
    return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t) stream) == cudaSuccess ? FNS_B200_OK
                                                                                                              : FNS_B200_ERR_CUDA;
}
int d_select(void * user, const void * logits, int dtype, int64_t row_stride, int vocab, int rows, int32_t id_base,
             const uint32_t * masks, int64_t mask_stride, const int32_t * history, int64_t history_stride,
             const int32_t * history_len, const fns_b200_params * params, fns_b200_cand * out, void * stream) {
    fns_b200_mg * m = static_cast<fns_b200_mg *>(user);
    const int rc = fns_b200_select_rows(m->sampler, logits, dtype, row_stride, vocab, rows, id_base, masks, mask_stride,
                                        history, history_stride, history_len, params, out, stream);
    if (rc != FNS_B200_OK) mfail(m, rc, fns_b200_last_error(m->sampler));
    return rc;
}
int d_finalize(void * user, const fns_b200_cand * cands, int lists, int list_len, int64_t list_stride, int64_t row_stride,
               int rows, const fns_b200_params * params, int32_t * out_tokens, void * stream) {
    fns_b200_mg * m = static_cast<fns_b200_mg *>(user);
    const int rc = fns_b200_finalize_rows(m->sampler, cands, lists, list_len, list_stride, row_stride, rows, params,
                                          out_tokens, nullptr, stream);
    if (rc != FNS_B200_OK) mfail(m, rc, fns_b200_last_error(m->sampler));
    return rc;
}
int d_sample(void * user, const void * logits, int dtype, int64_t row_stride, int vocab, int rows, const uint32_t * masks,
             int64_t mask_stride, const int32_t * history, int64_t history_stride, const int32_t * history_len,
             const fns_b200_params * params, int32_t * out_tokens, void * stream) {
    fns_b200_mg * m = static_cast<fns_b200_mg *>(user);
    const int rc = fns_b200_sample_rows(m->sampler, logits, dtype, row_stride, vocab, rows, masks, mask_stride, history,
                                        history_stride, history_len, params, out_tokens, stream);
    if (rc != FNS_B200_OK) mfail(m, rc, fns_b200_last_error(m->sampler));
    return rc;
}
int d_allgather(void * user, const void * send, void * recv, size_t bytes_per_rank, void * stream) {
    fns_b200_mg * m = static_cast<fns_b200_mg *>(user);
    if (!m->comm) return mfail(m, FNS_B200_ERR_ARG, "no communicator");
    const ncclResult_t r = nccl().AllGather(send, recv, bytes_per_rank, ncclChar, m->comm, (cudaStream_t) stream);
    if (r != ncclSuccess) {
        std::snprintf(m->msg, sizeof m->msg, "ncclAllGather: %s", nccl().GetErrorString(r));
        return FNS_B200_ERR_CUDA;
    }
    return FNS_B200_OK;
}

struct DevGuard {
    int prev = -1;
    bool active;
    explicit DevGuard(const fns_b200_mg * m) : active(m->default_ops) {
        if (!active) return;
        cudaGetDevice(&prev);
        if (prev != m->device) cudaSetDevice(m->device);
    }
    ~DevGuard() {
        int cur = -1;
        if (active && prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

void mark(fns_b200_mg * m, int which, void * stream) {  // which: 0 .. 3 of the call being recorded
    if (m->prof && m->default_ops && (size_t) (m->prof_calls + 1) * 4 <= m->ev.size())
        cudaEventRecord(m->ev[(size_t) m->prof_calls * 4 + which], (cudaStream_t) stream);
}

int create_common(int device, int rank, int world, int mode, int max_rows, int vocab, int k_cap, int max_history,
                  const fns_b200_mg_ops * ops, const void * unique_id, void * comm, fns_b200_mg ** out) {
    if (!out) return FNS_B200_ERR_ARG;
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world || (mode != FNS_B200_MG_ROWS && mode != FNS_B200_MG_VOCAB) || max_rows <= 0 ||
        vocab <= 0 || k_cap < 1 || k_cap > FNS_B200_MAX_K || max_history < 0)
        return FNS_B200_ERR_ARG;
    // every shard owns whole bitmask words; a shard without a word cannot be sampled
    if (mode == FNS_B200_MG_VOCAB && world > (vocab + 31) / 32) return FNS_B200_ERR_ARG;
    if (mode == FNS_B200_MG_VOCAB && (size_t) world * k_cap > 8192) return FNS_B200_ERR_CAPACITY;  // what the merge holds per row
    fns_b200_mg * m = new (std::nothrow) fns_b200_mg();
    if (!m) return FNS_B200_ERR_ARG;
    m->device = device;
    m->rank = rank;
    m->world = world;
    m->mode = mode;
    m->max_rows = max_rows;
    m->vocab = vocab;
    m->k_cap = k_cap;
    m->max_history = max_history;
    m->default_ops = ops == nullptr;
    m->msg[0] = 0;
    if (mode == FNS_B200_MG_VOCAB) {
        int wlo, whi;
        shard_range((vocab + 31) / 32, rank, world, &wlo, &whi);
        m->lo = wlo * 32;
        m->hi = whi * 32 < vocab ? whi * 32 : vocab;
    } else {
        m->lo = 0;
        m->hi = vocab;
    }
    if (ops) {
        m->ops = *ops;
    } else {
        m->ops = fns_b200_mg_ops{m, d_alloc, d_release, d_copy, d_select, d_finalize, d_sample, d_allgather};
    }
    DevGuard g(m);
    int rc = FNS_B200_OK;
    if (m->default_ops) {
        rc = fns_b200_create(device, max_rows, mode == FNS_B200_MG_VOCAB ? m->hi - m->lo : vocab, k_cap, max_history, &m->sampler);
        if (rc == FNS_B200_OK && world > 1) {
            if (comm) {
                m->comm = static_cast<ncclComm_t>(comm);
            } else if (!unique_id) {
                rc = FNS_B200_ERR_ARG;
            } else if (!nccl().ok) {
                rc = FNS_B200_ERR_CUDA;  // libnccl.so.2 not found
            } else {
                ncclUniqueId id;
                std::memcpy(&id, unique_id, sizeof id);
                rc = nccl().CommInitRank(&m->comm, world, id, rank) == ncclSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA;
                m->own_comm = rc == FNS_B200_OK;
            }
        }
    }
    void * p = nullptr;
    if (rc == FNS_B200_OK && mode == FNS_B200_MG_VOCAB) {
        const size_t one = (size_t) max_rows * k_cap * sizeof(fns_b200_cand);
        if ((rc = m->ops.alloc(m->ops.user, one, &p)) == FNS_B200_OK) m->local = static_cast<fns_b200_cand *>(p);
        if (rc == FNS_B200_OK && (rc = m->ops.alloc(m->ops.user, one * world, &p)) == FNS_B200_OK)
            m->gathered = static_cast<fns_b200_cand *>(p);
    }
    if (rc == FNS_B200_OK && mode == FNS_B200_MG_ROWS && world > 1) {
        const size_t one = (size_t) max_rows * sizeof(int32_t);
        if ((rc = m->ops.alloc(m->ops.user, one, &p)) == FNS_B200_OK) m->tok_pad = static_cast<int32_t *>(p);
        if (rc == FNS_B200_OK && (rc = m->ops.alloc(m->ops.user, one * world, &p)) == FNS_B200_OK)
            m->tok_all = static_cast<int32_t *>(p);
    }
    if (rc != FNS_B200_OK) {
        fns_b200_mg_destroy(m);
        return rc;
    }
    *out = m;
    return FNS_B200_OK;
}

}  // namespace

extern "C" {

int fns_b200_mg_unique_id(void * id_host) {
    if (!id_host) return FNS_B200_ERR_ARG;
    static_assert(sizeof(ncclUniqueId) == FNS_B200_MG_ID_BYTES, "the id travels as 128 bytes");
    if (!nccl().ok) return FNS_B200_ERR_CUDA;
    ncclUniqueId id;
    if (nccl().GetUniqueId(&id) != ncclSuccess) return FNS_B200_ERR_CUDA;
    std::memcpy(id_host, &id, sizeof id);
    return FNS_B200_OK;
}

int fns_b200_mg_create(int device, int rank, int world, int mode, int max_rows, int vocab, int k_cap, int max_history,
                       const void * unique_id_host, void * nccl_comm, fns_b200_mg ** out) {
    return create_common(device, rank, world, mode, max_rows, vocab, k_cap, max_history, nullptr, unique_id_host, nccl_comm, out);
}

int fns_b200_mg_create_with_ops(int rank, int world, int mode, int max_rows, int vocab, int k_cap, int max_history,
                                const fns_b200_mg_ops * ops, fns_b200_mg ** out) {
    if (!ops || !ops->alloc || !ops->release || !ops->copy || !ops->select_rows || !ops->finalize_rows || !ops->sample_rows ||
        !ops->allgather)
        return FNS_B200_ERR_ARG;
    return create_common(-1, rank, world, mode, max_rows, vocab, k_cap, max_history, ops, nullptr, nullptr, out);
}

int fns_b200_mg_destroy(fns_b200_mg * m) {
    if (!m) return FNS_B200_OK;
    DevGuard g(m);
    if (m->default_ops) cudaDeviceSynchronize();
    for (void * p : {(void *) m->local, (void *) m->gathered, (void *) m->tok_pad, (void *) m->tok_all})
        if (p) m->ops.release(m->ops.user, p);
    for (cudaEvent_t e : m->ev) cudaEventDestroy(e);
    if (m->own_comm && m->comm) nccl().CommDestroy(m->comm);
    if (m->sampler) fns_b200_destroy(m->sampler);
    delete m;
    return FNS_B200_OK;
}

const char * fns_b200_mg_last_error(const fns_b200_mg * m) { return m ? m->msg : "null dispatcher"; }

int fns_b200_mg_range(const fns_b200_mg * m, int total_rows, int * lo, int * hi) {
    if (!m || !lo || !hi) return FNS_B200_ERR_ARG;
    if (m->mode == FNS_B200_MG_VOCAB) {
        *lo = m->lo;
        *hi = m->hi;
    } else {
        if (total_rows < 0) return FNS_B200_ERR_ARG;
        shard_range(total_rows, m->rank, m->world, lo, hi);
    }
    return FNS_B200_OK;
}

int fns_b200_mg_sample_rows(fns_b200_mg * m, const void * logits, int dtype, int64_t row_stride, int rows,
                            const uint32_t * masks, int64_t mask_stride_words, const int32_t * history,
                            int64_t history_stride, const int32_t * history_len, const fns_b200_params * params,
                            int32_t * out_tokens, void * stream) {
    if (!m) return FNS_B200_ERR_ARG;
    if (!logits || !params || !out_tokens || rows <= 0) return mfail(m, FNS_B200_ERR_ARG, "logits / params / out_tokens null or rows <= 0");
    if (rows > m->max_rows) return mfail(m, FNS_B200_ERR_CAPACITY, "rows beyond the dispatcher's limit");
    DevGuard g(m);
    if (m->mode == FNS_B200_MG_ROWS) {  // this rank's rows: no collective on the data path
        mark(m, 0, stream);
        const int rc = m->ops.sample_rows(m->ops.user, logits, dtype, row_stride, m->vocab, rows, masks, mask_stride_words,
                                          history, history_stride, history_len, params, out_tokens, stream);
        mark(m, 1, stream);
        mark(m, 2, stream);
        mark(m, 3, stream);
        if (rc == FNS_B200_OK && m->prof) ++m->prof_calls;
        return rc;
    }
    // the shard's candidates -> one all-gather -> merge + draw, all on the caller's stream
    const size_t one = (size_t) rows * m->k_cap * sizeof(fns_b200_cand);
    mark(m, 0, stream);
    int rc = m->ops.select_rows(m->ops.user, logits, dtype, row_stride, m->hi - m->lo, rows, m->lo, masks, mask_stride_words,
                                history, history_stride, history_len, params, m->world > 1 ? m->local : m->gathered, stream);
    if (rc != FNS_B200_OK) return rc;
    mark(m, 1, stream);
    if (m->world > 1 && (rc = m->ops.allgather(m->ops.user, m->local, m->gathered, one, stream)) != FNS_B200_OK) return rc;
    mark(m, 2, stream);
    // gathered is [world][rows][k_cap]: list l of row r starts at l * rows * k_cap + r * k_cap
    rc = m->ops.finalize_rows(m->ops.user, m->gathered, m->world, m->k_cap, (int64_t) rows * m->k_cap, m->k_cap, rows, params,
                              out_tokens, stream);
    mark(m, 3, stream);
    if (rc == FNS_B200_OK && m->prof) ++m->prof_calls;
    return rc;
}

int fns_b200_mg_gather_tokens(fns_b200_mg * m, const int32_t * local_tokens, int total_rows, int32_t * all_tokens,
                              void * stream) {
    if (!m) return FNS_B200_ERR_ARG;
    if (m->mode != FNS_B200_MG_ROWS) return mfail(m, FNS_B200_ERR_ARG, "gather_tokens is for the row partition");
    if (!local_tokens || !all_tokens || total_rows <= 0) return mfail(m, FNS_B200_ERR_ARG, "tokens null or total_rows <= 0");
    DevGuard g(m);
    int lo, hi;
    shard_range(total_rows, m->rank, m->world, &lo, &hi);
    if (m->world == 1) return m->ops.copy(m->ops.user, all_tokens, local_tokens, (size_t) total_rows * 4, stream);
    const int width = (total_rows + m->world - 1) / m->world;  // the widest shard: equal contributions for the collective
    if (width > m->max_rows) return mfail(m, FNS_B200_ERR_CAPACITY, "a shard wider than max_rows");
    int rc = m->ops.copy(m->ops.user, m->tok_pad, local_tokens, (size_t) (hi - lo) * 4, stream);
    if (rc == FNS_B200_OK) rc = m->ops.allgather(m->ops.user, m->tok_pad, m->tok_all, (size_t) width * 4, stream);
    for (int r = 0; r < m->world && rc == FNS_B200_OK; ++r) {
        int a, z;
        shard_range(total_rows, r, m->world, &a, &z);
        if (z > a) rc = m->ops.copy(m->ops.user, all_tokens + a, m->tok_all + (size_t) r * width, (size_t) (z - a) * 4, stream);
    }
    return rc;
}

int fns_b200_mg_profile_begin(fns_b200_mg * m, int max_calls) {
    if (!m || max_calls <= 0 || max_calls > 100000) return FNS_B200_ERR_ARG;
    if (!m->default_ops) return mfail(m, FNS_B200_ERR_ARG, "stage timing needs the CUDA table");
    DevGuard g(m);
    while (m->ev.size() < (size_t) max_calls * 4) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return mfail(m, FNS_B200_ERR_CUDA, "cudaEventCreate");
        m->ev.push_back(e);
    }
    m->prof_calls = 0;
    m->prof = true;
    return FNS_B200_OK;
}

int fns_b200_mg_profile_end(fns_b200_mg * m, void * stream, double * select_us, double * exchange_us, double * finalize_us,
                            int * calls) {
    if (!m) return FNS_B200_ERR_ARG;
    m->prof = false;
    DevGuard g(m);
    if (cudaStreamSynchronize((cudaStream_t) stream) != cudaSuccess) return mfail(m, FNS_B200_ERR_CUDA, "profile_end");
    double t[3] = {0.0, 0.0, 0.0};
    for (int i = 0; i < m->prof_calls; ++i)
        for (int s = 0; s < 3; ++s) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, m->ev[(size_t) i * 4 + s], m->ev[(size_t) i * 4 + s + 1]) == cudaSuccess) t[s] += ms * 1e3;
        }
    const double n = m->prof_calls > 0 ? m->prof_calls : 1;
    if (select_us) *select_us = t[0] / n;
    if (exchange_us) *exchange_us = t[1] / n;
    if (finalize_us) *finalize_us = t[2] / n;
    if (calls) *calls = m->prof_calls;
    return FNS_B200_OK;
}

}  // extern "C"
