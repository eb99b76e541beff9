// fns_engine.cu - host-side glue around the sampler: what fns::Engine does around k::sample / k::argmax
// (NomenAK/FlintNSteel src/engine.cu:733-765, 796-866), for a batch of independent sessions.
//
//   pick_async   stage masks / histories / parameters through pinned memory, copy them to the device on the
//                caller's stream, sample, copy the tokens back, record an event     (src/engine.cu:823-847)
//   pick_wait    wait for that event, hand out the tokens                            (src/engine.cu:849-852)
//   verify       the same for verification windows plus the accept rule, synchronous (src/engine.cu:733-765,
//                tools/fns_serve/fns_serve.cpp:492-508)
//   reset/append the sessions' penalty state.  The reference keeps a dense float seen[V] per engine
//                (src/engine.cu:854-866); here it is a list of token ids per session, kept on the device and
//                extended by a one-block kernel, so a decode step uploads no history at all.
// Two staging slots alternate, so the next pick can be queued while the host still waits for the previous one.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <unordered_map>
#include <vector>

#include "fns_internal.h"

namespace {

constexpr int kSlots = 2;

__global__ void k_history_append(int32_t * history, int32_t * history_len, int64_t history_stride,
                                 const int32_t * tokens, int64_t tokens_stride, const int32_t * counts, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int n = counts ? counts[r] : 1;
    int len = history_len[r];
    for (int j = 0; j < n; ++j) {
        const int32_t t = tokens[r * tokens_stride + j];
        if (t >= 0 && len < history_stride) history[r * history_stride + len++] = t;  // -1: no token (kernels.cu:730)
    }
    history_len[r] = len;
}

struct Slot {
    // pinned host staging
    uint32_t * masks_h;
    int32_t * history_h;
    int32_t * history_len_h;
    fns_b200_params * params_h;
    int32_t * tokens_h;
    int32_t * draft_h;
    int32_t * accept_h;
    int32_t * mask_rows_h;
    // device copies
    uint32_t * masks_d;
    int32_t * history_d;
    int32_t * history_len_d;
    fns_b200_params * params_d;
    int32_t * tokens_d;
    int32_t * draft_d;
    int32_t * accept_d;
    int32_t * mask_rows_d;
    int32_t * tokens_hd;  // tokens_h as the GPU addresses it (NULL until first asked for, or if it cannot)
    void * logits_d;      // staging for logits that arrive in host memory: one per slot, since the kernel of the older
    size_t logits_bytes;  // pick may still read its copy; grows on first use (cudaFree waits for the device once)
    cudaEvent_t done;
    int rows;
    bool busy;
};

}  // namespace

struct fns_b200_engine {
    int device, max_rows, vocab, words, k_cap, max_history;
    fns_b200_sampler * sampler;
    Slot slot[kSlots];
    int head, tail;       // next slot to fill / oldest slot in flight
    int32_t * sess_history;      // [max_rows][max_history] device-side session histories
    int32_t * sess_history_len;  // [max_rows]
    int32_t * counts_d;
    int32_t * counts_h;
    const int32_t * last_tokens;
    // masks kept on the device by grammar state: slot 0 allows everything, slots 1 .. cache_slots hold states
    uint32_t * cache_d;               // [cache_slots + 1][words]
    int cache_slots;
    uint64_t tick;
    std::vector<uint64_t> slot_state; // [cache_slots + 1] the state a slot holds
    std::vector<uint64_t> slot_used;  // ... and when it was last asked for
    std::vector<uint8_t> slot_filled;
    std::unordered_map<uint64_t, int> * by_state;
    int64_t mask_bytes_uploaded, mask_hits, mask_misses;
    char msg[256];
};

namespace {

int efail(fns_b200_engine * e, int code, const char * what) {
    if (e) std::snprintf(e->msg, sizeof e->msg, "%s", what);
    return code;
}
int ecuda(fns_b200_engine * e, cudaError_t err, const char * where) {
    if (e) std::snprintf(e->msg, sizeof e->msg, "%s: %s", where, cudaGetErrorString(err));
    return FNS_B200_ERR_CUDA;
}
int esampler(fns_b200_engine * e, int rc) {
    if (rc != FNS_B200_OK) std::snprintf(e->msg, sizeof e->msg, "%s", fns_b200_last_error(e->sampler));
    return rc;
}

template <typename T>
bool alloc_pair(T ** host, T ** dev, size_t count) {
    return cudaMallocHost((void **) host, count * sizeof(T)) == cudaSuccess &&
           cudaMalloc((void **) dev, count * sizeof(T)) == cudaSuccess;
}

void free_slot(Slot & s) {
    cudaFreeHost(s.masks_h); cudaFreeHost(s.history_h); cudaFreeHost(s.history_len_h); cudaFreeHost(s.params_h);
    cudaFreeHost(s.tokens_h); cudaFreeHost(s.draft_h); cudaFreeHost(s.accept_h); cudaFreeHost(s.mask_rows_h);
    cudaFree(s.masks_d); cudaFree(s.history_d); cudaFree(s.history_len_d); cudaFree(s.params_d);
    cudaFree(s.tokens_d); cudaFree(s.draft_d); cudaFree(s.accept_d); cudaFree(s.mask_rows_d); cudaFree(s.logits_d);
    if (s.done) cudaEventDestroy(s.done);
}

struct Dev {
    int prev = -1;
    explicit Dev(int d) {
        cudaGetDevice(&prev);
        if (prev != d) cudaSetDevice(d);
    }
    ~Dev() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

// Host -> pinned -> device, asynchronous on st (the reference's memcpy + cudaMemcpyAsync, src/engine.cu:833-834).
template <typename T>
cudaError_t stage(T * pinned, T * dev, const T * src, size_t count, cudaStream_t st) {
    std::memcpy(pinned, src, count * sizeof(T));
    return cudaMemcpyAsync(dev, pinned, count * sizeof(T), cudaMemcpyHostToDevice, st);
}

// The device-side address of a page-locked host buffer, or NULL when the buffer is pageable (unknown to the driver).
const void * device_view(const void * host) {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, host) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}

// Host -> device on st: straight from the caller's buffer when it is page-locked and promised stable, else staged.
template <typename T>
cudaError_t bring(T * pinned, T * dev, const T * src, size_t count, bool stable, cudaStream_t st) {
    if (stable && device_view(src)) return cudaMemcpyAsync(dev, src, count * sizeof(T), cudaMemcpyHostToDevice, st);
    return stage(pinned, dev, src, count, st);
}

}  // namespace

extern "C" {

int fns_b200_engine_create(int device, int max_rows, int vocab, int k_cap, int max_history, fns_b200_engine ** out) {
    if (!out) return FNS_B200_ERR_ARG;
    *out = nullptr;
    if (max_rows <= 0 || vocab <= 0 || max_history < 0) return FNS_B200_ERR_ARG;
    Dev g(device);
    fns_b200_engine * e = new (std::nothrow) fns_b200_engine();
    if (!e) return FNS_B200_ERR_ARG;
    e->device = device;
    e->max_rows = max_rows;
    e->vocab = vocab;
    e->words = (vocab + 31) / 32;
    e->k_cap = k_cap;
    e->max_history = max_history;
    int rc = fns_b200_create(device, max_rows, vocab, k_cap, max_history, &e->sampler);
    if (rc != FNS_B200_OK) {
        delete e;
        return rc;
    }
    bool ok = true;
    const size_t hist = (size_t) max_rows * (max_history > 0 ? max_history : 1);
    for (int i = 0; i < kSlots && ok; ++i) {
        Slot & s = e->slot[i];
        ok = alloc_pair(&s.masks_h, &s.masks_d, (size_t) max_rows * e->words) &&
             alloc_pair(&s.history_h, &s.history_d, hist) && alloc_pair(&s.history_len_h, &s.history_len_d, max_rows) &&
             alloc_pair(&s.params_h, &s.params_d, max_rows) && alloc_pair(&s.tokens_h, &s.tokens_d, max_rows) &&
             alloc_pair(&s.draft_h, &s.draft_d, max_rows) && alloc_pair(&s.accept_h, &s.accept_d, max_rows) &&
             alloc_pair(&s.mask_rows_h, &s.mask_rows_d, max_rows) &&
             cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming) == cudaSuccess;
    }
    ok = ok && cudaMalloc(&e->sess_history, hist * sizeof(int32_t)) == cudaSuccess &&
         cudaMalloc(&e->sess_history_len, max_rows * sizeof(int32_t)) == cudaSuccess &&
         cudaMemset(e->sess_history_len, 0, max_rows * sizeof(int32_t)) == cudaSuccess &&
         cudaMalloc(&e->counts_d, max_rows * sizeof(int32_t)) == cudaSuccess &&
         cudaMallocHost(&e->counts_h, max_rows * sizeof(int32_t)) == cudaSuccess;
    if (!ok) {
        fns_b200_engine_destroy(e);
        return FNS_B200_ERR_CUDA;
    }
    *out = e;
    return FNS_B200_OK;
}

int fns_b200_engine_destroy(fns_b200_engine * e) {
    if (!e) return FNS_B200_OK;
    Dev g(e->device);
    cudaDeviceSynchronize();
    for (int i = 0; i < kSlots; ++i) free_slot(e->slot[i]);
    cudaFree(e->sess_history);
    cudaFree(e->sess_history_len);
    cudaFree(e->counts_d);
    cudaFreeHost(e->counts_h);
    cudaFree(e->cache_d);
    delete e->by_state;
    fns_b200_destroy(e->sampler);
    delete e;
    return FNS_B200_OK;
}

const char * fns_b200_engine_last_error(const fns_b200_engine * e) { return e ? e->msg : "null engine"; }
int fns_b200_engine_words(const fns_b200_engine * e) { return e ? e->words : 0; }
fns_b200_sampler * fns_b200_engine_sampler(fns_b200_engine * e) { return e ? e->sampler : nullptr; }
const int32_t * fns_b200_engine_device_tokens(const fns_b200_engine * e) { return e ? e->last_tokens : nullptr; }

int fns_b200_engine_pick_async(fns_b200_engine * e, const void * logits, int logits_on_host, int dtype,
                               int64_t row_stride, int rows, const uint32_t * masks_host,
                               const int32_t * history_host, int64_t history_stride,
                               const int32_t * history_len_host, const fns_b200_params * params_host, void * stream) {
    if (!e) return FNS_B200_ERR_ARG;
    if (!logits || !params_host || rows <= 0) return efail(e, FNS_B200_ERR_ARG, "logits / params null or rows <= 0");
    if (rows > e->max_rows) return efail(e, FNS_B200_ERR_CAPACITY, "rows beyond the engine's limit");
    if (history_host && (!history_len_host || history_stride <= 0 || history_stride > e->max_history))
        return efail(e, FNS_B200_ERR_CAPACITY, "history_stride outside (0, max_history] or history_len_host null");
    Dev g(e->device);
    cudaStream_t st = (cudaStream_t) stream;
    Slot & s = e->slot[e->head];
    if (s.busy) return efail(e, FNS_B200_ERR_ARG, "two picks already in flight: call pick_wait first");
    cudaError_t err = cudaSuccess;
    const size_t esz = dtype == FNS_B200_BF16 ? 2 : 4;
    const void * lg = logits;
    const bool stable = (logits_on_host & FNS_B200_HOST_STABLE) != 0;
    const void * in_place = (logits_on_host & FNS_B200_HOST_LOGITS) && stable && masks_host ? device_view(logits) : nullptr;
    if (in_place) {
        lg = in_place;  // the kernel loads the allowed vectors over PCIe; nothing else of the logits moves
    } else if (logits_on_host & FNS_B200_HOST_LOGITS) {
        const size_t bytes = ((size_t) (rows - 1) * row_stride + e->vocab) * esz;
        if (bytes > s.logits_bytes) {
            cudaFree(s.logits_d);
            s.logits_d = nullptr;
            s.logits_bytes = 0;
            if ((err = cudaMalloc(&s.logits_d, bytes)) != cudaSuccess) return ecuda(e, err, "logits staging");
            s.logits_bytes = bytes;
        }
        if ((err = cudaMemcpyAsync(s.logits_d, logits, bytes, cudaMemcpyHostToDevice, st)) != cudaSuccess)
            return ecuda(e, err, "logits copy");
        lg = s.logits_d;
    }
    if (masks_host && (err = bring(s.masks_h, s.masks_d, masks_host, (size_t) rows * e->words, stable, st)) != cudaSuccess)
        return ecuda(e, err, "mask copy");
    const int32_t * hist_d = nullptr, *hist_len_d = nullptr;
    int64_t hstride = 0;
    if (history_host) {
        // rows are packed to history_stride in the staging buffer
        if ((err = bring(s.history_h, s.history_d, history_host, (size_t) rows * history_stride, stable, st)) != cudaSuccess ||
            (err = bring(s.history_len_h, s.history_len_d, history_len_host, (size_t) rows, stable, st)) != cudaSuccess)
            return ecuda(e, err, "history copy");
        hist_d = s.history_d;
        hist_len_d = s.history_len_d;
        hstride = history_stride;
    } else if (e->max_history > 0) {
        hist_d = e->sess_history;
        hist_len_d = e->sess_history_len;
        hstride = e->max_history;
    }
    // One session (the reference's own shape, src/engine.cu:823-852): the parameters travel as a kernel argument and
    // the kernel writes the token straight into the slot's page-locked host word (which the GPU addresses too), so the
    // step costs the mask upload, one launch and the event - no copy of parameters in, no copy of the token out.
    if (rows == 1 && !s.tokens_hd) s.tokens_hd = static_cast<int32_t *>(const_cast<void *>(device_view(s.tokens_h)));
    int32_t * token_word = rows == 1 ? s.tokens_hd : nullptr;
    fns_b200_hint_host_logits(e->sampler, in_place != nullptr);
    int rc;
    if (token_word) {
        rc = fns_b200_sample_one_with_history(e->sampler, lg, dtype, e->vocab, masks_host ? s.masks_d : nullptr, hist_d, hstride,
                                              hist_len_d, params_host, token_word, st);
    } else {
        if ((err = bring(s.params_h, s.params_d, params_host, (size_t) rows, stable, st)) != cudaSuccess) {
            fns_b200_hint_host_logits(e->sampler, 0);
            return ecuda(e, err, "params copy");
        }
        rc = fns_b200_sample_rows(e->sampler, lg, dtype, row_stride, e->vocab, rows, masks_host ? s.masks_d : nullptr, e->words,
                                  hist_d, hstride, hist_len_d, s.params_d, s.tokens_d, st);
    }
    fns_b200_hint_host_logits(e->sampler, 0);
    if (rc != FNS_B200_OK) return esampler(e, rc);
    if ((!token_word &&
         (err = cudaMemcpyAsync(s.tokens_h, s.tokens_d, (size_t) rows * sizeof(int32_t), cudaMemcpyDeviceToHost, st)) != cudaSuccess) ||
        (err = cudaEventRecord(s.done, st)) != cudaSuccess)
        return ecuda(e, err, "token copy");
    s.rows = rows;
    s.busy = true;
    e->last_tokens = token_word ? token_word : s.tokens_d;
    e->head = (e->head + 1) % kSlots;
    return FNS_B200_OK;
}

// ---- the bitmask as its producer hands it over: xgrammar's DLTensor, with a device-side cache by grammar state ------
int fns_b200_mask_view(const fns_b200_dl_tensor * t, int vocab, int * rows, const uint32_t ** words_host, int64_t * stride_words) {
    if (!t || !rows || !words_host || !stride_words || vocab <= 0) return FNS_B200_ERR_ARG;
    const int words = (vocab + 31) / 32;
    // what xgrammar fills (tools/fns_serve/fns_serve.cpp:313-321): int32, on the CPU, [words] or [rows][words]
    if (!t->data || (t->device_type != 1 /* kDLCPU */ && t->device_type != 3 /* kDLCUDAHost */)) return FNS_B200_ERR_ARG;
    if (t->dtype_bits != 32 || t->dtype_lanes != 1 || (t->dtype_code != 0 /* kDLInt */ && t->dtype_code != 1 /* kDLUInt */))
        return FNS_B200_ERR_ARG;
    if ((t->ndim != 1 && t->ndim != 2) || !t->shape || t->shape[t->ndim - 1] != words) return FNS_B200_ERR_ARG;
    if (t->strides && t->strides[t->ndim - 1] != 1) return FNS_B200_ERR_ARG;  // words of a row side by side
    *rows = t->ndim == 2 ? (int) t->shape[0] : 1;
    *stride_words = t->ndim == 2 && t->strides ? t->strides[0] : words;
    if (*rows <= 0 || *stride_words < words) return FNS_B200_ERR_ARG;
    *words_host = reinterpret_cast<const uint32_t *>(static_cast<const char *>(t->data) + t->byte_offset);
    return FNS_B200_OK;
}

int fns_b200_engine_mask_cache(fns_b200_engine * e, int slots) {
    if (!e || slots < 0 || slots > 65535) return FNS_B200_ERR_ARG;
    Dev g(e->device);
    if (e->slot[0].busy || e->slot[1].busy) return efail(e, FNS_B200_ERR_ARG, "mask_cache: picks in flight");
    cudaFree(e->cache_d);
    e->cache_d = nullptr;
    e->cache_slots = 0;
    delete e->by_state;
    e->by_state = nullptr;
    if (slots == 0) return FNS_B200_OK;
    cudaError_t err = cudaMalloc(&e->cache_d, (size_t) (slots + 1) * e->words * sizeof(uint32_t));
    if (err == cudaSuccess) err = cudaMemset(e->cache_d, 0xff, (size_t) e->words * sizeof(uint32_t));  // slot 0: every id allowed
    if (err != cudaSuccess) return ecuda(e, err, "mask cache");
    e->cache_slots = slots;
    e->slot_state.assign(slots + 1, 0);
    e->slot_used.assign(slots + 1, 0);
    e->slot_filled.assign(slots + 1, 0);
    e->by_state = new std::unordered_map<uint64_t, int>();
    e->mask_bytes_uploaded = e->mask_hits = e->mask_misses = 0;
    return FNS_B200_OK;
}

int fns_b200_engine_mask_stats(const fns_b200_engine * e, int64_t * hits, int64_t * misses, int64_t * bytes_uploaded) {
    if (!e) return FNS_B200_ERR_ARG;
    if (hits) *hits = e->mask_hits;
    if (misses) *misses = e->mask_misses;
    if (bytes_uploaded) *bytes_uploaded = e->mask_bytes_uploaded;
    return FNS_B200_OK;
}

int fns_b200_engine_pick_async_dl(fns_b200_engine * e, const void * logits, int dtype, int64_t row_stride, int rows,
                                  const fns_b200_dl_tensor * masks, const uint64_t * mask_states_host,
                                  const fns_b200_params * params_host, void * stream) {
    if (!e) return FNS_B200_ERR_ARG;
    if (!logits || !params_host || rows <= 0) return efail(e, FNS_B200_ERR_ARG, "logits / params null or rows <= 0");
    if (rows > e->max_rows) return efail(e, FNS_B200_ERR_CAPACITY, "rows beyond the engine's limit");
    const uint32_t * words_host = nullptr;
    int mask_rows = 0;
    int64_t mstride = 0;
    if (masks) {
        if (fns_b200_mask_view(masks, e->vocab, &mask_rows, &words_host, &mstride) != FNS_B200_OK)
            return efail(e, FNS_B200_ERR_ARG, "masks: not an int32 CPU tensor of [rows][ceil(vocab / 32)] (or [ceil(vocab / 32)])");
        if (mask_rows != rows && mask_rows != 1) return efail(e, FNS_B200_ERR_ARG, "masks: one row, or one row per logit row");
    }
    if (!mask_states_host || !masks) {  // no cache: the plain path; rows of a strided tensor are packed on the way
        if (!masks) return fns_b200_engine_pick_async(e, logits, 0, dtype, row_stride, rows, nullptr, nullptr, 0, nullptr, params_host, stream);
        if (mask_rows == rows && mstride == e->words)
            return fns_b200_engine_pick_async(e, logits, 0, dtype, row_stride, rows, words_host, nullptr, 0, nullptr, params_host, stream);
        Slot & s = e->slot[e->head];
        if (s.busy) return efail(e, FNS_B200_ERR_ARG, "two picks already in flight: call pick_wait first");
        std::vector<uint32_t> packed((size_t) rows * e->words);
        for (int r = 0; r < rows; ++r)
            std::memcpy(packed.data() + (size_t) r * e->words, words_host + (size_t) (mask_rows == 1 ? 0 : r) * mstride, (size_t) e->words * 4);
        return fns_b200_engine_pick_async(e, logits, 0, dtype, row_stride, rows, packed.data(), nullptr, 0, nullptr, params_host, stream);
    }
    if (!e->cache_d) return efail(e, FNS_B200_ERR_ARG, "mask states given but no cache: call fns_b200_engine_mask_cache first");
    Dev g(e->device);
    cudaStream_t st = (cudaStream_t) stream;
    Slot & s = e->slot[e->head];
    if (s.busy) return efail(e, FNS_B200_ERR_ARG, "two picks already in flight: call pick_wait first");
    // a row's state either sits in a slot already (nothing moves), or takes the slot that has waited longest
    cudaError_t err = cudaSuccess;
    int staged = 0;
    ++e->tick;
    for (int r = 0; r < rows; ++r) {  // first the states that are here already: none of them may be pushed out by this call
        auto it = e->by_state->find(mask_states_host[r]);
        if (mask_states_host[r] != FNS_B200_NO_MASK && it != e->by_state->end()) e->slot_used[it->second] = e->tick;
    }
    for (int r = 0; r < rows; ++r) {
        const uint64_t state = mask_states_host[r];
        if (state == FNS_B200_NO_MASK) {
            s.mask_rows_h[r] = 0;
            continue;
        }
        auto it = e->by_state->find(state);
        int slot;
        if (it != e->by_state->end()) {
            slot = it->second;
            ++e->mask_hits;
        } else {
            slot = -1;
            uint64_t oldest = ~0ull;
            for (int c = 1; c <= e->cache_slots; ++c) {
                if (!e->slot_filled[c]) {
                    slot = c;
                    break;
                }
                if (e->slot_used[c] < e->tick && e->slot_used[c] < oldest) {  // (a slot asked for in this call stays)
                    oldest = e->slot_used[c];
                    slot = c;
                }
            }
            if (slot < 0) return efail(e, FNS_B200_ERR_CAPACITY, "more distinct grammar states in one call than cache slots");
            if (e->slot_filled[slot]) e->by_state->erase(e->slot_state[slot]);
            (*e->by_state)[state] = slot;
            e->slot_state[slot] = state;
            e->slot_filled[slot] = 1;
            // through pinned staging (the producer's buffer is pageable and refilled for the next token)
            uint32_t * stage_at = s.masks_h + (size_t) staged * e->words;
            std::memcpy(stage_at, words_host + (size_t) (mask_rows == 1 ? 0 : r) * mstride, (size_t) e->words * 4);
            err = cudaMemcpyAsync(e->cache_d + (size_t) slot * e->words, stage_at, (size_t) e->words * 4, cudaMemcpyHostToDevice, st);
            if (err != cudaSuccess) return ecuda(e, err, "mask upload");
            ++staged;
            ++e->mask_misses;
            e->mask_bytes_uploaded += (int64_t) e->words * 4;
        }
        e->slot_used[slot] = e->tick;
        s.mask_rows_h[r] = slot;
    }
    const bool hist = e->max_history > 0;
    // one session (see fns_b200_engine_pick_async): the mask is its cache slot, the parameters a kernel argument, the
    // token goes straight into the slot's page-locked host word - a state that the cache holds costs a launch and an event
    if (rows == 1 && !s.tokens_hd) s.tokens_hd = static_cast<int32_t *>(const_cast<void *>(device_view(s.tokens_h)));
    int32_t * token_word = rows == 1 ? s.tokens_hd : nullptr;
    int rc;
    if (token_word) {
        const uint32_t * one_mask = mask_states_host[0] == FNS_B200_NO_MASK ? nullptr : e->cache_d + (size_t) s.mask_rows_h[0] * e->words;
        rc = fns_b200_sample_one_with_history(e->sampler, logits, dtype, e->vocab, one_mask, hist ? e->sess_history : nullptr,
                                              hist ? e->max_history : 0, hist ? e->sess_history_len : nullptr, params_host, token_word, st);
    } else {
        if ((err = cudaMemcpyAsync(s.mask_rows_d, s.mask_rows_h, (size_t) rows * sizeof(int32_t), cudaMemcpyHostToDevice, st)) != cudaSuccess ||
            (err = stage(s.params_h, s.params_d, params_host, (size_t) rows, st)) != cudaSuccess)
            return ecuda(e, err, "mask rows / params copy");
        rc = fns_b200_sample_rows_shared_masks(e->sampler, logits, dtype, row_stride, e->vocab, rows, e->cache_d, e->words, s.mask_rows_d,
                                               hist ? e->sess_history : nullptr, hist ? e->max_history : 0,
                                               hist ? e->sess_history_len : nullptr, s.params_d, s.tokens_d, st);
    }
    if (rc != FNS_B200_OK) return esampler(e, rc);
    if ((!token_word &&
         (err = cudaMemcpyAsync(s.tokens_h, s.tokens_d, (size_t) rows * sizeof(int32_t), cudaMemcpyDeviceToHost, st)) != cudaSuccess) ||
        (err = cudaEventRecord(s.done, st)) != cudaSuccess)
        return ecuda(e, err, "token copy");
    s.rows = rows;
    s.busy = true;
    e->last_tokens = token_word ? token_word : s.tokens_d;
    e->head = (e->head + 1) % kSlots;
    return FNS_B200_OK;
}

int fns_b200_engine_pick_wait(fns_b200_engine * e, int32_t * tokens_host) {
    if (!e) return FNS_B200_ERR_ARG;
    Slot & s = e->slot[e->tail];
    if (!s.busy) return efail(e, FNS_B200_ERR_ARG, "no pick in flight");
    const cudaError_t err = cudaEventSynchronize(s.done);
    s.busy = false;
    e->tail = (e->tail + 1) % kSlots;
    if (err != cudaSuccess) return ecuda(e, err, "pick_wait");
    if (tokens_host) std::memcpy(tokens_host, s.tokens_h, (size_t) s.rows * sizeof(int32_t));
    return FNS_B200_OK;
}

int fns_b200_engine_reset(fns_b200_engine * e, void * stream) {
    if (!e) return FNS_B200_ERR_ARG;
    Dev g(e->device);
    const cudaError_t err = cudaMemsetAsync(e->sess_history_len, 0, (size_t) e->max_rows * sizeof(int32_t), (cudaStream_t) stream);
    return err == cudaSuccess ? FNS_B200_OK : ecuda(e, err, "reset");
}

int fns_b200_engine_append(fns_b200_engine * e, const int32_t * tokens, int64_t tokens_stride, int rows,
                           const int32_t * counts_host, void * stream) {
    if (!e) return FNS_B200_ERR_ARG;
    if (!tokens || rows <= 0 || rows > e->max_rows) return efail(e, FNS_B200_ERR_ARG, "tokens null or rows out of range");
    if (e->max_history <= 0) return efail(e, FNS_B200_ERR_CAPACITY, "engine was created without history");
    Dev g(e->device);
    cudaStream_t st = (cudaStream_t) stream;
    const int32_t * counts = nullptr;
    if (counts_host) {
        // counts_h is reused: wait until the previous append has read it
        cudaError_t err = cudaStreamSynchronize(st);
        if (err == cudaSuccess) err = stage(e->counts_h, e->counts_d, counts_host, (size_t) rows, st);
        if (err != cudaSuccess) return ecuda(e, err, "append counts");
        counts = e->counts_d;
    }
    k_history_append<<<(unsigned) ((rows + 127) / 128), 128, 0, st>>>(e->sess_history, e->sess_history_len, e->max_history,
                                                                     tokens, tokens_stride, counts, rows);
    const cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? FNS_B200_OK : ecuda(e, err, "append launch");
}

int fns_b200_engine_verify(fns_b200_engine * e, const void * logits, int dtype, int64_t row_stride, int windows,
                           int n_draft, const int32_t * draft_host, const uint32_t * masks_host,
                           const fns_b200_params * params_host, int32_t * tokens_host, int32_t * accept_host,
                           void * stream) {
    if (!e) return FNS_B200_ERR_ARG;
    if (!logits || !params_host || !tokens_host || !accept_host || windows <= 0 || n_draft < 0 || (n_draft > 0 && !draft_host))
        return efail(e, FNS_B200_ERR_ARG, "verify: null argument or windows <= 0");
    const int rows = windows * (n_draft + 1);
    if (rows > e->max_rows) return efail(e, FNS_B200_ERR_CAPACITY, "verify: windows * (n_draft + 1) beyond the engine's limit");
    Dev g(e->device);
    cudaStream_t st = (cudaStream_t) stream;
    Slot & s = e->slot[e->head];
    if (s.busy) return efail(e, FNS_B200_ERR_ARG, "verify: picks in flight, call pick_wait first");
    cudaError_t err = cudaSuccess;
    if (masks_host && (err = stage(s.masks_h, s.masks_d, masks_host, (size_t) rows * e->words, st)) != cudaSuccess)
        return ecuda(e, err, "verify mask copy");
    if (n_draft > 0 && (err = stage(s.draft_h, s.draft_d, draft_host, (size_t) windows * n_draft, st)) != cudaSuccess)
        return ecuda(e, err, "verify draft copy");
    if ((err = stage(s.params_h, s.params_d, params_host, (size_t) windows, st)) != cudaSuccess)
        return ecuda(e, err, "verify params copy");
    const bool hist = e->max_history > 0;
    const int rc = fns_b200_verify_accept(e->sampler, logits, dtype, row_stride, e->vocab, windows, n_draft, s.draft_d,
                                          masks_host ? s.masks_d : nullptr, e->words, hist ? e->sess_history : nullptr,
                                          hist ? e->max_history : 0, hist ? e->sess_history_len : nullptr, s.params_d,
                                          s.tokens_d, s.accept_d, st);
    if (rc != FNS_B200_OK) return esampler(e, rc);
    if ((err = cudaMemcpyAsync(s.tokens_h, s.tokens_d, (size_t) rows * sizeof(int32_t), cudaMemcpyDeviceToHost, st)) != cudaSuccess ||
        (err = cudaMemcpyAsync(s.accept_h, s.accept_d, (size_t) windows * sizeof(int32_t), cudaMemcpyDeviceToHost, st)) != cudaSuccess ||
        (err = cudaStreamSynchronize(st)) != cudaSuccess)
        return ecuda(e, err, "verify copy back");
    std::memcpy(tokens_host, s.tokens_h, (size_t) rows * sizeof(int32_t));
    std::memcpy(accept_host, s.accept_h, (size_t) windows * sizeof(int32_t));
    e->last_tokens = s.tokens_d;
    return FNS_B200_OK;
}

int fns_b200_lookup_draft(const int32_t * h, int n_h, int want, int32_t * out) {
    if (!h || !out || n_h < 0 || want <= 0) return 0;
    for (int n = 4; n >= 2; --n) {
        if (n_h < n + 1) continue;
        const int32_t * tail = h + n_h - n;
        for (int s = n_h - n - 1; s >= 0; --s) {
            bool same = true;
            for (int j = 0; j < n && same; ++j) same = h[s + j] == tail[j];
            if (!same) continue;
            int k = 0;
            for (; k < want && s + n + k < n_h; ++k) out[k] = h[s + n + k];
            if (k > 0) return k;
        }
    }
    return 0;
}

}  // extern "C"
