/* fns_b200.h - C ABI of the B200 (sm_100a) token sampler: logits -> token for one decoding step.
 *
 * Plain C: pointers and sizes only.  Unless a name ends in `_host`, every data pointer is DEVICE memory owned
 * by the caller; every call is asynchronous on the caller's stream (a cudaStream_t passed as void *; NULL is
 * the default stream) and performs no host synchronisation and no allocation.  The library owns only the
 * workspace created by fns_b200_create.  Every function returns a status (0 = FNS_B200_OK) and never aborts.
 *
 * Each entry point names the interface of the reference (NomenAK/FlintNSteel) that it replaces.
 */
#ifndef FNS_B200_H
#define FNS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    FNS_B200_OK = 0,
    FNS_B200_ERR_ARG = 1,      /* null pointer, size out of range, misuse */
    FNS_B200_ERR_CUDA = 2,     /* a CUDA call failed; see fns_b200_last_error */
    FNS_B200_ERR_CAPACITY = 3, /* rows / vocab / history beyond what the handle was created for */
    FNS_B200_ERR_DEVICE = 4    /* a kernel recorded an internal error (fns_b200_device_status) */
};

enum { FNS_B200_F32 = 0, FNS_B200_BF16 = 1 };

/* Empty candidate slot, as the reference's (-FLT_MAX, 0x7fffffff) (src/kernels.cu:632-633). */
#define FNS_B200_EMPTY_ID 0x7fffffff
/* Largest k_cap a handle accepts.  k_cap = 64 is the reference's kSampleMaxK (src/kernels.cu:598). */
#define FNS_B200_MAX_K 1024
#define FNS_B200_MAX_HISTORY 65000
/* Verification window width limit; the reference's engine uses at most 8 columns (src/engine.cu:74,718). */
#define FNS_B200_MAX_WINDOW 32

/* Per-row sampling parameters; an array of these lives in device memory.
 * Extends fns::SampleParams (include/fns/engine.h:75-84: temperature, top_p, top_k, seed, presence_penalty)
 * with the Philox counter that Engine::pick_async takes beside it (src/engine.cu:823) and with min_p,
 * repetition and frequency, which the reference does not have (neutral values: 0, 1, 0).
 *   temperature <= 0 : greedy, first candidate in the total order (src/kernels.cu:701)
 *   top_k <= 0 or > k_cap : k_cap candidates (src/kernels.cu:778)
 *   top_p : cut on the temperature-1 softmax over the k candidates (src/kernels.cu:702-710)
 *   min_p : after the top-p cut, keep the longest prefix with exp(v_j - v_0) >= min_p
 *   penalties, for an id that occurs c > 0 times in the row's history, fp32, each step rounded:
 *       x = x > 0 ? x / repetition : x * repetition;  x -= frequency * c;  x -= presence
 *     (with repetition 1 and frequency 0: the reference's x - presence * seen, src/kernels.cu:726) */
typedef struct fns_b200_params {
    float temperature;
    float top_p;
    float min_p;
    float repetition;
    float presence;
    float frequency;
    int32_t top_k;
    int32_t reserved;
    uint64_t seed;
    uint64_t counter;
} fns_b200_params;

/* One top-k candidate: penalised logit and GLOBAL token id.  Lists are sorted in the reference's total order
 * (value descending, then id ascending, src/kernels.cu:594) and padded with (-FLT_MAX, FNS_B200_EMPTY_ID).
 * This is the (value, id) pair the reference keeps in g_cand_v / g_cand_i (src/kernels.cu:601-602) and the
 * unit that vocabulary shards exchange. */
typedef struct fns_b200_cand {
    float value;
    int32_t id;
} fns_b200_cand;

typedef struct fns_b200_sampler fns_b200_sampler;

/* Workspace for up to max_rows rows of up to max_vocab logits per call, k_cap in [1, FNS_B200_MAX_K], histories
 * of up to max_history ids per row.  Replaces the reference's file-scope candidate arrays
 * (src/kernels.cu:601-602), which make its sampler one-row-at-a-time; a handle serves one stream at a time,
 * separate handles run concurrently.  Allocates device memory on `device` (the only allocating call besides
 * the lazy default handle of the fns::k compatibility layer). */
int fns_b200_create(int device, int max_rows, int max_vocab, int k_cap, int max_history, fns_b200_sampler ** out);
int fns_b200_destroy(fns_b200_sampler * s);
/* Text of the last failure on this handle (host string, valid until the next call on the handle). */
const char * fns_b200_last_error(const fns_b200_sampler * s);
/* Synchronises the stream and returns FNS_B200_ERR_DEVICE if a kernel of this handle recorded an internal
 * error since the last call: a bulk copy into shared memory that did not complete within the kernel's bounded wait
 * (the rows of that call are then not valid).  For tests; the sampling calls themselves never synchronise. */
int fns_b200_device_status(fns_b200_sampler * s, void * stream);
int fns_b200_k_cap(const fns_b200_sampler * s);

/* Rows of logits -> one token id per row.
 * Replaces, for each row, the launch sequence of Engine::pick_async (src/engine.cu:837-843):
 *   k::presence_apply (src/kernels.cuh:79)  +  k::argmax (:69) or k::sample (:74-75)
 * in one fused pass that leaves the logits untouched.
 *   logits       [rows][row_stride] elements of `dtype`; the first `vocab` of each row are used
 *   masks        NULL, or [rows][mask_stride_words] packed uint32, token i <-> bit (i & 31) of word (i >> 5),
 *                1 = allowed: the xgrammar bitmask as Engine::pick_async receives it
 *                (include/fns/engine.h:115, src/kernels.cu:635)
 *   history      NULL, or [rows][history_stride] token ids, of which history_len[r] are used for row r;
 *                ids outside [0, vocab) are ignored (src/kernels.cu:730)
 *   params       [rows]
 *   out_tokens   [rows] int32; -1 when no allowed finite candidate exists (src/kernels.cu:700) */
int fns_b200_sample_rows(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
                         const uint32_t * masks, int64_t mask_stride_words, const int32_t * history,
                         int64_t history_stride, const int32_t * history_len, const fns_b200_params * params,
                         int32_t * out_tokens, void * stream);

/* The same when rows share masks: row r reads the mask masks[mask_rows[r]] (device int32[rows]).  Serves a device-side
 * cache of grammar states (fns_b200_engine_pick_async_dl): a state's mask is uploaded once and named by its slot. */
int fns_b200_sample_rows_shared_masks(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab,
                                      int rows, const uint32_t * masks, int64_t mask_stride_words, const int32_t * mask_rows,
                                      const int32_t * history, int64_t history_stride, const int32_t * history_len,
                                      const fns_b200_params * params, int32_t * out_tokens, void * stream);

/* One row with parameters passed by value from the host: the shape of k::sample / k::argmax
 * (src/kernels.cuh:69,74-75).  `params_host` is read during the call. */
int fns_b200_sample_one(fns_b200_sampler * s, const void * logits, int dtype, int vocab, const uint32_t * mask,
                        const int32_t * history, int history_len, const fns_b200_params * params_host,
                        int32_t * out_token, void * stream);

/* Sampling for hosts that must not allocate GPU memory: the same result as fns_b200_sample_rows with k_cap = 64,
 * without a handle.  (No counterpart in the reference; its sampler keeps its candidates in file-scope device
 * arrays too, src/kernels.cu:601-602, but nothing there is exposed as an interface.)
 *
 * Who needs it: an engine that gives the whole GPU to its own memory arena at start-up, so that a later cudaMalloc
 * fails or is forbidden, and call sites where an allocation is unacceptable because it synchronises the device.
 * fns_b200_create allocates; this entry point, and everything it calls, never calls cudaMalloc, cudaFree or any
 * allocating routine.  What a handle would own (the slices' candidate lists, one ticket per row, an error flag)
 * lives in a static device array of 2 MiB + 512 bytes that every GPU loading the library holds until exit.
 *
 * Limits: rows <= 64 per call, k_cap fixed at 64 (params.top_k <= 0 or > 64 means 64); larger calls are refused
 * with FNS_B200_ERR_CAPACITY and a text in error_text (may be NULL).  All other arguments as
 * fns_b200_sample_rows; `device` is the GPU that owns the buffers.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device) and loads
 * and configures every kernel the entry point can launch, whatever the shape of that first call: make it before
 * starting any stream capture; later calls of any shape set nothing up.
 * All calls on a GPU share the one array, which keeps the previous call's contents (this call clears what has to
 * start at zero): calls that overlap on the GPU, on any streams, race with each other; issue them on one stream
 * or order them with events. */
int fns_b200_sample_rows_noalloc(int device, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
                                 const uint32_t * masks, int64_t mask_stride_words, const int32_t * history,
                                 int64_t history_stride, const int32_t * history_len, const fns_b200_params * params,
                                 int32_t * out_tokens, void * stream, char * error_text, int error_len);

/* First half of the path only: per-row top-k candidates of a vocabulary SHARD, in the total order.
 * The reference does the same per slice in k_topk_part (src/kernels.cu:624-648); here a shard is the slice
 * that one GPU owns.  `id_base` is the global id of the shard's element 0: history ids are global, reported
 * ids are global, `masks` points at the shard's own words (id_base must be a multiple of 32).
 *   out_cands    [rows][k_cap]; entries beyond the row's k are empty */
int fns_b200_select_rows(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
                         int32_t id_base, const uint32_t * masks, int64_t mask_stride_words,
                         const int32_t * history, int64_t history_stride, const int32_t * history_len,
                         const fns_b200_params * params, fns_b200_cand * out_cands, void * stream);

/* Second half of the path: merge `lists` candidate lists per row (e.g. one per vocabulary shard, gathered into
 * local memory) and draw.  This is k_sample (src/kernels.cu:671-721): selection rounds over the slices'
 * candidates, then softmax / top-p / temperature / Philox draw.
 *   cands        entry j of list l of row r is cands[r * row_stride + l * list_stride + j] (strides in entries);
 *                lists * list_len <= 8192.  [rows][lists][list_len] is (row_stride = lists * list_len,
 *                list_stride = list_len); an all-gather of per-shard [rows][k_cap] blocks is
 *                (row_stride = k_cap, list_stride = rows * k_cap).  Lists of more than 64 entries must be what
 *                fns_b200_select_rows writes: descending in the total order, empty entries last, no key in two
 *                lists (shards do not overlap); shorter lists may come in any order
 *   out_cands    NULL, or [rows][k_cap]: the merged list, for inspection */
int fns_b200_finalize_rows(fns_b200_sampler * s, const fns_b200_cand * cands, int lists, int list_len,
                           int64_t list_stride, int64_t row_stride, int rows, const fns_b200_params * params,
                           int32_t * out_tokens, fns_b200_cand * out_cands, void * stream);

/* Speculative verification of `windows` windows of W = n_draft + 1 logit rows each (row = window * W + c).
 * Replaces the per-column loop of Engine::verify (src/engine.cu:750-757: k::presence_apply_col + k::argmax /
 * k::sample with counter + c) and moves the host accept loop (tools/fns_serve/fns_serve.cpp:492-508) onto
 * the device.  Column c is penalised with the window's history plus draft[0 .. c) (src/kernels.cu:738-741).
 *   draft        [windows][n_draft] token ids proposed for columns 1 .. n_draft
 *   params       [windows]; column c draws with params.counter + c
 *   out_tokens   [windows][W]
 *   out_accept   [windows]: a = number of leading c < n_draft with out_tokens[c] == draft[c]; the tokens to
 *                emit are out_tokens[0 .. a] */
int fns_b200_verify_accept(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab,
                           int windows, int n_draft, const int32_t * draft, const uint32_t * masks,
                           int64_t mask_stride_words, const int32_t * history, int64_t history_stride,
                           const int32_t * history_len, const fns_b200_params * params, int32_t * out_tokens,
                           int32_t * out_accept, void * stream);

/* Dense presence state of the reference, kept for callers that drive it directly (src/kernels.cuh:77-88).
 * Same arithmetic, same in-place update of the logits. */
int fns_b200_presence_apply(float * x, const float * seen, int n, float penalty, void * stream);        /* :79 */
int fns_b200_presence_mark(float * seen, const int32_t * token, void * stream);                         /* :80 */
int fns_b200_presence_apply_col(float * x, const float * seen, const int32_t * draft, int c, int n,
                                float penalty, void * stream);                                          /* :83-84 */
int fns_b200_presence_mark_n(float * seen, const int32_t * tokens, int n, void * stream);               /* :85 */
int fns_b200_io_advance(int32_t * io, int pos, void * stream);                                          /* :88 */

/* Number of kernels this handle has launched since it was created (benchmarks report it). */
int64_t fns_b200_launch_count(const fns_b200_sampler * s);
/* Per-kernel device timing for benchmarks: between profile_begin and profile_end every sampling call on the
 * handle brackets its select kernel and its finalize kernel with CUDA events recorded on the caller's stream
 * (at most max_calls calls are recorded).  profile_end synchronises the stream and returns the summed
 * durations in milliseconds and the number of calls recorded. */
int fns_b200_profile_begin(fns_b200_sampler * s, int max_calls);
int fns_b200_profile_end(fns_b200_sampler * s, void * stream, double * select_ms, double * finalize_ms, int * calls);

/* ---- host-side glue: the sampler part of fns::Engine ---------------------------------------------------------
 * The reference's Engine stages the host bitmask through pinned memory, launches the sampler after the forward
 * pass on its stream, copies the 4-byte token back and records an event (Engine::pick_async / pick_wait,
 * src/engine.cu:823-852); Engine::verify does the same for a window and synchronises (src/engine.cu:733-765).
 * fns_b200_engine is that glue for `rows` independent sessions at once.  Pointers ending in _host are host
 * memory (pageable is accepted; it is staged through the engine's pinned buffers, as src/engine.cu:833 does).
 * Two picks may be in flight; pick_wait returns them in order. */
typedef struct fns_b200_engine fns_b200_engine;

int fns_b200_engine_create(int device, int max_rows, int vocab, int k_cap, int max_history, fns_b200_engine ** out);
int fns_b200_engine_destroy(fns_b200_engine * e);
const char * fns_b200_engine_last_error(const fns_b200_engine * e);
fns_b200_sampler * fns_b200_engine_sampler(fns_b200_engine * e);

/* Engine::pick_async (src/engine.cu:823-847).  logits: device [rows][row_stride], or host memory when
 * logits_on_host has FNS_B200_HOST_LOGITS set (then they reach the device inside the call).  masks_host: NULL or
 * [rows][ceil(vocab / 32)].  history_host: NULL to use the sessions' device-side histories (see
 * fns_b200_engine_reset / append), else [rows][history_stride] with history_len_host[rows].
 *
 * By default every host buffer is copied into the engine's own pinned memory before the call returns, so the
 * caller may reuse it at once (what src/engine.cu:833 does).  With FNS_B200_HOST_STABLE the caller promises to
 * leave its host buffers unchanged until the matching pick_wait; buffers that are page-locked (cudaHostAlloc,
 * cudaHostRegister) are then read by the GPU where they lie: masks, histories and parameters by one DMA each
 * without the intermediate memcpy, and - when a mask is given - the logits by the kernel itself, which loads
 * only the 16-byte vectors that hold an allowed id, so masked-out logits never cross PCIe.  Pageable buffers are
 * staged as before. */
#define FNS_B200_HOST_LOGITS 1
#define FNS_B200_HOST_STABLE 2
int fns_b200_engine_pick_async(fns_b200_engine * e, const void * logits, int logits_on_host, int dtype,
                               int64_t row_stride, int rows, const uint32_t * masks_host,
                               const int32_t * history_host, int64_t history_stride,
                               const int32_t * history_len_host, const fns_b200_params * params_host, void * stream);
/* The bitmask as its producer hands it over.  fns-serve gives the sampler xgrammar's own tensor: a DLTensor of int32 on
 * the CPU with GetBitmaskSize(vocab) = ceil(vocab / 32) words, refilled per token by FillNextTokenBitmask and per
 * window column into [W][words] (tools/fns_serve/fns_serve.cpp:306-328, 340-354; bit order tests/xgrammar_smoke.cpp:87-102).
 * fns_b200_dl_tensor has the layout of DLTensor (dlpack.h), so a `const DLTensor *` can be passed as it is. */
typedef struct fns_b200_dl_tensor {
    void * data;
    int32_t device_type; /* 1 = kDLCPU, 3 = kDLCUDAHost */
    int32_t device_id;
    int32_t ndim;        /* 1: [words], 2: [rows][words] */
    uint8_t dtype_code;  /* 0 = kDLInt (what xgrammar uses), 1 = kDLUInt */
    uint8_t dtype_bits;  /* 32 */
    uint16_t dtype_lanes;
    int64_t * shape;
    int64_t * strides;   /* NULL = compact; in elements */
    uint64_t byte_offset;
} fns_b200_dl_tensor;
/* Checks the tensor against the vocabulary and returns its rows, the first word and the row stride in words. */
int fns_b200_mask_view(const fns_b200_dl_tensor * t, int vocab, int * rows, const uint32_t ** words_host, int64_t * stride_words);
/* Keeps up to `slots` masks on the device, one per grammar state (0 frees the cache).  A matcher that is in a state it
 * has been in before produces the same mask: with the cache that mask is not uploaded again. */
int fns_b200_engine_mask_cache(fns_b200_engine * e, int slots);
int fns_b200_engine_mask_stats(const fns_b200_engine * e, int64_t * hits, int64_t * misses, int64_t * bytes_uploaded);
/* Engine::pick_async with the producer's tensor (one mask row, or one per logit row; NULL = unmasked).  Logits on the
 * device, session histories on the device (fns_b200_engine_append).  mask_states_host NULL: the masks are staged and
 * uploaded as in fns_b200_engine_pick_async.  Else mask_states_host[rows] names every row's grammar state (any 64-bit
 * id the caller keeps per matcher state; FNS_B200_NO_MASK = this row is unmasked): a state the cache holds uploads
 * nothing, a new one replaces the state that was not asked for longest.  All picks of an engine that use the cache
 * must be issued on one stream (the uploads are ordered with the kernels that read the slots by that stream). */
#define FNS_B200_NO_MASK 0xffffffffffffffffull
int fns_b200_engine_pick_async_dl(fns_b200_engine * e, const void * logits, int dtype, int64_t row_stride, int rows,
                                  const fns_b200_dl_tensor * masks, const uint64_t * mask_states_host,
                                  const fns_b200_params * params_host, void * stream);
/* ceil(vocab / 32): the words of one mask row of this engine (xgrammar::GetBitmaskSize, src/engine.cu:825). */
int fns_b200_engine_words(const fns_b200_engine * e);
/* Engine::pick_wait (src/engine.cu:849-852): waits for the oldest pick in flight; tokens_host[rows]. */
int fns_b200_engine_pick_wait(fns_b200_engine * e, int32_t * tokens_host);
/* The tokens of the latest pick where the GPU can read them (the reference's io_ + 2), for a forward pass that is
 * queued before the host has seen the token (Engine::step_next, src/engine.cu:796-800).  After a pick of one row this
 * is a page-locked host word that the GPU addresses (the kernel writes the token there and nothing is copied back);
 * after a pick of several rows it is device memory. */
const int32_t * fns_b200_engine_device_tokens(const fns_b200_engine * e);
/* Engine::reset_presence (src/engine.cu:854-860): forgets the device-side history of every session. */
int fns_b200_engine_reset(fns_b200_engine * e, void * stream);
/* Engine::presence_commit / k::presence_mark (src/engine.cu:843,862-866): appends, per session, the first
 * counts_host[r] of tokens [rows][tokens_stride] (device memory; ids < 0 are skipped) to the device-side
 * history.  counts_host NULL: one token per session. */
int fns_b200_engine_append(fns_b200_engine * e, const int32_t * tokens, int64_t tokens_stride, int rows,
                           const int32_t * counts_host, void * stream);
/* Engine::verify, sampler part (src/engine.cu:733-765), for `windows` windows of n_draft + 1 rows, with the
 * accept rule of fns-serve (tools/fns_serve/fns_serve.cpp:492-508) computed on the device.  Synchronous, like the
 * reference.  draft_host [windows][n_draft]; masks_host NULL or [windows * (n_draft + 1)][words];
 * tokens_host [windows][n_draft + 1]; accept_host [windows]. */
int fns_b200_engine_verify(fns_b200_engine * e, const void * logits, int dtype, int64_t row_stride, int windows,
                           int n_draft, const int32_t * draft_host, const uint32_t * masks_host,
                           const fns_b200_params * params_host, int32_t * tokens_host, int32_t * accept_host,
                           void * stream);
/* Prompt-lookup draft (include/fns/lookup.h:12-27) on the host: the continuation of the latest earlier
 * occurrence of the final n-gram of the history, n = 4 down to 2.  Returns the number of ids written. */
int fns_b200_lookup_draft(const int32_t * history_host, int n_history, int want, int32_t * out_host);

/* The same draft for a batch of sessions on the device: history [rows][history_stride] with history_len[rows];
 * out [rows][out_stride] receives at most `want` ids per row, out_n[rows] their count. */
int fns_b200_lookup_draft_rows(const int32_t * history, int64_t history_stride, const int32_t * history_len, int rows,
                               int want, int32_t * out, int64_t out_stride, int32_t * out_n, void * stream);

/* ---- the speculation driver of fns-serve (tools/fns_serve/fns_serve.cpp:340-354, 410-519) ----------------------------
 * Host code.  The grammar matcher and the model stay the caller's, behind callbacks. */
typedef struct fns_b200_grammar {  /* xgrammar::GrammarMatcher as fns-serve drives it */
    void * user;
    void (*fill)(void * user, int32_t * mask_words);   /* FillNextTokenBitmask into ceil(vocab / 32) words */
    int (*accept)(void * user, int32_t token);         /* AcceptToken: 0 = rejected */
    int (*terminated)(void * user);                    /* IsTerminated; may be NULL */
    void (*rollback)(void * user, int tokens);         /* Rollback */
} fns_b200_grammar;
/* Masks for the columns of a window (fns_serve.cpp:340-354): column c's mask follows the committed prefix plus
 * draft[0 .. c).  wmask [(nd + 1)][words].  Returns the number of usable columns W (a draft id the grammar rejects
 * cuts the window) and leaves the matcher at the committed prefix; without a grammar (g NULL) W = nd + 1. */
int fns_b200_spec_window_masks(const fns_b200_grammar * g, const int32_t * draft, int nd, int words, uint32_t * wmask);

typedef struct fns_b200_spec_counters {  /* the counters of fns-serve's "done" line (fns_serve.cpp:523-532) */
    int32_t generated, windows, drafted, accepted, emitted, skipped, iterations;
} fns_b200_spec_counters;
/* The accept / commit loop over one verified window (fns_serve.cpp:486-508): out[W] are the columns' choices; the
 * choice of column c is committed while every earlier column matched its draft.  committed[W] receives the tokens to
 * emit, *engaged their number (what Engine::presence_commit takes).  Returns 0 = go on, 1 = a stop token was
 * committed, 2 = max_tokens reached, negative = argument error / token rejected by the grammar. */
int fns_b200_spec_commit(const int32_t * out, int W, const int32_t * draft, int nd, const int32_t * stop, int n_stop,
                         int max_tokens, const fns_b200_grammar * g, fns_b200_spec_counters * c, int32_t * committed,
                         int * engaged, int * window_accepted, int * window_offered);

/* Adaptive window width (fns_serve.cpp:430-459): from the acceptance rate of this request and the measured cost of
 * windows of each width, the number of draft ids that maximises expected tokens per unit of time (0 = do not
 * speculate this step).  Costs are exponentially weighted means of wall-clock seconds and persist across requests. */
typedef struct fns_b200_spec_policy {
    int32_t spec;                /* widest window (columns) */
    int32_t skipped_proposals;
    uint64_t accepted, offered;  /* of this request */
    double cost[FNS_B200_MAX_WINDOW + 1];  /* cost[w]: a window of w columns; cost[1]: an ordinary step; 0 = unknown */
} fns_b200_spec_policy;
void fns_b200_spec_policy_init(fns_b200_spec_policy * p, int spec);
void fns_b200_spec_policy_new_request(fns_b200_spec_policy * p);
int fns_b200_spec_choose_width(fns_b200_spec_policy * p, int nd_max);
void fns_b200_spec_observe(fns_b200_spec_policy * p, int width, double elapsed_s, int window_accepted, int window_offered);

/* The model behind the sampler: logits of W columns, column c after ids[0 .. c] at positions p0 .. p0 + c
 * (Engine::prefill / step_logits / verify's forward pass).  *logits: device [W][*row_stride]. */
typedef struct fns_b200_model {
    void * user;
    int (*forward)(void * user, const int32_t * ids, int W, int p0, const void ** logits, int64_t * row_stride);
} fns_b200_model;
/* The decode loop of fns-serve for one request (fns_serve.cpp:383-521): sequential when spec <= 1, else
 * speculative with prompt-lookup drafts of up to spec - 1 ids, verification windows (fns_b200_engine_verify), the
 * accept rule and presence_commit.  Column c draws with Philox counter (generated-token index), so both modes give
 * the same tokens for the same seed.  e: an engine for one session with max_rows >= spec (and max_history >=
 * max_tokens when a penalty is set).  out_tokens[max_tokens]; counters->generated is their number. */
int fns_b200_spec_decode(fns_b200_engine * e, const fns_b200_model * m, const fns_b200_grammar * g, const int32_t * prompt,
                         int n_prompt, int max_tokens, const int32_t * stop, int n_stop, const fns_b200_params * sp, int dtype,
                         int spec, fns_b200_spec_policy * policy, int32_t * out_tokens, fns_b200_spec_counters * counters,
                         void * stream);

/* The sampling fields of one request line of fns-serve (fns_serve.cpp:291-303, defaults serve/fns_server.py:387-395):
 * "temperature" (0 = greedy), "top_p" (1), "top_k" (0 = k_cap), "seed" (0), "presence_penalty" (0), and this
 * library's "min_p" (0), "repetition_penalty" (1), "frequency_penalty" (0).  A missing or non-numeric field keeps
 * its default; counter is set to 0 (the caller counts generated tokens). */
int fns_b200_params_from_json(const char * json_line, fns_b200_params * out);

/* ---- multi-GPU dispatcher ---------------------------------------------------------------------------------------
 * No counterpart in the reference, which is single-GPU and samples one row per call (docs/ENGINE.md:132).  One
 * process per GPU; every rank creates a dispatcher with its own rank.  Two partitions of the sampler's work:
 *   FNS_B200_MG_ROWS   independent sessions: every rank samples the rows its own LM head produced; no collective
 *                      on the data path (fns_b200_mg_gather_tokens collects the tokens afterwards if wanted)
 *   FNS_B200_MG_VOCAB  one large vocabulary split evenly on 32-id boundaries: per-shard top-k_cap
 *                      (fns_b200_select_rows), ONE NCCL all-gather of the (value, id) lists over NVLink
 *                      (k_cap * 8 bytes per row and rank), then the merge + draw (fns_b200_finalize_rows) on every
 *                      rank, so every rank ends with the same tokens.  The result does not depend on the number of
 *                      shards: the global top-k lies in the union of the shards' top-k (the reference's argument
 *                      for its 128 slices, src/kernels.cu:594-597) and the merge orders by (value, id) alone.
 * All three steps are enqueued on the caller's stream with no host work in between.  NCCL is loaded at run time
 * (libnccl.so.2) and only when world > 1. */
typedef struct fns_b200_mg fns_b200_mg;
enum { FNS_B200_MG_ROWS = 0, FNS_B200_MG_VOCAB = 1 };
#define FNS_B200_MG_ID_BYTES 128
/* ncclGetUniqueId: rank 0 calls it and hands the 128 bytes to every rank (by whatever channel the host has). */
int fns_b200_mg_unique_id(void * id_host);
/* Collective over the ranks when world > 1 (ncclCommInitRank) unless nccl_comm, an existing ncclComm_t of the same
 * ranks, is given (then unique_id_host may be NULL; the communicator stays the caller's).  vocab is the FULL
 * vocabulary in both modes; in VOCAB mode k_cap * world <= 8192. */
int fns_b200_mg_create(int device, int rank, int world, int mode, int max_rows, int vocab, int k_cap, int max_history,
                       const void * unique_id_host, void * nccl_comm, fns_b200_mg ** out);
int fns_b200_mg_destroy(fns_b200_mg * m);
const char * fns_b200_mg_last_error(const fns_b200_mg * m);
/* What this rank owns: ROWS: rows [lo, hi) of a batch of total_rows; VOCAB: token ids [lo, hi) (lo a multiple of 32). */
int fns_b200_mg_range(const fns_b200_mg * m, int total_rows, int * lo, int * hi);
/* ROWS: as fns_b200_sample_rows on this rank's rows.  VOCAB: logits are [rows][row_stride] holding this rank's ids
 * [lo, hi) of every row, masks the matching words [rows][mask_stride_words] (word 0 = ids lo .. lo + 31), history
 * GLOBAL ids; out_tokens [rows] is the same on every rank.  Every rank must make the same sequence of calls. */
int fns_b200_mg_sample_rows(fns_b200_mg * m, const void * logits, int dtype, int64_t row_stride, int rows,
                            const uint32_t * masks, int64_t mask_stride_words, const int32_t * history,
                            int64_t history_stride, const int32_t * history_len, const fns_b200_params * params,
                            int32_t * out_tokens, void * stream);
/* ROWS: every rank receives the tokens of all total_rows rows in row order (one all-gather of 4 bytes per row). */
int fns_b200_mg_gather_tokens(fns_b200_mg * m, const int32_t * local_tokens, int total_rows, int32_t * all_tokens,
                              void * stream);
/* Device time of the three steps for benchmarks (CUDA events on the caller's stream around select, exchange and
 * finalize of every call between begin and end); end synchronises the stream and returns microseconds per call. */
int fns_b200_mg_profile_begin(fns_b200_mg * m, int max_calls);
int fns_b200_mg_profile_end(fns_b200_mg * m, void * stream, double * select_us, double * exchange_us,
                            double * finalize_us, int * calls);

#ifdef __cplusplus
}
#endif
#endif /* FNS_B200_H */
