// fns_sampler.cu - the sampler kernels for sm_100a and the C ABI declared in include/fns_b200.h.
//
// HBM-streaming / latency work with no contraction in it (no tensor cores):
//
//   k_select   grid (slices, rows); one block per (row, slice).  With many rows a slice is the whole row and a
//              block has 512 threads (two per SM: 296 rows in flight at once); with few rows a row is cut into
//              slices of 256-thread blocks so that the whole GPU works on it.  Per slice:
//                1. the grammar bitmask and the penalty history are folded into a shared-memory bit set;
//                2. pass 1 streams the logits once with 128-bit coalesced loads, two epochs in flight, and keeps
//                   nothing but maxima: per thread the maximum seen, per vector group one flag "reaches the
//                   running bound".  The bound is a value that at least k elements of the slice are known to
//                   reach, found with warp-wide max reductions over the threads' maxima; nothing is appended,
//                   nothing is compared element by element, regions the bit set masks out are never loaded;
//                3. pass 2 reads the flagged groups again (L2) and appends the elements that reach the final
//                   bound (about k to 2k of them) to a shared buffer; penalised candidates join them;
//                4. the best k of the buffer, sorted, are the slice's answer (rank by counting, or radix select
//                   when an adversarial input has filled the buffer; the buffer is compacted whenever it fills,
//                   so any input is handled exactly);
//                5. the last block of a row to finish (a ticket, no waiting) merges the slices' lists and does
//                   the candidate softmax, top-p / min-p cut, temperature weights and Philox draw.
//              Replaces k_topk_part (src/kernels.cu:624-648, which rescans its slice k times), k_presence_apply /
//              _col (src/kernels.cu:724-742, which rewrite the whole row) and k_sample (src/kernels.cu:671-721)
//              of the reference: a whole call is ONE launch.
//   k_finalize grid (rows).  The merge + draw as a kernel of its own, for candidate lists that come from
//              elsewhere (vocabulary shards gathered from other GPUs).
//
// Nothing here waits on another block, so there is no spin loop anywhere in the sampler.
#include "fns_device.cuh"

#include <cooperative_groups.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <mutex>
#include <vector>

namespace fnsb {

#ifdef FNS_PHASE_TIMING  // development aid: block time per phase, summed over blocks (thread 0's clock)
__device__ unsigned long long g_phase[16];
#define FNS_PHASE_BEGIN long long ph_t = clock64();
#define FNS_PHASE(i)                                                           \
    if (threadIdx.x == 0) {                                                    \
        const long long ph_n = clock64();                                      \
        atomicAdd(&g_phase[i], (unsigned long long) (ph_n - ph_t));            \
        ph_t = ph_n;                                                           \
    }
#define FNS_MARK(i) __syncthreads(); FNS_PHASE(i)
#else
#define FNS_PHASE_BEGIN
#define FNS_PHASE(i)
#define FNS_MARK(i)
#endif

constexpr int kHashEmpty = -1;
constexpr int kMaxMergeKeys = 8192;   // k_finalize holds the lists of one row in shared memory
constexpr int kMaxSlices = 128;
constexpr int kEpochElems = 16;       // elements per thread and epoch
// epochs per slice: at most 16 for 256-thread blocks and 32 for 512-thread blocks (64 flag bits per thread)
constexpr int kMaxWarps = 16;
constexpr int kRankSelectMax = 384;   // candidate sets up to this size are ranked by counting

struct SelectArgs {
    const void * logits;
    int64_t row_stride;
    int vocab;
    int id_base;
    const uint32_t * masks;
    int64_t mask_stride;
    const int32_t * history;
    int64_t history_stride;
    const int32_t * history_len;
    const int32_t * draft;  // verification windows: [windows][n_draft]; row = window * (n_draft + 1) + column
    int n_draft;
    const fns_b200_params * params;  // per window (per row when n_draft == 0); null: p0
    fns_b200_params p0;
    int k_cap;
    int slices;
    int slice_len;   // a multiple of the block's epoch
    int cap;         // candidate buffer entries (>= 4 * k_cap)
    int trigger;     // compact when the buffer holds this many
    int ht_size;     // history table slots (power of two >= 1024), 0: no table
    int ht_shift;    // 32 - log2(ht_size): the table index is the high bits of a multiplicative hash
    int stash_cap;   // entries of the flagged-vector stash
    int list_cap;    // entries of the allowed-vector list (it shares the stash's memory)
    uint64_t * cand;  // [rows][slices][k_cap] sorted keys, 0 = empty
    unsigned * tickets;         // [rows], zero between launches
    int32_t * out_tokens;       // [rows], may be null
    fns_b200_cand * out_cands;  // [rows][k_cap], may be null
    int * err;
};

struct SelectShared {
    SelectScratch sc;
    uint64_t thr_key;     // the exact k-th best key of the buffer at its last compaction
    uint32_t n_cand;      // append cursor; may run past cap (the excess was not stored: see `lost`)
    uint32_t epoch_mask;  // epochs of the slice that have an allowed element
    uint32_t n_list;      // occupied slots of the history table
    uint32_t n_stash;     // flagged vectors kept in shared memory for pass 2
    uint32_t n_av;        // vectors of the slice with an allowed element
    uint32_t n_vl;        // cursor of the allowed-vector list
    int keep;
    int is_last;
    __align__(16) uint32_t warp_bound[kMaxWarps];  // per warp: a value that r of its lanes have reached
    uint64_t red[kMaxWarps];
};

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

// 16-byte load of VEC consecutive elements, widened to fp32.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T * p, float (&out)[VEC]) {
    if constexpr (VEC == 1) {
        out[0] = to_float(*p);
    } else if constexpr (sizeof(T) == 4) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
        out[0] = v.x;
        out[1] = v.y;
        out[2] = v.z;
        out[3] = v.w;
    } else {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[2 * j] = __uint_as_float(w[j] << 16);
            out[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

// One key into the candidate buffer.  False when the buffer is full: the caller remembers the element and
// offers it again after the next compaction.  One reservation serves all the lanes that are here together:
// atomics on one shared word serialise.
__device__ __forceinline__ bool push(uint64_t key, uint64_t * buf, SelectShared & sh, int cap) {
    const cooperative_groups::coalesced_group g = cooperative_groups::coalesced_threads();
    uint32_t base = 0u;
    if (g.thread_rank() == 0) base = atomicAdd(&sh.n_cand, g.size());
    const uint32_t pos = g.shfl(base, 0) + g.thread_rank();
    if (pos < (uint32_t) cap) {
        buf[pos] = key;
        return true;
    }
    return false;
}

// Keeps the best k keys of the buffer in buf[0 .. k) and records the k-th as the new bar.  All threads; the
// block is synchronised on entry (every append is visible) and on exit.
template <int NT>
__device__ void compact(uint64_t * buf, uint64_t * sel, int k, int cap, SelectShared & sh) {
    const int n = (int) min(sh.n_cand, (uint32_t) cap);
    if (n <= k) return;
    const uint64_t tau = block_kth_key<NT>(buf, n, k, sh.sc);
    const int got = block_take<NT>(buf, n, k, tau, sel, sh.sc);
    for (int i = threadIdx.x; i < got; i += NT) buf[i] = sel[i];
    if (threadIdx.x == 0) {
        sh.n_cand = (uint32_t) got;
        sh.thr_key = tau;
    }
    __syncthreads();
}

// `lists` lists of `len` keys each in buf, every list sorted in the total order with its empty slots (0) at the
// end, merged into sorted[0 .. k): the selection rounds of k_sample (src/kernels.cu:680-695).  With few lists
// every key is ranked directly (its position plus, by binary search, the number of larger keys in each other
// list; no barrier), else by radix selection.  Returns the number of candidates (< k when fewer tokens are
// allowed, src/kernels.cu:698-699); sorted[nk .. k_cap) = 0.  All NT threads; block synchronised on entry and
// exit.
template <int NT>
__device__ int merge_lists(uint64_t * buf, int lists, int len, uint64_t * sel, uint64_t * sorted, SelectScratch & sc,
                           int k, int k_cap) {
    const int tid = threadIdx.x;
    const int total = lists * len;
    int nk;
    if (lists <= 8) {
        for (int j = tid; j < k_cap; j += NT) sorted[j] = 0ull;
        if (tid == 0) sc.count = 0u;
        __syncthreads();
        int mine = 0;
        for (int i = tid; i < total; i += NT) {
            const uint64_t key = buf[i];
            if (key == 0ull) continue;
            ++mine;
            const int l = i / len;
            int rank = i - l * len;
            for (int o = 0; o < lists && rank < k; ++o) {
                if (o == l) continue;
                const uint64_t * other = buf + o * len;
                int lo = 0, hi = len;  // number of keys of `other` that are larger (it is sorted descending)
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (other[mid] > key) lo = mid + 1;
                    else hi = mid;
                }
                rank += lo;
            }
            if (rank < k) sorted[rank] = key;
        }
        if (mine) atomicAdd(&sc.count, (uint32_t) mine);
        __syncthreads();
        nk = (int) min(sc.count, (uint32_t) k);
    } else {
        if (tid == 0) sc.count = 0u;
        __syncthreads();
        // squeeze out the empty slots (the order does not matter to the selection)
        for (int base = 0; base < total; base += NT) {
            const int i = base + tid;
            const uint64_t key = i < total ? buf[i] : 0ull;
            __syncthreads();
            if (key != 0ull) buf[atomicAdd(&sc.count, 1u)] = key;
            __syncthreads();
        }
        const int n = (int) sc.count;
        __syncthreads();
        const uint64_t tau = block_kth_key<NT>(buf, n, k, sc);
        nk = block_take<NT>(buf, n, k, tau, sel, sc);
        for (int j = nk + tid; j < k_cap; j += NT) sorted[j] = 0ull;
        block_rank_sort<NT>(sel, nk, sorted);
        __syncthreads();
    }
    return nk;
}

// The tail of k_sample (src/kernels.cu:698-720) over the nk sorted candidates: candidate softmax, top-p / min-p
// cut, temperature weights, Philox draw.  exp and the quotients are per-element and run in parallel; the three
// running sums keep the reference's left-to-right order: `sum` then `cum` on thread 0, the weight prefix (which
// is both wsum and the acc of the inverse-CDF walk) on thread 32.  qj aliases the selection staging (k_cap
// doubles).  All NT threads; block synchronised on entry.  p.counter is the counter of this row.
template <int NT>
__device__ void draw_tail(const uint64_t * sorted, int nk, double * pj, double * acc, double * qj, SelectScratch & sc,
                          const fns_b200_params & p, int k_cap, int32_t * out_token, fns_b200_cand * out_cands) {
    const int tid = threadIdx.x;
    if (out_cands)
        for (int j = tid; j < k_cap; j += NT) out_cands[j] = key_to_cand(sorted[j]);
    if (!out_token) return;
    if (nk == 0) {
        if (tid == 0) *out_token = -1;
        return;
    }
    if (p.temperature <= 0.0f || nk == 1) {
        if (tid == 0) *out_token = key_id(sorted[0]);
        return;
    }
    const double v0 = (double) key_value(sorted[0]);
    for (int j = tid; j < nk; j += NT) {
        const double d = (double) key_value(sorted[j]) - v0;
        pj[j] = exp(d);
        acc[j] = exp(d / p.temperature);
    }
    __syncthreads();
    volatile double * sum_slot = reinterpret_cast<volatile double *>(&sc.hist[0]);
    if (tid == 0) {
        double sum = 0.0;
        for (int j = 0; j < nk; ++j) sum += pj[j];
        *sum_slot = sum;
    } else if (tid == 32) {
        double run = 0.0;
        for (int j = 0; j < nk; ++j) {
            run += acc[j];
            acc[j] = run;
        }
    }
    __syncthreads();
    {
        const double sum = *sum_slot;
        for (int j = tid; j < nk; j += NT) qj[j] = pj[j] / sum;
    }
    __syncthreads();
    if (tid == 0) {
        int keep = nk;
        double cum = 0.0;
        for (int j = 0; j < nk; ++j) {
            cum += qj[j];
            if (cum >= p.top_p) { keep = j + 1; break; }
        }
        if (p.min_p > 0.0f) {
            int m = 1;
            while (m < keep && pj[m] >= (double) p.min_p) ++m;
            keep = m;
        }
        const double wsum = acc[keep - 1];
        const double u = philox_uniform(p.seed, p.counter) * wsum;
        int pick = keep - 1;
        for (int j = 0; j < keep; ++j)
            if (u < acc[j]) { pick = j; break; }
        *out_token = key_id(sorted[pick]);
    }
}

// Largest float of the allowed, finite elements of one vector (-inf if none).  NaN never wins an fmaxf and
// fails the `<= FLT_MAX` test; +inf is never a candidate (src/kernels.cu:629-639).
template <int VEC>
__device__ __forceinline__ float vector_max(const float (&xv)[VEC], uint32_t bits) {
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < VEC; ++j) m = fmaxf(m, ((bits >> j) & 1u) ? xv[j] : -INFINITY);
    if (m <= FLT_MAX) return m;  // the common case: no +inf among the allowed elements
    m = -INFINITY;
#pragma unroll
    for (int j = 0; j < VEC; ++j)
        if (((bits >> j) & 1u) && xv[j] <= FLT_MAX) m = fmaxf(m, xv[j]);
    return m;
}

template <typename T, int VEC, int NT>
__global__ void __launch_bounds__(NT, 1024 / NT) k_select(const SelectArgs a) {
    constexpr int NV = kEpochElems / VEC;                    // vectors per thread per epoch
    constexpr int FPE = (NV < 4 ? NV : 4) / (NT / 256) > 0 ? (NV < 4 ? NV : 4) / (NT / 256) : 1;  // flags per epoch
    constexpr int VPF = NV / FPE;                            // vectors per flag (a "group")
    constexpr int GPR = 16 / (VPF * VEC) > 0 ? 16 / (VPF * VEC) : 1;  // groups per thread per pass-2 round
    constexpr int kEpoch = NT * kEpochElems;                 // elements per block per epoch
    constexpr int kWarps = NT / 32;
    constexpr uint32_t kVecBits = VEC == 32 ? 0xffffffffu : (1u << VEC) - 1u;
    constexpr int kWordsPerVec = NT * VEC / 32;              // bit-set words between two vectors of one thread
    static_assert(FPE * (NT == 256 ? 16 : 32) <= 64, "flag word too small for the longest slice");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.y, slice = blockIdx.x;
    const int W = a.n_draft + 1, win = row / W, col = row - win * W;
    fns_b200_params p = a.params ? a.params[win] : a.p0;
    const int k = p.temperature <= 0.0f ? 1 : clamp_k(p.top_k, a.k_cap);
    const int lo = slice * a.slice_len;
    const int n_s = max(0, min(a.vocab, lo + a.slice_len) - lo);
    uint64_t * out = a.cand + ((size_t) row * a.slices + slice) * a.k_cap;

    // shared memory: candidate buffer | selection staging | sorted | p, acc (fp64) | slice bit set |
    // history table: offsets, counts | list of the table's occupied slots | their logits | stash: tags, values
    uint64_t * buf = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t * sel = buf + a.cap;
    uint64_t * sorted = sel + a.k_cap;
    double * pj = reinterpret_cast<double *>(sorted + a.k_cap);
    double * acc = pj + a.k_cap;
    uint32_t * eff = reinterpret_cast<uint32_t *>(acc + a.k_cap);
    int * hoff = reinterpret_cast<int *>(eff + a.slice_len / 32);
    uint32_t * hcnt = reinterpret_cast<uint32_t *>(hoff + a.ht_size);
    int * hlist = reinterpret_cast<int *>(hcnt + a.ht_size);
    float * hval = reinterpret_cast<float *>(hlist + a.ht_size / 2);  // raw logits of the listed ids
    uint32_t * stash_tag = reinterpret_cast<uint32_t *>(hval + a.ht_size / 2);
    float * stash_val = reinterpret_cast<float *>(stash_tag + a.stash_cap);  // [stash_cap][max(VEC, 4)]
    SelectShared & sh = *reinterpret_cast<SelectShared *>(stash_val + (size_t) a.stash_cap * (VEC < 4 ? 4 : VEC));

    const T * x = reinterpret_cast<const T *>(a.logits) + (size_t) row * a.row_stride + lo;
    const uint32_t * mrow = a.masks ? a.masks + (size_t) row * a.mask_stride + (lo >> 5) : nullptr;
    const uint32_t id0 = (uint32_t) (a.id_base + lo);

    FNS_PHASE_BEGIN
#ifdef FNS_PHASE_TIMING
    if (k == 12345) atomicExch(a.err, 3);  // consumes the parameters: phase 10 = their arrival
    FNS_PHASE(10)
#endif
    // The first history ids are requested before anything else: their addresses do not depend on the row's
    // history length, which is itself still in flight.
    const bool any_pen = p.repetition != 1.0f || p.presence != 0.0f || p.frequency != 0.0f;
    const bool use_hist = any_pen && a.ht_size > 0 && n_s > 0;
    const int32_t * hrow = a.history ? a.history + (size_t) win * a.history_stride : nullptr;
    const int32_t * drow = a.draft ? a.draft + (size_t) win * a.n_draft : nullptr;
    int32_t ids0[4] = {-1, -1, -1, -1};
    if (use_hist && hrow) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = u * NT + tid;
            if (j < (int) a.history_stride) ids0[u] = hrow[j];
        }
    }
    int n_hist = 0;
    if (a.history && a.history_len) {
        n_hist = a.history_len[win];
        n_hist = n_hist < 0 ? 0 : (n_hist > (int) a.history_stride ? (int) a.history_stride : n_hist);
    }
    const int n_pen = n_hist + (a.draft ? col : 0);

    // 1. The slice's bit set: bit e = element lo + e is allowed.  Bits past the end of the row are 0, so the
    // streaming loop needs no bounds handling.  A warp's 32 words lie in one epoch: the epochs that have any
    // allowed element are collected in sh.epoch_mask, the others are never visited.
    if (tid == 0) {
        sh.n_cand = 0u;
        sh.thr_key = 0ull;
        sh.epoch_mask = 0u;
        sh.n_list = 0u;
        sh.n_stash = 0u;
        sh.n_av = 0u;
        sh.n_vl = 0u;
    }
    if (tid < kWarps) sh.warp_bound[tid] = 0u;
    {
        int4 * h4 = reinterpret_cast<int4 *>(hoff);  // offsets empty, counts (the array behind them) zero
        for (int i = tid; i < a.ht_size / 2; i += NT) {
            const int fill = i < a.ht_size / 4 ? kHashEmpty : 0;
            h4[i] = make_int4(fill, fill, fill, fill);
        }
    }
    __syncthreads();
    const int words = (n_s + 31) >> 5;
    for (int w0 = 0; w0 < a.slice_len / 32; w0 += NT * 4) {  // slice_len / 32 is a multiple of NT / 2
        uint32_t m[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {  // four independent loads in flight
            const int w = w0 + u * NT + tid;
            m[u] = w < words ? (mrow ? mrow[w] : 0xffffffffu) : 0u;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int w = w0 + u * NT + tid;
            if (w >= a.slice_len / 32) continue;  // uniform per warp: NT / 2 divides slice_len / 32
            if (w == words - 1 && (n_s & 31)) m[u] &= (1u << (n_s & 31)) - 1u;
            eff[w] = m[u];
            if (__any_sync(kFull, m[u] != 0u) && lane == 0) atomicOr(&sh.epoch_mask, 1u << (w / (kEpoch / 32)));
        }
    }
    uint64_t best = 0ull;      // k == 1: this thread's best key
    uint32_t lost = 0u;        // elements of the current round that found the buffer full
    float hv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool hv_ok[4] = {false, false, false, false};
    FNS_MARK(0)
#ifdef FNS_PHASE_TIMING
    if (ids0[0] == 0x7ffffff0 || n_hist == 0x7ffffff0) atomicExch(a.err, 3);  // consumes the prefetched ids
    FNS_MARK(11)
#endif

    // 2. Penalties.  The row's history (plus the draft prefix of a verification column) is scattered into a
    // shared hash table: in-slice offset -> occurrence count; the thread that claims a slot also appends it to
    // a list, so the distinct ids can be walked densely afterwards.  Each distinct id then leaves the bit set
    // (whether the mask allowed it is kept in bit 30 of its list entry), so the streaming passes pay nothing for
    // penalties; its penalised value is offered as a candidate after pass 1, when a bound exists that most of
    // them fail.  Traffic: 4 bytes per history id (every slice reads the list; it stays in L2).
    if (use_hist && n_pen > 0) {
        const uint32_t hmask = (uint32_t) a.ht_size - 1u;
        for (int j0 = 0; j0 < n_pen; j0 += NT * 4) {
            int32_t ids[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {  // four independent loads in flight
                const int j = j0 + u * NT + tid;
                if (j0 == 0 && hrow) ids[u] = j < n_hist ? ids0[u] : (j < n_pen ? drow[j - n_hist] : -1);
                else ids[u] = j < n_hist ? hrow[j] : (j < n_pen ? drow[j - n_hist] : -1);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t off = (uint32_t) (ids[u] - a.id_base - lo);
                if (off >= (uint32_t) n_s || ids[u] < a.id_base) continue;
                // double hashing: with linear probing the clusters at load 1/2 make the slowest lane of a warp walk
                // dozens of slots, each a dependent shared-memory access
                uint32_t h = (off * 2654435761u) >> a.ht_shift;
                const uint32_t step = ((off * 0x85EBCA6Bu) >> a.ht_shift) | 1u;
                for (int probe = 0; probe <= a.ht_size; ++probe) {
                    if (probe == a.ht_size) { atomicExch(a.err, 2); break; }  // table full: cannot happen (load <= 1/2)
                    int cur = hoff[h];
                    if (cur == kHashEmpty) cur = atomicCAS(&hoff[h], kHashEmpty, (int) off);  // the old value
                    if (cur == kHashEmpty || (uint32_t) cur == off) {
                        const bool claimed = cur == kHashEmpty;
#ifndef FNS_DBG_NOCNT
                        atomicAdd(&hcnt[h], 1u);
#endif
#ifdef FNS_DBG_NOLIST
                        if (false) {
#else
                        if (claimed) {
#endif
                            const cooperative_groups::coalesced_group cg = cooperative_groups::coalesced_threads();
                            uint32_t base = 0u;
                            if (cg.thread_rank() == 0) base = atomicAdd(&sh.n_list, cg.size());
                            hlist[cg.shfl(base, 0) + cg.thread_rank()] = (int) h;
                        }
                        break;
                    }
                    h = (h + step) & hmask;
                }
            }
        }
        __syncthreads();
        FNS_PHASE(8)
        const int n_list = (int) sh.n_list;
        for (int j = tid; j < n_list; j += NT) {
            const int h = hlist[j];
            const uint32_t off = (uint32_t) hoff[h];
            const uint32_t bit = 1u << (off & 31);
            if (atomicAnd(&eff[off >> 5], ~bit) & bit) hlist[j] = h | (1 << 30);
        }
        FNS_MARK(9)
        // the logits of the first ids of the list are requested now and parked in shared memory once the first
        // epochs of pass 1 are in flight, so that nobody waits for them
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = u * NT + tid;
            hv_ok[u] = j < n_list && (hlist[j] & (1 << 30));
            if (hv_ok[u]) hv[u] = to_float(x[hoff[hlist[j] & ~(1 << 30)]]);
        }
    }
    __syncthreads();
    // The row's ragged end: the elements of a last, partial vector are taken here one by one and removed from
    // the bit set, so that the vector loads below never reach past the row.
    if (VEC > 1 && (n_s % VEC) != 0) {
        if (tid < (n_s % VEC)) {
            const int e = n_s - (n_s % VEC) + tid;
            const uint32_t bit = 1u << (e & 31);
            if (atomicAnd(&eff[e >> 5], ~bit) & bit) {
                const float xi = to_float(x[e]);
                if (is_finite(xi)) {
                    const uint64_t key = make_key(xi, id0 + (uint32_t) e);
                    if (k == 1) {
                        best = key > best ? key : best;
                    } else if (!push(key, buf, sh, a.cap)) {
                        atomicExch(a.err, 1);  // cannot happen: the buffer is empty here
                    }
                }
            }
        }
        __syncthreads();
    }
    FNS_PHASE(1)

    // 3. Pass 1 over the slice: maxima only.  An epoch gives every thread NV vectors (16 elements); two epochs
    // are in flight (the loads of the next one are issued before the current one is reduced); a vector whose
    // elements the bit set excludes is not loaded.  Every thread keeps the maximum of what it has seen, and a
    // 64-bit flag word marks the vector groups whose maximum reaches the running bound.  The bound needs no
    // buffer: if r = ceil(k / warps) lanes of EVERY warp hold a maximum >= v, the slice has at least k elements
    // >= v, so nothing below v can be among its best k.  Each warp finds its r-th largest lane maximum with r
    // warp-wide max reductions and publishes it; the bound is the minimum over the warps (for k = 1: the
    // maximum).  It is refreshed after epochs 1, 2, 4, 8, 16 and once more at the end.
    const uint32_t * effp = eff + ((tid * VEC) >> 5);
    const int bshift = (tid * VEC) & 31;
    const int r_need = (k + kWarps - 1) / kWarps;  // lanes per warp that must hold a value above the bound
    const bool bounded = r_need <= 32;             // otherwise every group is flagged
    float tmax = -INFINITY;                        // this thread's maximum so far
    float thr_v = -FLT_MAX;                        // the bound as a float: x < thr_v cannot be a candidate
    uint32_t thr_word = 0u;
    uint64_t flags = 0ull;
    int done = 0;

    auto refresh = [&]() {  // all threads of the warp
        uint32_t v = tmax > -INFINITY ? order_word(tmax) : 0u, bound = 0u;
        int cnt = 0;
        while (cnt < r_need) {
            const uint32_t m = __reduce_max_sync(kFull, v);
            if (m == 0u) { bound = 0u; break; }
            cnt += __popc(__ballot_sync(kFull, v == m));
            if (v == m) v = 0u;
            bound = m;
        }
        if (lane == 0) *(volatile uint32_t *) &sh.warp_bound[warp] = bound;
    };
    auto read_bound = [&]() {
        const volatile uint32_t * wb = sh.warp_bound;
        uint32_t b = wb[0];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) b = k == 1 ? max(b, wb[w]) : min(b, wb[w]);
        if (b > thr_word) {
            thr_word = b;
            thr_v = word_value(b < 0x00800000u ? 0x00800000u : b);
        }
    };
    auto issue = [&](int ep, float (&xv)[NV][VEC], uint32_t (&mb)[NV]) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            mb[i] = (effp[ep * (kEpoch / 32) + i * kWordsPerVec] >> bshift) & kVecBits;
            if (mb[i]) load_vec<T, VEC>(x + (size_t) ((ep * NT * NV + i * NT + tid) * VEC), xv[i]);
        }
    };
    auto reduce = [&](int ep, float (&xv)[NV][VEC], uint32_t (&mb)[NV]) {
        float vmx[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            vmx[i] = mb[i] ? vector_max<VEC>(xv[i], mb[i]) : -INFINITY;
            tmax = fmaxf(tmax, vmx[i]);
        }
        if (bounded && (done & (done + 1)) == 0) {  // done = 0, 1, 3, 7, 15
            refresh();
            if (done == 0) __syncthreads();  // the first bound needs every warp's share
            read_bound();
        }
        ++done;
#pragma unroll
        for (int g = 0; g < FPE; ++g) {
            uint32_t q = 0u;  // the vectors of this group that reach the bound
#pragma unroll
            for (int u = 0; u < VPF; ++u) q |= (vmx[g * VPF + u] >= thr_v ? 1u : 0u) << u;
            if (!q) continue;
            // Their values go to the stash (pass 2 then needs no memory access).  The group's slots are reserved
            // together: if they do not all fit, none is used (the reserved ones are marked void) and the flag of
            // the group makes pass 2 read it again, so no element can be offered twice.
            const uint32_t want = (uint32_t) __popc(q);
            uint32_t slot = atomicAdd(&sh.n_stash, want);
            const bool fits = slot + want <= (uint32_t) a.stash_cap;
            if (!fits) flags |= 1ull << (ep * FPE + g);
#pragma unroll
            for (int u = 0; u < VPF; ++u) {
                if (!((q >> u) & 1u)) continue;
                const int i = g * VPF + u;
                if (fits) {
                    float4 * dst = reinterpret_cast<float4 *>(stash_val + (size_t) slot * (VEC < 4 ? 4 : VEC));
                    if constexpr (VEC == 1) {
                        dst[0] = make_float4(xv[i][0], 0.0f, 0.0f, 0.0f);
                    } else {
#pragma unroll
                        for (int w4 = 0; w4 < VEC / 4; ++w4)
                            dst[w4] = make_float4(xv[i][4 * w4], xv[i][4 * w4 + 1], xv[i][4 * w4 + 2], xv[i][4 * w4 + 3]);
                    }
                    stash_tag[slot] = (uint32_t) (ep * NV + i) | ((uint32_t) tid << 9) | (mb[i] << 18);
                } else if (slot < (uint32_t) a.stash_cap) {
                    stash_tag[slot] = 0xffffffffu;  // void
                }
                ++slot;
            }
        }
    };
    // How many vectors of the slice have an allowed element?  (One bit per vector: the OR of its mask bits.)
    auto vector_units = [](uint32_t m) -> uint32_t {
        if constexpr (VEC == 1) return m;
        if constexpr (VEC == 4) return (m | (m >> 1) | (m >> 2) | (m >> 3)) & 0x11111111u;
        m |= m >> 4;
        return (m | (m >> 1) | (m >> 2) | (m >> 3)) & 0x01010101u;
    };
    {
        uint32_t cnt = 0u;
        for (int w = tid; w < a.slice_len / 32; w += NT) cnt += (uint32_t) __popc(vector_units(eff[w]));
        cnt = __reduce_add_sync(kFull, cnt);
        if (lane == 0 && cnt) atomicAdd(&sh.n_av, cnt);
    }
    __syncthreads();
    constexpr int LPT = VEC == 8 ? 4 : 8;  // list entries per thread: 32 elements, one `lost` bit each
    const int n_av = (int) sh.n_av;
    const bool sparse = n_av <= min(NT * LPT, a.list_cap);
    if (sparse) {
        // 3a. Few allowed vectors (a grammar mask that admits little): no epochs.  The allowed vectors are listed
        // from the bit set, every thread requests all of its (at most LPT) at once, and after ONE memory round
        // trip the bound is known and the candidates are appended straight from registers.
        uint32_t * vlist = stash_tag;  // the stash is not used on this path
        for (int w = tid; w < a.slice_len / 32; w += NT) {
            uint32_t t = vector_units(eff[w]);
            if (!t) continue;
            uint32_t at = atomicAdd(&sh.n_vl, (uint32_t) __popc(t));
            for (; t; t &= t - 1u) vlist[at++] = (uint32_t) (w * (32 / VEC) + (__ffs(t) - 1) / VEC);
        }
        __syncthreads();
        float xv[LPT][VEC];
        uint32_t mb[LPT];
        int ev[LPT];
#pragma unroll
        for (int u = 0; u < LPT; ++u) {
            const int j = u * NT + tid;
            mb[u] = 0u;
            ev[u] = 0;
            if (j < n_av) {
                ev[u] = (int) vlist[j] * VEC;
                mb[u] = (eff[ev[u] >> 5] >> (ev[u] & 31)) & kVecBits;
                load_vec<T, VEC>(x + ev[u], xv[u]);
            }
        }
        {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (hv_ok[u]) hval[u * NT + tid] = hv[u];
        }
        float vmx[LPT];
#pragma unroll
        for (int u = 0; u < LPT; ++u) {
            vmx[u] = mb[u] ? vector_max<VEC>(xv[u], mb[u]) : -INFINITY;
            tmax = fmaxf(tmax, vmx[u]);
        }
        if (bounded) {
            refresh();
            __syncthreads();
            read_bound();
        }
        done = 1;
        const uint64_t tk0 = (uint64_t) thr_word << 32;
#pragma unroll
        for (int u = 0; u < LPT; ++u) {
            if (!(vmx[u] >= thr_v)) continue;
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                if (((mb[u] >> j) & 1u) && xv[u][j] >= thr_v && xv[u][j] <= FLT_MAX) {
                    const uint64_t key = make_key(xv[u][j], id0 + (uint32_t) (ev[u] + j));
                    if (k == 1) best = key > best ? key : best;
                    else if (key >= tk0 && !push(key, buf, sh, a.cap)) lost |= 1u << (u * VEC + j);
                }
            }
        }
        if (k > 1 && n_av * VEC + VEC > a.trigger) {  // uniform: only then can the buffer fill
            uint64_t tk = tk0;
            while (__syncthreads_or(lost != 0u || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                compact<NT>(buf, sel, k, a.cap, sh);
                if (sh.thr_key > tk) tk = sh.thr_key;
                uint32_t still = 0u;
#pragma unroll
                for (int u = 0; u < LPT; ++u) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        if (!((lost >> (u * VEC + j)) & 1u)) continue;
                        const uint64_t key = make_key(xv[u][j], id0 + (uint32_t) (ev[u] + j));
                        if (key >= tk && !push(key, buf, sh, a.cap)) still |= 1u << (u * VEC + j);
                    }
                }
                lost = still;
                if (!__syncthreads_or(lost != 0u)) break;
            }
        }
        __syncthreads();
    } else
    {
        uint32_t todo = sh.epoch_mask;  // the same for every thread: read after the barrier above
        auto next = [&]() -> int {
            if (!todo) return -1;
            const int ep = __ffs(todo) - 1;
            todo &= todo - 1u;
            return ep;
        };
        float xa[NV][VEC], xb[NV][VEC];
        uint32_t ma[NV], mb[NV];
        int ea = next(), eb = -1;
        if (ea >= 0) issue(ea, xa, ma);
        bool parked = false;
        while (ea >= 0) {
            eb = next();
            if (eb >= 0) issue(eb, xb, mb);
            if (!parked) {
                parked = true;
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (hv_ok[u]) hval[u * NT + tid] = hv[u];
            }
            reduce(ea, xa, ma);
            if (eb < 0) break;
            ea = next();
            if (ea >= 0) issue(ea, xa, ma);
            reduce(eb, xb, mb);
        }
    }
    if (done == 0) {  // no epoch had an allowed element: the parked logits were not stored yet
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (hv_ok[u]) hval[u * NT + tid] = hv[u];
    }
    if (bounded && done > 1) {  // the final bound (after one epoch the first refresh already is)
        refresh();
        __syncthreads();
        read_bound();
    } else {
        __syncthreads();  // the stash is complete
    }
    FNS_PHASE(2)

    // The penalised candidates: every distinct history id that the mask allowed, with its penalised value,
    // against the bound (the bound came from the other elements alone, which can only make it lower than the
    // true k-th best: still a valid bar).  32 list entries per thread between two votes (one `lost` bit each),
    // four at a time so that their logit loads overlap.
    uint64_t thr_key = (uint64_t) thr_word << 32;
    if (use_hist && n_pen > 0) {
        const int n_list = (int) sh.n_list;
        auto entry_key = [&](int h, float v) -> uint64_t {  // v: the raw logit; 0 if the result is not finite
            const float cnt = (float) hcnt[h];
            // each step rounded on its own: no fused multiply-add
            v = v > 0.0f ? __fdiv_rn(v, p.repetition) : __fmul_rn(v, p.repetition);
            v = __fsub_rn(v, __fmul_rn(p.frequency, cnt));
            v = __fsub_rn(v, p.presence);
            return is_finite(v) ? make_key(v, id0 + (uint32_t) hoff[h]) : 0ull;
        };
        for (int j0 = 0; j0 < n_list; j0 += NT * 32) {
            for (int g = 0; g < 8 && j0 + g * 4 * NT < n_list; ++g) {
                int h[4];
                float v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + (g * 4 + u) * NT + tid;
                    const int e = j < n_list ? hlist[j] : 0;
                    h[u] = (e & (1 << 30)) ? (e & ~(1 << 30)) : -1;
                    if (h[u] >= 0) v[u] = j < 4 * NT ? hval[j] : to_float(x[hoff[h[u]]]);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (h[u] < 0) continue;
                    const uint64_t key = entry_key(h[u], v[u]);
                    if (key == 0ull) continue;
                    if (k == 1) best = key > best ? key : best;
                    else if (key >= thr_key && !push(key, buf, sh, a.cap)) lost |= 1u << (g * 4 + u);
                }
            }
            if (k > 1 && n_list + VEC > a.trigger) {  // uniform: only a long list can fill the buffer
                while (__syncthreads_or(lost != 0u || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                    compact<NT>(buf, sel, k, a.cap, sh);
                    const uint64_t tk = sh.thr_key;
                    if (tk > thr_key) { thr_key = tk; thr_v = key_floor_value(tk); }
                    uint32_t still = 0u;
                    for (uint32_t m = lost; m; m &= m - 1u) {
                        const int b = __ffs(m) - 1;
                        const int h = hlist[j0 + b * NT + tid] & ~(1 << 30);
                        const uint64_t key = entry_key(h, to_float(x[hoff[h]]));
                        if (key >= thr_key && !push(key, buf, sh, a.cap)) still |= 1u << b;
                    }
                    lost = still;
                    if (!__syncthreads_or(lost != 0u)) break;
                }
            }
        }
    }

    // Pass 2, first the stash: the vectors that reached the bound when they were streamed, values and all, are
    // compared with the final bound; what passes is appended.  No memory access, no rounds: the entries are
    // spread evenly over the threads.
    {
        constexpr int SE = VEC < 4 ? 4 : VEC;  // floats per stash entry
        const int n_st = (int) min(sh.n_stash, (uint32_t) a.stash_cap);
        // a vote is needed only if the appends could fill the buffer.  The decision must be the same in every
        // thread, so it uses counts that no longer change here (the append cursor itself is moving): what the
        // penalty list and the ragged end can have appended at most, plus every stashed element
        const bool may_fill = (int) sh.n_list + VEC + n_st * VEC > a.trigger;
        for (int i0 = 0; i0 < n_st; i0 += NT) {
            const int i = i0 + tid;
            uint32_t ebase = 0u;
            const uint32_t tag = i < n_st ? stash_tag[i] : 0xffffffffu;
            if (tag != 0xffffffffu) {
                const int vi = (int) (tag & 511u), owner = (int) ((tag >> 9) & 511u);
                const uint32_t bits = tag >> 18;
                const int ep = vi / NV, iv = vi - ep * NV;
                ebase = (uint32_t) ((ep * NT * NV + iv * NT + owner) * VEC);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    const float xi = stash_val[(size_t) i * SE + j];
                    if (((bits >> j) & 1u) && xi >= thr_v && xi <= FLT_MAX) {
                        const uint64_t key = make_key(xi, id0 + ebase + (uint32_t) j);
                        if (k == 1) best = key > best ? key : best;
                        else if (key >= thr_key && !push(key, buf, sh, a.cap)) lost |= 1u << j;
                    }
                }
            }
            if (k > 1 && may_fill) {
                while (__syncthreads_or(lost != 0u || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                    compact<NT>(buf, sel, k, a.cap, sh);
                    const uint64_t tk = sh.thr_key;
                    if (tk > thr_key) { thr_key = tk; thr_v = key_floor_value(tk); }
                    uint32_t still = 0u;
                    for (uint32_t m = lost; m; m &= m - 1u) {
                        const int b = __ffs(m) - 1;
                        const uint64_t key = make_key(stash_val[(size_t) i * SE + b], id0 + ebase + (uint32_t) b);
                        if (key >= thr_key && !push(key, buf, sh, a.cap)) still |= 1u << b;
                    }
                    lost = still;
                    if (!__syncthreads_or(lost != 0u)) break;
                }
            }
        }
    }

    // Pass 2, then the groups that did not fit the stash (none unless the input is adversarial or k is large):
    // they are read again (from L1 / L2: the slice was just streamed) and their
    // elements compared with the final bound, up to GPR groups per thread and round, their loads issued
    // together.  What passes is appended; the block votes once per round on whether to compact (buffer filling
    // up, or an append that found it full, which is then offered again after the compaction).
    if (k == 1) {
        while (flags) {
            const int b = __ffsll((long long) flags) - 1;
            flags &= flags - 1ull;
            const int ep = b / FPE, g = b - ep * FPE;
#pragma unroll
            for (int u = 0; u < VPF; ++u) {
                const int i = g * VPF + u;
                const int e = (ep * NT * NV + i * NT + tid) * VEC;
                const uint32_t bits = (effp[ep * (kEpoch / 32) + i * kWordsPerVec] >> bshift) & kVecBits;
                if (!bits) continue;
                float xv[VEC];
                load_vec<T, VEC>(x + e, xv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    if (((bits >> j) & 1u) && xv[j] >= thr_v && xv[j] <= FLT_MAX) {
                        const uint64_t key = make_key(xv[j], id0 + (uint32_t) (e + j));
                        best = key > best ? key : best;
                    }
                }
            }
        }
    } else {
        while (__syncthreads_or(flags != 0ull)) {
            int eoff[GPR * VPF];      // element offset of each vector of this round (-1: none)
            uint32_t bits[GPR * VPF];
            float xv[GPR * VPF][VEC];
#pragma unroll
            for (int q = 0; q < GPR; ++q) {
                int b = -1;
                if (flags) {
                    b = __ffsll((long long) flags) - 1;
                    flags &= flags - 1ull;
                }
                const int ep = b / FPE, g = b - ep * FPE;
#pragma unroll
                for (int u = 0; u < VPF; ++u) {
                    const int i = g * VPF + u;
                    const int v = q * VPF + u;
                    eoff[v] = -1;
                    bits[v] = 0u;
                    if (b >= 0) {
                        bits[v] = (effp[ep * (kEpoch / 32) + i * kWordsPerVec] >> bshift) & kVecBits;
                        if (bits[v]) {
                            eoff[v] = (ep * NT * NV + i * NT + tid) * VEC;
                            load_vec<T, VEC>(x + eoff[v], xv[v]);
                        }
                    }
                }
            }
#pragma unroll
            for (int v = 0; v < GPR * VPF; ++v) {
                if (eoff[v] < 0) continue;
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    if (((bits[v] >> j) & 1u) && xv[v][j] >= thr_v && xv[v][j] <= FLT_MAX) {
                        const uint64_t key = make_key(xv[v][j], id0 + (uint32_t) (eoff[v] + j));
                        if (key >= thr_key && !push(key, buf, sh, a.cap)) lost |= 1u << (v * VEC + j);
                    }
                }
            }
            while (__syncthreads_or(lost != 0u || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                compact<NT>(buf, sel, k, a.cap, sh);
                const uint64_t tk = sh.thr_key;
                if (tk > thr_key) { thr_key = tk; thr_v = key_floor_value(tk); }
                uint32_t still = 0u;
#pragma unroll
                for (int v = 0; v < GPR * VPF; ++v) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        if (!((lost >> (v * VEC + j)) & 1u)) continue;
                        const int e = eoff[v] + j;
                        const uint64_t key = make_key(to_float(x[e]), id0 + (uint32_t) e);
                        if (key >= thr_key && !push(key, buf, sh, a.cap)) still |= 1u << (v * VEC + j);
                    }
                }
                lost = still;
                if (!__syncthreads_or(lost != 0u)) break;
            }
        }
    }
    __syncthreads();
    FNS_PHASE(3)

    // 4. The slice's answer: its best k keys in the total order.  A row that is one slice goes straight on to
    // the draw; otherwise the list goes to global memory and the last block of the row merges.
    const bool whole_row = a.slices == 1;
    p.counter += (uint64_t) col;  // column c of a window draws with counter + c (src/engine.cu:756)
    int32_t * tok = a.out_tokens ? a.out_tokens + row : nullptr;
    fns_b200_cand * oc = a.out_cands ? a.out_cands + (size_t) row * a.k_cap : nullptr;
    if (k == 1) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const uint64_t other = __shfl_xor_sync(kFull, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) sh.red[warp] = best;
        __syncthreads();
        if (tid == 0) {
            uint64_t b = sh.red[0];
            for (int w = 1; w < kWarps; ++w) b = sh.red[w] > b ? sh.red[w] : b;
            if (whole_row) {
                if (tok) *tok = b ? key_id(b) : -1;
                if (oc) oc[0] = key_to_cand(b);
            } else {
                out[0] = b;
            }
        }
        if (whole_row) {
            if (oc)
                for (int j = 1 + tid; j < a.k_cap; j += NT) oc[j] = key_to_cand(0ull);
            return;
        }
    } else {
        const int n = (int) min(sh.n_cand, (uint32_t) a.cap);
        uint64_t * dst = whole_row ? sorted : out;
        int got;
        if (n <= kRankSelectMax) {
            got = block_rank_select<NT>(buf, n, k, dst);
        } else {
            const uint64_t tau = block_kth_key<NT>(buf, n, k, sh.sc);
            got = block_take<NT>(buf, n, k, tau, sel, sh.sc);
            block_rank_sort<NT>(sel, got, dst);
        }
        for (int j = got + tid; j < (whole_row ? a.k_cap : k); j += NT) dst[j] = 0ull;
        if (whole_row) {
            __syncthreads();
            FNS_PHASE(4)
            draw_tail<NT>(sorted, got, pj, acc, reinterpret_cast<double *>(sel), sh.sc, p, a.k_cap, tok, oc);
            FNS_PHASE(5)
            return;
        }
    }
    FNS_PHASE(4)

    // 5. The last block of the row to get here merges the slices' lists and draws.  Nobody waits: every block
    // takes a ticket after its list is visible, and the one that draws the last ticket does the work.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned t = atomicAdd(&a.tickets[row], 1u);
        sh.is_last = t == (unsigned) a.slices - 1u;
        if (sh.is_last) a.tickets[row] = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (!sh.is_last) return;
    __threadfence();
    const uint64_t * lists = a.cand + (size_t) row * a.slices * a.k_cap;
    if (k == 1) {  // greedy: the largest of the slices' best keys, no sort, no draw
        uint64_t b = 0ull;
        for (int l = tid; l < a.slices; l += NT) {
            const uint64_t key = __ldcg(lists + (size_t) l * a.k_cap);
            b = key > b ? key : b;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const uint64_t other = __shfl_xor_sync(kFull, b, o);
            b = other > b ? other : b;
        }
        if (lane == 0) sh.red[warp] = b;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < kWarps; ++w) b = sh.red[w] > b ? sh.red[w] : b;
            if (tok) *tok = b ? key_id(b) : -1;
            if (oc) oc[0] = key_to_cand(b);
        }
        if (oc)
            for (int j = 1 + tid; j < a.k_cap; j += NT) oc[j] = key_to_cand(0ull);
        FNS_PHASE(5)
        return;
    }
    // the slices' lists, each sorted, side by side in the buffer: [slices][k]
    for (int i = tid; i < a.slices * k; i += NT) {
        const int l = i / k, j = i - l * k;
        buf[i] = __ldcg(lists + (size_t) l * a.k_cap + j);
    }
    __syncthreads();
    const int nk = merge_lists<NT>(buf, a.slices, k, sel, sorted, sh.sc, k, a.k_cap);
    draw_tail<NT>(sorted, nk, pj, acc, reinterpret_cast<double *>(sel), sh.sc, p, a.k_cap, tok, oc);
    FNS_PHASE(5)
}

// ---- finalize as a kernel of its own -------------------------------------------------------------------------
constexpr int kFinalThreads = 256;

struct FinalArgs {
    const fns_b200_cand * cands;  // entry j of list l of row r at r * row_stride + l * list_stride + j
    int lists;
    int list_len;
    int64_t list_stride;
    int64_t row_stride;
    int k_cap;
    const fns_b200_params * params;
    int32_t * out_tokens;      // may be null (merge only)
    fns_b200_cand * out_cands; // may be null; [rows][k_cap]
};

struct FinalShared {
    SelectScratch sc;
};

__global__ void __launch_bounds__(kFinalThreads) k_finalize(const FinalArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x;
    const int row = blockIdx.x;
    const fns_b200_params p = a.params[row];
    const int k = p.temperature <= 0.0f ? 1 : clamp_k(p.top_k, a.k_cap);

    // shared memory: all keys of the row | selection staging | sorted result | p / acc (fp64)
    uint64_t * buf = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t * sel = buf + a.lists * a.list_len;
    uint64_t * sorted = sel + a.k_cap;
    double * pj = reinterpret_cast<double *>(sorted + a.k_cap);
    double * acc = pj + a.k_cap;
    FinalShared & sh = *reinterpret_cast<FinalShared *>(acc + a.k_cap);

    // the row's lists side by side: [lists][list_len]
    const size_t row_base = (size_t) row * a.row_stride;
    for (int i = tid; i < a.lists * a.list_len; i += kFinalThreads) {
        const int l = i / a.list_len, j = i - l * a.list_len;
        buf[i] = cand_to_key(a.cands[row_base + (size_t) l * a.list_stride + j]);
    }
    __syncthreads();
    const int nk = merge_lists<kFinalThreads>(buf, a.lists, a.list_len, sel, sorted, sh.sc, k, a.k_cap);
    draw_tail<kFinalThreads>(sorted, nk, pj, acc, reinterpret_cast<double *>(sel), sh.sc, p, a.k_cap,
                             a.out_tokens ? a.out_tokens + row : nullptr,
                             a.out_cands ? a.out_cands + (size_t) row * a.k_cap : nullptr);
}

// a = number of leading columns whose token equals the draft (tools/fns_serve/fns_serve.cpp:492-508).
__global__ void k_accept(const int32_t * tokens, const int32_t * draft, int n_draft, int windows, int32_t * accept) {
    const int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= windows) return;
    const int32_t * t = tokens + (size_t) w * (n_draft + 1);
    const int32_t * d = draft + (size_t) w * n_draft;
    int a = 0;
    while (a < n_draft && t[a] == d[a]) ++a;
    accept[w] = a;
}

// ---- the reference's dense presence state (src/kernels.cu:724-752) ----------------------------------------
__global__ void k_presence_apply(float * x, const float * seen, int n, float penalty) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __fsub_rn(x[i], __fmul_rn(penalty, seen[i]));
}
__global__ void k_presence_apply_col(float * x, const float * seen, const int32_t * draft, int c, int n, float penalty) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = seen[i];
    for (int j = 0; j < c; ++j)
        if (draft[j] == i) s = 1.0f;
    x[i] = __fsub_rn(x[i], __fmul_rn(penalty, s));
}
__global__ void k_presence_mark_n(float * seen, const int32_t * tokens, int n) {
    const int j = threadIdx.x;
    if (j < n && tokens[j] >= 0) seen[tokens[j]] = 1.0f;
}
__global__ void k_io_advance(int32_t * io, int pos) {
    io[0] = io[2] < 0 ? 0 : io[2];
    io[1] = pos;
}

}  // namespace fnsb

// ================================================ host side ================================================
using namespace fnsb;

struct fns_b200_sampler {
    int device;
    int max_rows, max_vocab, k_cap, max_history;
    int sm_count;
    int force_slices;
    int force_threads;
    uint64_t * cand;   // [rows][slices][k_cap] sorted keys of the slices
    size_t cand_entries;
    unsigned * tickets;  // [max_rows], zero between launches
    int * err;
    int64_t launches;
    bool prof_on;
    int prof_calls;                   // calls recorded so far
    std::vector<cudaEvent_t> prof_ev; // three per call: before select, after select, after finalize
    char msg[256];
};

namespace {

struct Plan {
    int threads, slices, slice_len, cap, trigger, ht_size, vec, stash_cap;
    size_t smem_select;
};

int round_up(int x, int m) { return (x + m - 1) / m * m; }
int next_pow2(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

int fail(fns_b200_sampler * s, int code, const char * what) {
    if (s) std::snprintf(s->msg, sizeof s->msg, "%s", what);
    return code;
}
int fail_cuda(fns_b200_sampler * s, cudaError_t e, const char * where) {
    if (s) std::snprintf(s->msg, sizeof s->msg, "%s: %s", where, cudaGetErrorString(e));
    return FNS_B200_ERR_CUDA;
}

// Launch geometry.  With at least one row per SM a row is one slice and a block has 512 threads: two blocks fit
// an SM, so up to 2 * SMs rows stream at once, and setup, history and draw are paid once per row.  With fewer
// rows a row is cut into slices of 256-thread blocks, about four per SM in total, so that the whole GPU works on
// the call.  A slice is a whole number of epochs (16 elements per thread) and at most 16 (256 threads) or 32
// (512 threads) of them; the slices' lists of one row must fit the merge (kMaxMergeKeys).
bool make_plan(const fns_b200_sampler * s, int dtype, int vocab, int rows, int hist_bound, bool aligned, Plan & pl) {
    const int k_cap = s->k_cap;
    pl.threads = s->force_threads > 0 ? s->force_threads : (s->force_slices > 0 ? 256 : (rows >= s->sm_count ? 512 : 256));
    const int epoch = pl.threads * kEpochElems;
    const int max_slice_len = (pl.threads == 256 ? 16 : 32) * epoch;
    const int min_slices = (vocab + max_slice_len - 1) / max_slice_len;
    int max_slices = kMaxMergeKeys / k_cap;
    if (max_slices > kMaxSlices) max_slices = kMaxSlices;
    if (min_slices > max_slices) return false;
    int want;
    if (s->force_slices > 0) want = s->force_slices;
    else if (pl.threads == 512) want = 1;
    else want = (s->sm_count * 4 + rows - 1) / rows;
    const int by_len = (vocab + epoch - 1) / epoch;  // no slice shorter than one epoch
    if (want > by_len) want = by_len;
    if (s->force_slices <= 0 && want > 64) want = 64;
    if (want < min_slices) want = min_slices;
    if (want > max_slices) want = max_slices;
    if (want < 1) want = 1;
    pl.slice_len = round_up((vocab + want - 1) / want, epoch);
    if (pl.slice_len > max_slice_len) pl.slice_len = max_slice_len;
    pl.slices = (vocab + pl.slice_len - 1) / pl.slice_len;
    pl.vec = aligned ? (dtype == FNS_B200_BF16 ? 8 : 4) : 1;
    const int base_cap = 4 * k_cap > 2048 ? 4 * k_cap : 2048;
    pl.trigger = base_cap / 2;
    pl.cap = base_cap;
    if (pl.slices * k_cap > pl.cap) pl.cap = pl.slices * k_cap;  // room to merge the row's lists
    pl.ht_size = 0;
    if (hist_bound > 0) {
        const int distinct = hist_bound < pl.slice_len ? hist_bound : pl.slice_len;
        pl.ht_size = next_pow2(2 * distinct);
        if (pl.ht_size < 1024) pl.ht_size = 1024;
    }
    // stash: 16 KB of flagged vectors (tag + max(vec, 4) floats each)
    const int entry_floats = pl.vec < 4 ? 4 : pl.vec;
    pl.stash_cap = 16384 / (4 * entry_floats + 4) / 4 * 4;  // a multiple of 4: what follows stays 16-byte aligned
    pl.smem_select = (size_t) pl.cap * 8 + (size_t) k_cap * 8 * 4 + (size_t) pl.slice_len / 8 + (size_t) pl.ht_size * 12 +
                     (size_t) pl.stash_cap * (4 * entry_floats + 4) + sizeof(SelectShared) + 16;
    return pl.smem_select <= 200 * 1024;
}

size_t final_smem(int lists, int list_len, int k_cap) {
    return (size_t) lists * list_len * 8 + (size_t) k_cap * 8 * 4 + sizeof(FinalShared) + 16;
}

template <typename T, int VEC, int NT>
cudaError_t launch_select_t(const SelectArgs & a, int rows, size_t smem, cudaStream_t st) {
    auto kern = k_select<T, VEC, NT>;
    static bool configured[64] = {};  // per device: the opt-in to large dynamic shared memory is sticky
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    kern<<<dim3((unsigned) a.slices, (unsigned) rows), NT, smem, st>>>(a);
    return cudaGetLastError();
}

template <int NT>
cudaError_t launch_select_nt(const SelectArgs & a, int dtype, int vec, int rows, size_t smem, cudaStream_t st) {
    if (dtype == FNS_B200_BF16)
        return vec == 8 ? launch_select_t<__nv_bfloat16, 8, NT>(a, rows, smem, st)
                        : launch_select_t<__nv_bfloat16, 1, NT>(a, rows, smem, st);
    return vec == 4 ? launch_select_t<float, 4, NT>(a, rows, smem, st) : launch_select_t<float, 1, NT>(a, rows, smem, st);
}

cudaError_t launch_select(const SelectArgs & a, int threads, int dtype, int vec, int rows, size_t smem, cudaStream_t st) {
    return threads == 512 ? launch_select_nt<512>(a, dtype, vec, rows, smem, st)
                          : launch_select_nt<256>(a, dtype, vec, rows, smem, st);
}

cudaError_t launch_final(const FinalArgs & a, int rows, cudaStream_t st) {
    const size_t smem = final_smem(a.lists, a.list_len, a.k_cap);
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(k_finalize, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    k_finalize<<<(unsigned) rows, kFinalThreads, smem, st>>>(a);
    return cudaGetLastError();
}

struct DeviceGuard {
    int prev = -1;
    bool ok;
    explicit DeviceGuard(int dev) {
        ok = cudaGetDevice(&prev) == cudaSuccess && (prev == dev || cudaSetDevice(dev) == cudaSuccess);
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

// Shared front end of sample_rows / select_rows / verify_accept: argument checks, plan, the select launch.
int run_select(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
               int32_t id_base, const uint32_t * masks, int64_t mask_stride, const int32_t * history,
               int64_t history_stride, const int32_t * history_len, const int32_t * draft, int n_draft,
               const fns_b200_params * params, const fns_b200_params * p0, int32_t * out_tokens,
               fns_b200_cand * out_cands, cudaStream_t st, Plan & pl) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!logits || rows <= 0 || vocab <= 0) return fail(s, FNS_B200_ERR_ARG, "logits null, or rows / vocab <= 0");
    if (dtype != FNS_B200_F32 && dtype != FNS_B200_BF16) return fail(s, FNS_B200_ERR_ARG, "dtype must be F32 or BF16");
    if (!params && !p0) return fail(s, FNS_B200_ERR_ARG, "params null");
    if (rows > s->max_rows || vocab > s->max_vocab) return fail(s, FNS_B200_ERR_CAPACITY, "rows or vocab beyond the handle's limits");
    // a stride of 0 repeats one row (or one mask) for every row of the call
    if (row_stride != 0 && row_stride < vocab && rows > 1) return fail(s, FNS_B200_ERR_ARG, "row_stride < vocab");
    if (masks && mask_stride != 0 && mask_stride < (vocab + 31) / 32 && rows > 1) return fail(s, FNS_B200_ERR_ARG, "mask_stride_words < ceil(vocab / 32)");
    if (id_base < 0 || (id_base & 31)) return fail(s, FNS_B200_ERR_ARG, "id_base must be a non-negative multiple of 32");
    if ((history != nullptr) != (history_len != nullptr)) return fail(s, FNS_B200_ERR_ARG, "history and history_len go together");
    if (history && (history_stride <= 0 || history_stride > s->max_history)) return fail(s, FNS_B200_ERR_CAPACITY, "history_stride outside (0, max_history]");
    if (n_draft < 0 || n_draft >= FNS_B200_MAX_WINDOW) return fail(s, FNS_B200_ERR_ARG, "n_draft outside [0, FNS_B200_MAX_WINDOW)");
    if (n_draft > 0 && !draft) return fail(s, FNS_B200_ERR_ARG, "draft null");
    const size_t esz = dtype == FNS_B200_BF16 ? 2 : 4;
    const bool aligned = ((uintptr_t) logits % 16 == 0) && ((size_t) row_stride * esz % 16 == 0 || rows == 1);
    const int hist_bound = (history ? (int) history_stride : 0) + n_draft;
    if (!make_plan(s, dtype, vocab, rows, hist_bound, aligned, pl)) return fail(s, FNS_B200_ERR_CAPACITY, "no launch plan fits (vocab too large for k_cap)");
    if ((size_t) rows * pl.slices * s->k_cap > s->cand_entries) return fail(s, FNS_B200_ERR_CAPACITY, "workspace too small for this call");
    SelectArgs a{};
    a.logits = logits;
    a.row_stride = row_stride;
    a.vocab = vocab;
    a.id_base = id_base;
    a.masks = masks;
    a.mask_stride = mask_stride;
    a.history = history;
    a.history_stride = history_stride;
    a.history_len = history_len;
    a.draft = n_draft > 0 ? draft : nullptr;
    a.n_draft = n_draft;
    a.params = params;
    if (p0) a.p0 = *p0;
    a.k_cap = s->k_cap;
    a.slices = pl.slices;
    a.slice_len = pl.slice_len;
    a.cap = pl.cap;
    a.trigger = pl.trigger;
    a.ht_size = pl.ht_size;
    a.ht_shift = 32;
    for (int t = pl.ht_size; t > 1; t >>= 1) --a.ht_shift;
    a.stash_cap = pl.stash_cap;
    a.list_cap = pl.stash_cap * ((pl.vec < 4 ? 4 : pl.vec) + 1);  // 32-bit words in the stash's memory
    a.cand = s->cand;
    a.tickets = s->tickets;
    a.out_tokens = out_tokens;
    a.out_cands = out_cands;
    a.err = s->err;
    const bool prof = s->prof_on && (size_t) (s->prof_calls + 1) * 3 <= s->prof_ev.size();
    if (prof) cudaEventRecord(s->prof_ev[(size_t) s->prof_calls * 3], st);
    const cudaError_t e = launch_select(a, pl.threads, dtype, pl.vec, rows, pl.smem_select, st);
    if (e != cudaSuccess) return fail_cuda(s, e, "select launch");
    ++s->launches;
    if (prof) {  // the merge and the draw happen inside k_select: the record closes here
        cudaEventRecord(s->prof_ev[(size_t) s->prof_calls * 3 + 1], st);
        cudaEventRecord(s->prof_ev[(size_t) s->prof_calls * 3 + 2], st);
        ++s->prof_calls;
    }
    return FNS_B200_OK;
}

}  // namespace

extern "C" {

int fns_b200_create(int device, int max_rows, int max_vocab, int k_cap, int max_history, fns_b200_sampler ** out) {
    if (!out) return FNS_B200_ERR_ARG;
    *out = nullptr;
    if (max_rows <= 0 || max_vocab <= 0 || k_cap < 1 || k_cap > FNS_B200_MAX_K || max_history < 0 ||
        max_history > FNS_B200_MAX_HISTORY)
        return FNS_B200_ERR_ARG;
    DeviceGuard g(device);
    if (!g.ok) return FNS_B200_ERR_CUDA;
    fns_b200_sampler * s = new (std::nothrow) fns_b200_sampler();
    if (!s) return FNS_B200_ERR_ARG;
    s->device = device;
    s->max_rows = max_rows;
    s->max_vocab = max_vocab;
    s->k_cap = k_cap;
    s->max_history = max_history;
    s->force_slices = 0;
    s->force_threads = 0;
    s->launches = 0;
    s->prof_on = false;
    s->prof_calls = 0;
    s->msg[0] = 0;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        delete s;
        return FNS_B200_ERR_CUDA;
    }
    s->sm_count = prop.multiProcessorCount;
    // Candidate workspace: the largest rows * slices any plan can produce, bounded by the merge limit.
    int max_slices = kMaxMergeKeys / k_cap;
    if (max_slices > kMaxSlices) max_slices = kMaxSlices;
    size_t per_row = (size_t) max_slices * k_cap;
    // many rows never use many slices: slices <= max(ceil(4 * SMs / rows), vocab / 65536) unless forced
    s->cand_entries = (size_t) max_rows * per_row;
    const size_t cap_entries = (size_t) 1 << 27;  // 1 GiB of keys at most
    if (s->cand_entries > cap_entries) s->cand_entries = cap_entries;
    if (cudaMalloc(&s->cand, s->cand_entries * sizeof(uint64_t)) != cudaSuccess ||
        cudaMalloc(&s->err, sizeof(int)) != cudaSuccess || cudaMemset(s->err, 0, sizeof(int)) != cudaSuccess ||
        cudaMalloc(&s->tickets, (size_t) max_rows * sizeof(unsigned)) != cudaSuccess ||
        cudaMemset(s->tickets, 0, (size_t) max_rows * sizeof(unsigned)) != cudaSuccess) {
        if (s->cand) cudaFree(s->cand);
        if (s->err) cudaFree(s->err);
        if (s->tickets) cudaFree(s->tickets);
        delete s;
        return FNS_B200_ERR_CUDA;
    }
    *out = s;
    return FNS_B200_OK;
}

int fns_b200_destroy(fns_b200_sampler * s) {
    if (!s) return FNS_B200_OK;
    DeviceGuard g(s->device);
    cudaFree(s->cand);
    cudaFree(s->err);
    cudaFree(s->tickets);
    for (cudaEvent_t ev : s->prof_ev) cudaEventDestroy(ev);
    delete s;
    return FNS_B200_OK;
}

int64_t fns_b200_launch_count(const fns_b200_sampler * s) { return s ? s->launches : 0; }

int fns_b200_profile_begin(fns_b200_sampler * s, int max_calls) {
    if (!s || max_calls <= 0 || max_calls > 100000) return FNS_B200_ERR_ARG;
    DeviceGuard g(s->device);
    while (s->prof_ev.size() < (size_t) max_calls * 3) {
        cudaEvent_t ev;
        if (cudaEventCreate(&ev) != cudaSuccess) return fail(s, FNS_B200_ERR_CUDA, "cudaEventCreate");
        s->prof_ev.push_back(ev);
    }
    s->prof_calls = 0;
    s->prof_on = true;
    return FNS_B200_OK;
}

int fns_b200_profile_end(fns_b200_sampler * s, void * stream, double * select_ms, double * finalize_ms, int * calls) {
    if (!s) return FNS_B200_ERR_ARG;
    s->prof_on = false;
    const cudaError_t e = cudaStreamSynchronize((cudaStream_t) stream);
    if (e != cudaSuccess) return fail_cuda(s, e, "profile_end");
    double a = 0.0, b = 0.0;
    for (int i = 0; i < s->prof_calls; ++i) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, s->prof_ev[(size_t) i * 3], s->prof_ev[(size_t) i * 3 + 1]) == cudaSuccess) a += ms;
        if (cudaEventElapsedTime(&ms, s->prof_ev[(size_t) i * 3 + 1], s->prof_ev[(size_t) i * 3 + 2]) == cudaSuccess) b += ms;
    }
    if (select_ms) *select_ms = a;
    if (finalize_ms) *finalize_ms = b;
    if (calls) *calls = s->prof_calls;
    return FNS_B200_OK;
}

const char * fns_b200_last_error(const fns_b200_sampler * s) { return s ? s->msg : "null handle"; }
int fns_b200_k_cap(const fns_b200_sampler * s) { return s ? s->k_cap : 0; }

int fns_b200_device_status(fns_b200_sampler * s, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    int flag = 0;
    cudaError_t e = cudaMemcpyAsync(&flag, s->err, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t) stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t) stream);
    if (e != cudaSuccess) return fail_cuda(s, e, "device_status");
    if (flag != 0) {
        cudaMemsetAsync(s->err, 0, sizeof(int), (cudaStream_t) stream);
        return fail(s, FNS_B200_ERR_DEVICE, flag == 1 ? "candidate buffer overflow" : "history table overflow");
    }
    return FNS_B200_OK;
}

int fns_b200_set_slices(fns_b200_sampler * s, int slices) {
    if (!s || slices < 0 || slices > kMaxSlices) return FNS_B200_ERR_ARG;
    s->force_slices = slices;
    return FNS_B200_OK;
}

int fns_b200_set_threads(fns_b200_sampler * s, int threads) {
    if (!s || (threads != 0 && threads != 256 && threads != 512)) return FNS_B200_ERR_ARG;
    s->force_threads = threads;
    return FNS_B200_OK;
}

int fns_b200_plan(const fns_b200_sampler * s, int dtype, int vocab, int rows, int history_bound, int * slices,
                  int * slice_len, int * smem_bytes) {
    if (!s || vocab <= 0 || rows <= 0) return FNS_B200_ERR_ARG;
    Plan pl;
    if (!make_plan(s, dtype, vocab, rows, history_bound, true, pl)) return FNS_B200_ERR_CAPACITY;
    if (slices) *slices = pl.slices;
    if (slice_len) *slice_len = pl.slice_len;
    if (smem_bytes) *smem_bytes = (int) pl.smem_select;
    return FNS_B200_OK;
}

int fns_b200_sample_rows(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
                         const uint32_t * masks, int64_t mask_stride_words, const int32_t * history,
                         int64_t history_stride, const int32_t * history_len, const fns_b200_params * params,
                         int32_t * out_tokens, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_tokens || !params) return fail(s, FNS_B200_ERR_ARG, "out_tokens or params null");
    DeviceGuard g(s->device);
    Plan pl;
    int rc = run_select(s, logits, dtype, row_stride, vocab, rows, 0, masks, mask_stride_words, history, history_stride,
                        history_len, nullptr, 0, params, nullptr, out_tokens, nullptr, (cudaStream_t) stream, pl);
    return rc;
}

int fns_b200_sample_one(fns_b200_sampler * s, const void * logits, int dtype, int vocab, const uint32_t * mask,
                        const int32_t * history, int history_len, const fns_b200_params * params_host,
                        int32_t * out_token, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_token || !params_host) return fail(s, FNS_B200_ERR_ARG, "out_token or params_host null");
    if (history && history_len > 0) return fail(s, FNS_B200_ERR_ARG, "sample_one takes no history: use sample_rows");
    DeviceGuard g(s->device);
    Plan pl;
    int rc = run_select(s, logits, dtype, vocab, vocab, 1, 0, mask, (vocab + 31) / 32, nullptr, 0, nullptr, nullptr, 0,
                        nullptr, params_host, out_token, nullptr, (cudaStream_t) stream, pl);
    return rc;
}

int fns_b200_select_rows(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
                         int32_t id_base, const uint32_t * masks, int64_t mask_stride_words,
                         const int32_t * history, int64_t history_stride, const int32_t * history_len,
                         const fns_b200_params * params, fns_b200_cand * out_cands, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_cands || !params) return fail(s, FNS_B200_ERR_ARG, "out_cands or params null");
    DeviceGuard g(s->device);
    Plan pl;
    int rc = run_select(s, logits, dtype, row_stride, vocab, rows, id_base, masks, mask_stride_words, history,
                        history_stride, history_len, nullptr, 0, params, nullptr, nullptr, out_cands,
                        (cudaStream_t) stream, pl);
    return rc;
}

int fns_b200_finalize_rows(fns_b200_sampler * s, const fns_b200_cand * cands, int lists, int list_len,
                           int64_t list_stride, int64_t row_stride, int rows, const fns_b200_params * params,
                           int32_t * out_tokens, fns_b200_cand * out_cands, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!cands || !params || (!out_tokens && !out_cands)) return fail(s, FNS_B200_ERR_ARG, "cands / params null, or no output");
    if (lists <= 0 || list_len <= 0 || rows <= 0 || (int64_t) lists * list_len > kMaxMergeKeys)
        return fail(s, FNS_B200_ERR_ARG, "lists * list_len outside (0, 8192]");
    if (list_stride < 0 || row_stride < 0) return fail(s, FNS_B200_ERR_ARG, "negative stride");
    DeviceGuard g(s->device);
    FinalArgs f{};
    f.cands = cands;
    f.lists = lists;
    f.list_len = list_len;
    f.list_stride = list_stride;
    f.row_stride = row_stride;
    f.k_cap = s->k_cap;
    f.params = params;
    f.out_tokens = out_tokens;
    f.out_cands = out_cands;
    const cudaError_t e = launch_final(f, rows, (cudaStream_t) stream);
    if (e != cudaSuccess) return fail_cuda(s, e, "finalize launch");
    return FNS_B200_OK;
}

int fns_b200_verify_accept(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab,
                           int windows, int n_draft, const int32_t * draft, const uint32_t * masks,
                           int64_t mask_stride_words, const int32_t * history, int64_t history_stride,
                           const int32_t * history_len, const fns_b200_params * params, int32_t * out_tokens,
                           int32_t * out_accept, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_tokens || !out_accept || !params) return fail(s, FNS_B200_ERR_ARG, "out_tokens / out_accept / params null");
    if (windows <= 0) return fail(s, FNS_B200_ERR_ARG, "windows <= 0");
    DeviceGuard g(s->device);
    const int rows = windows * (n_draft + 1);
    Plan pl;
    int rc = run_select(s, logits, dtype, row_stride, vocab, rows, 0, masks, mask_stride_words, history, history_stride,
                        history_len, draft, n_draft, params, nullptr, out_tokens, nullptr, (cudaStream_t) stream, pl);
    if (rc != FNS_B200_OK) return rc;
    k_accept<<<(unsigned) ((windows + 127) / 128), 128, 0, (cudaStream_t) stream>>>(out_tokens, draft, n_draft, windows,
                                                                                  out_accept);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(s, e, "accept launch");
    ++s->launches;
    return FNS_B200_OK;
}

#ifdef FNS_PHASE_TIMING
// development aid (not part of the ABI header): reads and clears the phase clocks
int fns_b200_debug_phases(unsigned long long * out8) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out8, fnsb::g_phase, sizeof(unsigned long long) * 16);
    unsigned long long zero[16] = {};
    cudaMemcpyToSymbol(fnsb::g_phase, zero, sizeof zero);
    return 0;
}
#endif

int fns_b200_presence_apply(float * x, const float * seen, int n, float penalty, void * stream) {
    if (!x || !seen || n <= 0) return FNS_B200_ERR_ARG;
    k_presence_apply<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(x, seen, n, penalty);
    return cudaGetLastError() == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA;
}

// Single token: the reference's k_presence_mark (src/kernels.cu:729-731) is the n = 1 case of k_presence_mark_n.
int fns_b200_presence_mark(float * seen, const int32_t * token, void * stream) {
    if (!seen || !token) return FNS_B200_ERR_ARG;
    k_presence_mark_n<<<1, 32, 0, (cudaStream_t) stream>>>(seen, token, 1);
    return cudaGetLastError() == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA;
}

int fns_b200_presence_apply_col(float * x, const float * seen, const int32_t * draft, int c, int n, float penalty,
                                void * stream) {
    if (!x || !seen || n <= 0 || c < 0 || (c > 0 && !draft)) return FNS_B200_ERR_ARG;
    k_presence_apply_col<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(x, seen, draft, c, n, penalty);
    return cudaGetLastError() == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA;
}

int fns_b200_presence_mark_n(float * seen, const int32_t * tokens, int n, void * stream) {
    if (!seen || !tokens || n < 0 || n > 32) return FNS_B200_ERR_ARG;
    k_presence_mark_n<<<1, 32, 0, (cudaStream_t) stream>>>(seen, tokens, n);
    return cudaGetLastError() == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA;
}

int fns_b200_io_advance(int32_t * io, int pos, void * stream) {
    if (!io) return FNS_B200_ERR_ARG;
    k_io_advance<<<1, 1, 0, (cudaStream_t) stream>>>(io, pos);
    return cudaGetLastError() == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA;
}

}  // extern "C"

// ---- sampling without any allocation ----------------------------------------------------------------------
// For hosts that may not allocate GPU memory when they sample: engines that hand the whole device to their own
// arena at start-up and leave nothing for cudaMalloc, and call sites where an allocation, which synchronises
// the device, is not allowed.  The candidate lists, the per-row tickets and the error flag that a handle would
// own live in one file-scope device array instead.  Every GPU that loads the library carries this array until
// the process exits.
namespace {

constexpr int kNoAllocRows = 64;                       // rows per call
constexpr int kNoAllocK = 64;                          // k_cap, the reference's kSampleMaxK
constexpr size_t kNoAllocCand = (size_t) kNoAllocRows * 64 * kNoAllocK;  // keys: 64 rows x 64 slices x 64 = 2 MiB
constexpr size_t kNoAllocBytes = kNoAllocCand * sizeof(uint64_t) + kNoAllocRows * sizeof(unsigned) + 256;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

std::mutex g_noalloc_lock;
unsigned char * g_noalloc_ptr[64];  // per device: the array's DEVICE address (its name in host code is not one)

}  // namespace

extern "C" int fns_b200_sample_rows_noalloc(int device, const void * logits, int dtype, int64_t row_stride, int vocab,
                                            int rows, const uint32_t * masks, int64_t mask_stride_words,
                                            const int32_t * history, int64_t history_stride,
                                            const int32_t * history_len, const fns_b200_params * params,
                                            int32_t * out_tokens, void * stream, char * error_text, int error_len) {
    auto fail_text = [&](int code, const char * what) {
        if (error_text && error_len > 0) std::snprintf(error_text, (size_t) error_len, "%s", what);
        return code;
    };
    if (device < 0 || device >= 64) return fail_text(FNS_B200_ERR_ARG, "device outside [0, 64)");
    if (!out_tokens || !params) return fail_text(FNS_B200_ERR_ARG, "out_tokens or params null");
    if (rows > kNoAllocRows) return fail_text(FNS_B200_ERR_CAPACITY, "rows > 64: the static scratch holds 64 rows per call");
    DeviceGuard g(device);
    if (!g.ok) return fail_text(FNS_B200_ERR_CUDA, "cannot make the device current");
    unsigned char * base = nullptr;
    {
        // Set-up, once per device, with that device current: ask the runtime where the array lives on it.
        std::lock_guard<std::mutex> hold(g_noalloc_lock);
        if (!g_noalloc_ptr[device]) {
            void * p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) return fail_text(FNS_B200_ERR_CUDA, cudaGetErrorString(e));
            g_noalloc_ptr[device] = static_cast<unsigned char *>(p);
        }
        base = g_noalloc_ptr[device];
    }
    fns_b200_sampler s{};  // a handle on the stack whose workspace is the static array; nothing is allocated
    s.device = device;
    s.max_rows = kNoAllocRows;
    s.max_vocab = 0x7fffffff;
    s.k_cap = kNoAllocK;
    s.max_history = FNS_B200_MAX_HISTORY;
    if (cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return fail_text(FNS_B200_ERR_CUDA, "cudaDeviceGetAttribute failed");
    s.cand = reinterpret_cast<uint64_t *>(base);
    s.cand_entries = kNoAllocCand;
    s.tickets = reinterpret_cast<unsigned *>(base + kNoAllocCand * sizeof(uint64_t));
    s.err = reinterpret_cast<int *>(base + kNoAllocCand * sizeof(uint64_t) + kNoAllocRows * sizeof(unsigned));
    // The array keeps whatever the last call left: the tickets and the error flag must start at zero.
    const cudaError_t e = cudaMemsetAsync(s.tickets, 0, kNoAllocRows * sizeof(unsigned) + sizeof(int), (cudaStream_t) stream);
    if (e != cudaSuccess) return fail_text(FNS_B200_ERR_CUDA, cudaGetErrorString(e));
    Plan pl;
    const int rc = run_select(&s, logits, dtype, row_stride, vocab, rows, 0, masks, mask_stride_words, history,
                              history_stride, history_len, nullptr, 0, params, nullptr, out_tokens, nullptr,
                              (cudaStream_t) stream, pl);
    if (rc != FNS_B200_OK) return fail_text(rc, s.msg);
    return FNS_B200_OK;
}
