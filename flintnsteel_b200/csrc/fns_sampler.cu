// fns_sampler.cu - the sampler kernels for sm_100a and the C ABI declared in include/fns_b200.h.
//
// Two kernels per call, both HBM-streaming / latency work with no contraction in it (no tensor cores):
//
//   k_select   grid (slices, rows).  One pass over a slice of one row of logits: 128-bit coalesced loads, the
//              grammar bitmask and the penalty history folded into a shared-memory bit set, and an exact
//              top-k of the slice by threshold filtering: elements that beat the current k-th best key are
//              appended to a shared buffer; when the buffer passes its high-water mark the block radix-selects
//              the best k and raises the threshold.  Replaces k_topk_part of the reference
//              (src/kernels.cu:624-648), which rescans its slice k times, and k_presence_apply / _col
//              (src/kernels.cu:724-742), which rewrite the whole row in place.
//   k_finalize grid (rows).  Merges the slices' candidates, then does the candidate softmax, top-p / min-p cut,
//              temperature weights and Philox draw of k_sample's tail (src/kernels.cu:698-720).
//
// Nothing here waits on another block, so there is no spin loop anywhere in the sampler.
#include "fns_device.cuh"

#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

namespace fnsb {

constexpr int kHashEmpty = -1;             // 0xffffffff
constexpr int kMaxMergeKeys = 8192;        // k_finalize holds the lists of one row in shared memory
constexpr int kMaxSlices = 128;
constexpr int kMaxSliceLen = 65536;        // a history table entry keeps the in-slice offset in 16 bits
constexpr int kSliceAlign = 1024;          // slice length granularity (elements); keeps loads 16-byte aligned

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
    int slice_len;
    int cap;         // candidate buffer entries
    int high_water;  // compaction trigger; cap - high_water >= elements one block iteration can append
    int ht_size;     // history table slots (power of two, multiple of kThreads), 0: no table
    uint64_t * cand;  // [rows][slices][k_cap] sorted keys, 0 = empty
    int * err;
};

struct SelectShared {
    SelectScratch sc;
    uint64_t thr_key;   // keys below this cannot be among the slice's best k
    float thr_value;    // x < thr_value  =>  key < thr_key
    uint32_t n_cand;
    uint64_t red[kThreads / 32];
};

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

// 16-byte load of VEC consecutive elements, widened to fp32.  Streaming: each logit is read once.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T * p, float (&out)[VEC]) {
    if constexpr (VEC == 1) {
        out[0] = to_float(*p);
    } else if constexpr (sizeof(T) == 4) {
        const float4 v = __ldcs(reinterpret_cast<const float4 *>(p));
        out[0] = v.x;
        out[1] = v.y;
        out[2] = v.z;
        out[3] = v.w;
    } else {
        const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(p));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[2 * j] = __uint_as_float(w[j] << 16);
            out[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

// Keeps the best k keys of buf[0 .. n_cand) in buf[0 .. k) and raises the threshold.  All threads; block
// synchronised on entry (every append is visible) and on exit.
__device__ void compact(uint64_t * buf, uint64_t * sel, int k, SelectShared & sh) {
    const int n = (int) sh.n_cand;
    if (n <= k) return;
    const uint64_t tau = block_kth_key(buf, n, k, sh.sc);
    const int got = block_take(buf, n, k, tau, sel, sh.sc);
    for (int i = threadIdx.x; i < got; i += kThreads) buf[i] = sel[i];
    if (threadIdx.x == 0) {
        sh.n_cand = (uint32_t) got;
        sh.thr_key = tau;
        sh.thr_value = key_floor_value(tau);
    }
    __syncthreads();
}

template <typename T, int VEC, int UNROLL>
__global__ void __launch_bounds__(kThreads) k_select(const SelectArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31;
    const int row = blockIdx.y, slice = blockIdx.x;
    const int W = a.n_draft + 1, win = row / W, col = row - win * W;
    const fns_b200_params p = a.params ? a.params[win] : a.p0;
    const int k = p.temperature <= 0.0f ? 1 : clamp_k(p.top_k, a.k_cap);
    const int lo = slice * a.slice_len;
    const int n_s = min(a.vocab, lo + a.slice_len) - lo;
    uint64_t * out = a.cand + ((size_t) row * a.slices + slice) * a.k_cap;
    if (n_s <= 0) {
        for (int j = tid; j < k; j += kThreads) out[j] = 0ull;
        return;
    }
    // shared memory: candidate buffer | selection staging | slice bit set | history table | scalars
    uint64_t * buf = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t * sel = buf + a.cap;
    uint32_t * eff = reinterpret_cast<uint32_t *>(sel + a.k_cap);
    int * htab = reinterpret_cast<int *>(eff + a.slice_len / 32);
    SelectShared & sh = *reinterpret_cast<SelectShared *>(htab + a.ht_size);

    const T * x = reinterpret_cast<const T *>(a.logits) + (size_t) row * a.row_stride + lo;
    const uint32_t * mrow = a.masks ? a.masks + (size_t) row * a.mask_stride + (lo >> 5) : nullptr;

    // 1. The slice's bit set: bit e = element lo + e is allowed.  Bits past the end of the row are 0, so the
    // streaming loop needs no other bounds handling for the mask.
    const int words = (n_s + 31) >> 5;
    for (int w = tid; w < words; w += kThreads) {
        uint32_t m = mrow ? mrow[w] : 0xffffffffu;
        if (w == words - 1 && (n_s & 31)) m &= (1u << (n_s & 31)) - 1u;
        eff[w] = m;
    }
    for (int i = tid; i < a.ht_size; i += kThreads) htab[i] = kHashEmpty;
    if (tid == 0) {
        sh.n_cand = 0u;
        sh.thr_key = 0ull;
        sh.thr_value = -FLT_MAX;
    }
    uint64_t best = 0ull;  // k == 1: this thread's best key
    float best_v = -FLT_MAX;
    __syncthreads();

    // 2. Penalties.  The row's history (plus the draft prefix of a verification column) is scattered into a
    // shared hash table: in-slice offset -> occurrence count.  Each distinct id is then removed from the bit
    // set and offered once as a candidate with its penalised value, so the streaming loop below pays nothing
    // for penalties.  Traffic: 4 bytes per history id (every slice reads the list; it stays in L2).
    const bool any_pen = p.repetition != 1.0f || p.presence != 0.0f || p.frequency != 0.0f;
    int n_hist = 0;
    if (a.history && a.history_len) {
        n_hist = a.history_len[win];
        n_hist = n_hist < 0 ? 0 : (n_hist > (int) a.history_stride ? (int) a.history_stride : n_hist);
    }
    const int n_pen = n_hist + (a.draft ? col : 0);
    if (any_pen && n_pen > 0 && a.ht_size > 0) {
        const int32_t * hrow = a.history ? a.history + (size_t) win * a.history_stride : nullptr;
        const int32_t * drow = a.draft ? a.draft + (size_t) win * a.n_draft : nullptr;
        const uint32_t hmask = (uint32_t) a.ht_size - 1u;
        for (int j = tid; j < n_pen; j += kThreads) {
            const int32_t id = j < n_hist ? hrow[j] : drow[j - n_hist];
            const uint32_t off = (uint32_t) (id - a.id_base - lo);
            if (off >= (uint32_t) n_s || id < a.id_base) continue;
            uint32_t h = (off * 2654435761u) & hmask;
            for (int probe = 0; probe <= a.ht_size; ++probe) {
                if (probe == a.ht_size) { atomicExch(a.err, 2); break; }  // table full: cannot happen (load <= 1/2)
                int cur = htab[h];
                if (cur == kHashEmpty) {
                    cur = atomicCAS(&htab[h], kHashEmpty, (int) ((off << 16) | 1u));
                    if (cur == kHashEmpty) break;
                }
                if (((uint32_t) cur >> 16) == off) {
                    atomicAdd(&htab[h], 1);
                    break;
                }
                h = (h + 1u) & hmask;
            }
        }
        __syncthreads();
        for (int base = 0; base < a.ht_size; base += kThreads) {
            if (k > 1 && __syncthreads_or(*(volatile uint32_t *) &sh.n_cand > (uint32_t) a.high_water))
                compact(buf, sel, k, sh);
            const int e = htab[base + tid];
            if (e == kHashEmpty) continue;
            const uint32_t off = (uint32_t) e >> 16;
            const float cnt = (float) ((uint32_t) e & 0xffffu);
            const uint32_t bit = 1u << (off & 31);
            const uint32_t old = atomicAnd(&eff[off >> 5], ~bit);
            if (!(old & bit)) continue;  // not allowed by the grammar mask
            float v = to_float(x[off]);
            // each step rounded on its own: no fused multiply-add
            v = v > 0.0f ? __fdiv_rn(v, p.repetition) : __fmul_rn(v, p.repetition);
            v = __fsub_rn(v, __fmul_rn(p.frequency, cnt));
            v = __fsub_rn(v, p.presence);
            if (!is_finite(v)) continue;
            const uint64_t key = make_key(v, (uint32_t) (a.id_base + lo) + off);
            if (k == 1) {
                if (key > best) { best = key; best_v = v; }
            } else if (key >= *(volatile uint64_t *) &sh.thr_key) {
                const uint32_t pos = atomicAdd(&sh.n_cand, 1u);
                if (pos < (uint32_t) a.cap) buf[pos] = key;
                else atomicExch(a.err, 1);
            }
        }
        __syncthreads();
    }

    // 3. The streaming pass.  Per block iteration every thread takes UNROLL vectors; a vector is touched only
    // if the bit set allows one of its elements.
    const int n_vec = (n_s + VEC - 1) / VEC;
    const uint32_t id0 = (uint32_t) (a.id_base + lo);
    for (int v0 = 0; v0 < n_vec; v0 += kThreads * UNROLL) {
        if (k > 1 && __syncthreads_or(*(volatile uint32_t *) &sh.n_cand > (uint32_t) a.high_water))
            compact(buf, sel, k, sh);
        float xv[UNROLL][VEC];
        uint32_t mb[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int e = (v0 + u * kThreads + tid) * VEC;
            mb[u] = e < n_s ? (eff[e >> 5] >> (e & 31)) & ((VEC == 32) ? 0xffffffffu : ((1u << VEC) - 1u)) : 0u;
            if (mb[u]) {
                if (VEC == 1 || e + VEC <= n_s) {
                    load_vec<T, VEC>(x + e, xv[u]);
                } else {  // the row's ragged end
#pragma unroll
                    for (int j = 0; j < VEC; ++j) xv[u][j] = e + j < n_s ? to_float(x[e + j]) : 0.0f;
                }
            }
        }
        if (k == 1) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (!mb[u]) continue;
                const int e = (v0 + u * kThreads + tid) * VEC;
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    const float xi = xv[u][j];
                    if (((mb[u] >> j) & 1u) && xi >= best_v && xi <= FLT_MAX) {
                        const uint64_t key = make_key(xi, id0 + (uint32_t) (e + j));
                        if (key > best) { best = key; best_v = xi; }
                    }
                }
            }
            continue;
        }
        const float thr_v = *(volatile float *) &sh.thr_value;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            uint32_t pass = 0u;
            if (mb[u]) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) pass |= (xv[u][j] >= thr_v ? 1u : 0u) << j;
                pass &= mb[u];
            }
            if (!__any_sync(kFull, pass != 0u)) continue;
            const uint64_t thr_key = *(volatile uint64_t *) &sh.thr_key;
            const int e = (v0 + u * kThreads + tid) * VEC;
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                uint64_t key = 0ull;
                bool take = (pass >> j) & 1u;
                if (take) {
                    const float xi = xv[u][j];
                    key = make_key(xi, id0 + (uint32_t) (e + j));
                    take = xi <= FLT_MAX && key >= thr_key;  // +inf is never a candidate
                }
                const uint32_t ballot = __ballot_sync(kFull, take);
                if (ballot) {
                    uint32_t base = 0u;
                    const int leader = __ffs(ballot) - 1;
                    if (lane == leader) base = atomicAdd(&sh.n_cand, (uint32_t) __popc(ballot));
                    base = __shfl_sync(kFull, base, leader);
                    if (take) {
                        const uint32_t pos = base + (uint32_t) __popc(ballot & ((1u << lane) - 1u));
                        if (pos < (uint32_t) a.cap) buf[pos] = key;
                        else atomicExch(a.err, 1);
                    }
                }
            }
        }
    }
    __syncthreads();

    // 4. The slice's answer: its best k keys in the total order.
    if (k == 1) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const uint64_t other = __shfl_xor_sync(kFull, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) sh.red[tid >> 5] = best;
        __syncthreads();
        if (tid == 0) {
            uint64_t b = sh.red[0];
            for (int w = 1; w < kThreads / 32; ++w) b = sh.red[w] > b ? sh.red[w] : b;
            out[0] = b;
        }
        return;
    }
    const int n = (int) min(sh.n_cand, (uint32_t) a.cap);
    const uint64_t tau = block_kth_key(buf, n, k, sh.sc);
    const int got = block_take(buf, n, k, tau, sel, sh.sc);
    block_rank_sort(sel, got, out);
    for (int j = got + tid; j < k; j += kThreads) out[j] = 0ull;
}

// ---- finalize ---------------------------------------------------------------------------------------------
struct FinalArgs {
    const uint64_t * keys;        // internal lists (sorted keys, 0 = empty), or
    const fns_b200_cand * cands;  // external lists; entry j of list l of row r at r * row_stride + l * list_stride + j
    int lists;
    int list_len;  // entries to read from each list
    int64_t list_stride;
    int64_t row_stride;
    int k_cap;
    int n_draft;
    const fns_b200_params * params;
    fns_b200_params p0;
    int32_t * out_tokens;      // may be null (merge only)
    fns_b200_cand * out_cands; // may be null; [rows][k_cap]
};

struct FinalShared {
    SelectScratch sc;
    uint32_t n_keys;
    int nk;
    int keep;
};

__global__ void __launch_bounds__(kThreads) k_finalize(const FinalArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x;
    const int row = blockIdx.x;
    const int W = a.n_draft + 1, win = row / W, col = row - win * W;
    fns_b200_params p = a.params ? a.params[win] : a.p0;
    p.counter += (uint64_t) col;  // column c of a window draws with counter + c (src/engine.cu:756)
    const bool greedy = p.temperature <= 0.0f;
    const int k = greedy ? 1 : clamp_k(p.top_k, a.k_cap);
    const int take_len = a.keys ? min(a.list_len, k) : a.list_len;  // internal lists hold exactly the row's k

    // shared memory: all keys of the row | selection staging | sorted result | p / acc (fp64)
    const int max_keys = a.lists * a.list_len;
    uint64_t * buf = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t * sel = buf + max_keys;
    uint64_t * sorted = sel + a.k_cap;
    double * pj = reinterpret_cast<double *>(sorted + a.k_cap);
    double * acc = pj + a.k_cap;
    FinalShared & sh = *reinterpret_cast<FinalShared *>(acc + a.k_cap);

    if (tid == 0) {
        sh.n_keys = 0u;
        sh.nk = 0;
        sh.keep = 0;
    }
    for (int j = tid; j < a.k_cap; j += kThreads) sorted[j] = 0ull;
    __syncthreads();
    // Gather the non-empty keys (their order does not matter: the selection below is by key alone, which makes
    // the result independent of how many slices or shards produced the lists).
    const size_t row_base = (size_t) row * a.row_stride;
    for (int i = tid; i < a.lists * take_len; i += kThreads) {
        const int l = i / take_len, j = i - l * take_len;
        const size_t at = row_base + (size_t) l * a.list_stride + j;
        const uint64_t key = a.keys ? a.keys[at] : cand_to_key(a.cands[at]);
        if (key != 0ull) buf[atomicAdd(&sh.n_keys, 1u)] = key;
    }
    __syncthreads();
    const int n = (int) sh.n_keys;
    const uint64_t tau = block_kth_key(buf, n, k, sh.sc);
    const int got = block_take(buf, n, k, tau, sel, sh.sc);
    block_rank_sort(sel, got, sorted);
    __syncthreads();
    const int nk = got;  // number of candidates (fewer than k allowed tokens: src/kernels.cu:698-699)
    if (a.out_cands)
        for (int j = tid; j < a.k_cap; j += kThreads) a.out_cands[(size_t) row * a.k_cap + j] = key_to_cand(sorted[j]);
    if (!a.out_tokens) return;
    if (nk == 0) {
        if (tid == 0) a.out_tokens[row] = -1;
        return;
    }
    if (greedy || nk == 1) {
        if (tid == 0) a.out_tokens[row] = key_id(sorted[0]);
        return;
    }
    // k_sample's tail (src/kernels.cu:702-719).  exp and the quotients are per-element and computed in parallel;
    // the three running sums keep the reference's left-to-right order, one chain per thread: `sum` then `cum`
    // on thread 0, the weight prefix (which is both wsum and the inverse-CDF walk's acc) on thread 32.
    const double v0 = (double) key_value(sorted[0]);
    for (int j = tid; j < nk; j += kThreads) {
        const double d = (double) key_value(sorted[j]) - v0;
        pj[j] = exp(d);
        acc[j] = exp(d / p.temperature);
    }
    __syncthreads();
    if (tid == 0) {
        double sum = 0.0;
        for (int j = 0; j < nk; ++j) sum += pj[j];
        int keep = nk;
        double cum = 0.0;
        for (int j = 0; j < nk; ++j) {
            cum += pj[j] / sum;
            if (cum >= p.top_p) { keep = j + 1; break; }
        }
        if (p.min_p > 0.0f) {
            int m = 1;
            while (m < keep && pj[m] >= (double) p.min_p) ++m;
            keep = m;
        }
        sh.keep = keep;
    } else if (tid == 32) {
        double run = 0.0;
        for (int j = 0; j < nk; ++j) {
            run += acc[j];
            acc[j] = run;
        }
    }
    __syncthreads();
    if (tid == 0) {
        const int keep = sh.keep;
        const double wsum = acc[keep - 1];
        const double u = philox_uniform(p.seed, p.counter) * wsum;
        int pick = keep - 1;
        for (int j = 0; j < keep; ++j)
            if (u < acc[j]) { pick = j; break; }
        a.out_tokens[row] = key_id(sorted[pick]);
    }
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
    uint64_t * cand;   // [max_rows][kMaxSlices or fewer][k_cap]
    size_t cand_entries;
    int * err;
    int64_t launches;
    bool prof_on;
    int prof_calls;                   // calls recorded so far
    std::vector<cudaEvent_t> prof_ev; // three per call: before select, after select, after finalize
    char msg[256];
};

namespace {

struct Plan {
    int slices, slice_len, cap, high_water, ht_size, vec, unroll;
    size_t smem_select, smem_final;
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

// Launch geometry.  Slices per row: enough blocks to fill the GPU (about four 256-thread blocks per SM) when
// rows are few, long slices when rows are many (the per-slice selection cost is amortised over the stream).
bool make_plan(const fns_b200_sampler * s, int dtype, int vocab, int rows, int hist_bound, bool aligned, Plan & pl) {
    const int k_cap = s->k_cap;
    const int min_slices = (vocab + kMaxSliceLen - 1) / kMaxSliceLen;
    int max_slices = kMaxMergeKeys / k_cap;
    if (max_slices > kMaxSlices) max_slices = kMaxSlices;
    if (min_slices > max_slices) return false;
    int want = s->force_slices > 0 ? s->force_slices : (s->sm_count * 4 + rows - 1) / rows;
    const int by_len = (vocab + 2 * kSliceAlign - 1) / (2 * kSliceAlign);  // no slice shorter than 2048 elements
    if (s->force_slices <= 0 && want > by_len) want = by_len;
    if (want < min_slices) want = min_slices;
    if (want > max_slices) want = max_slices;
    if (want < 1) want = 1;
    pl.slice_len = round_up((vocab + want - 1) / want, kSliceAlign);
    if (pl.slice_len > kMaxSliceLen) pl.slice_len = kMaxSliceLen;
    pl.slices = (vocab + pl.slice_len - 1) / pl.slice_len;
    pl.vec = aligned ? (dtype == FNS_B200_BF16 ? 8 : 4) : 1;
    pl.unroll = 2;
    const int tile = kThreads * pl.unroll * pl.vec;
    pl.high_water = 3 * k_cap > 1024 ? 3 * k_cap : 1024;
    pl.cap = pl.high_water + (tile > kThreads ? tile : kThreads);
    pl.ht_size = 0;
    if (hist_bound > 0) {
        const int distinct = hist_bound < pl.slice_len ? hist_bound : pl.slice_len;
        pl.ht_size = next_pow2(2 * distinct);
        if (pl.ht_size < kThreads) pl.ht_size = kThreads;
    }
    pl.smem_select = (size_t) pl.cap * 8 + (size_t) k_cap * 8 + (size_t) pl.slice_len / 8 + (size_t) pl.ht_size * 4 +
                     sizeof(SelectShared) + 16;
    return pl.smem_select <= 200 * 1024;
}

size_t final_smem(int lists, int list_len, int k_cap) {
    return (size_t) lists * list_len * 8 + (size_t) k_cap * 8 * 4 + sizeof(FinalShared) + 16;
}

template <typename T, int VEC>
cudaError_t launch_select_t(const SelectArgs & a, int rows, size_t smem, cudaStream_t st) {
    auto kern = k_select<T, VEC, 2>;
    static bool configured[64] = {};  // per device: the opt-in to large dynamic shared memory is sticky
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    kern<<<dim3((unsigned) a.slices, (unsigned) rows), kThreads, smem, st>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_select(const SelectArgs & a, int dtype, int vec, int rows, size_t smem, cudaStream_t st) {
    if (dtype == FNS_B200_BF16)
        return vec == 8 ? launch_select_t<__nv_bfloat16, 8>(a, rows, smem, st)
                        : launch_select_t<__nv_bfloat16, 1>(a, rows, smem, st);
    return vec == 4 ? launch_select_t<float, 4>(a, rows, smem, st) : launch_select_t<float, 1>(a, rows, smem, st);
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
    k_finalize<<<(unsigned) rows, kThreads, smem, st>>>(a);
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
               const fns_b200_params * params, const fns_b200_params * p0, cudaStream_t st, Plan & pl) {
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
    a.high_water = pl.high_water;
    a.ht_size = pl.ht_size;
    a.cand = s->cand;
    a.err = s->err;
    const bool prof = s->prof_on && (size_t) (s->prof_calls + 1) * 3 <= s->prof_ev.size();
    if (prof) cudaEventRecord(s->prof_ev[(size_t) s->prof_calls * 3], st);
    const cudaError_t e = launch_select(a, dtype, pl.vec, rows, pl.smem_select, st);
    if (e != cudaSuccess) return fail_cuda(s, e, "select launch");
    if (prof) cudaEventRecord(s->prof_ev[(size_t) s->prof_calls * 3 + 1], st);
    ++s->launches;
    return FNS_B200_OK;
}

int run_final_internal(fns_b200_sampler * s, const Plan & pl, int rows, int n_draft, const fns_b200_params * params,
                       const fns_b200_params * p0, int32_t * out_tokens, fns_b200_cand * out_cands, cudaStream_t st) {
    FinalArgs f{};
    f.keys = s->cand;
    f.lists = pl.slices;
    f.list_len = s->k_cap;
    f.list_stride = s->k_cap;
    f.row_stride = (int64_t) pl.slices * s->k_cap;
    f.k_cap = s->k_cap;
    f.n_draft = n_draft;
    f.params = params;
    if (p0) f.p0 = *p0;
    f.out_tokens = out_tokens;
    f.out_cands = out_cands;
    const cudaError_t e = launch_final(f, rows, st);
    if (e != cudaSuccess) return fail_cuda(s, e, "finalize launch");
    ++s->launches;
    if (s->prof_on && (size_t) (s->prof_calls + 1) * 3 <= s->prof_ev.size()) {
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
        cudaMalloc(&s->err, sizeof(int)) != cudaSuccess || cudaMemset(s->err, 0, sizeof(int)) != cudaSuccess) {
        if (s->cand) cudaFree(s->cand);
        if (s->err) cudaFree(s->err);
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
                        history_len, nullptr, 0, params, nullptr, (cudaStream_t) stream, pl);
    if (rc != FNS_B200_OK) return rc;
    return run_final_internal(s, pl, rows, 0, params, nullptr, out_tokens, nullptr, (cudaStream_t) stream);
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
                        nullptr, params_host, (cudaStream_t) stream, pl);
    if (rc != FNS_B200_OK) return rc;
    return run_final_internal(s, pl, 1, 0, nullptr, params_host, out_token, nullptr, (cudaStream_t) stream);
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
                        history_stride, history_len, nullptr, 0, params, nullptr, (cudaStream_t) stream, pl);
    if (rc != FNS_B200_OK) return rc;
    return run_final_internal(s, pl, rows, 0, params, nullptr, nullptr, out_cands, (cudaStream_t) stream);
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
    f.n_draft = 0;
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
                        history_len, draft, n_draft, params, nullptr, (cudaStream_t) stream, pl);
    if (rc != FNS_B200_OK) return rc;
    rc = run_final_internal(s, pl, rows, n_draft, params, nullptr, out_tokens, nullptr, (cudaStream_t) stream);
    if (rc != FNS_B200_OK) return rc;
    k_accept<<<(unsigned) ((windows + 127) / 128), 128, 0, (cudaStream_t) stream>>>(out_tokens, draft, n_draft, windows,
                                                                                  out_accept);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(s, e, "accept launch");
    ++s->launches;
    return FNS_B200_OK;
}

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
