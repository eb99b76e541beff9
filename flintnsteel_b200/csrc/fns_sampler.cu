// fns_sampler.cu - the sampler kernels for sm_100a and the C ABI declared in include/fns_b200.h.
//
// HBM-streaming / latency work with no contraction in it (no tensor cores):
//
//   k_select   grid (slices, rows); one block per (row, slice).  With many rows a slice is the whole row and a
//              block has 512 threads (two per SM: 296 rows in flight at once); with few rows a row is cut into
//              slices so that the whole GPU works on it.  Per slice:
//                1. the grammar bitmask becomes a shared-memory bit set and a list of the 512-byte segments that
//                   have an allowed id; every history id clears its bit, and the thread that clears it owns the id;
//                2. pass 1 streams the listed segments once with 128-bit coalesced loads, two groups in flight,
//                   and keeps nothing but maxima: per thread the maximum seen, per vector group one flag "reaches
//                   the running bound".  The bound is a value that at least k elements of the slice are known to
//                   reach, found from the threads' maxima alone; nothing is appended, nothing is compared element
//                   by element, and what the mask excludes is never loaded;
//                3. the bound is tightened to (nearly) the k-th largest thread maximum with a counted bisection;
//                4. the few flagged vectors of the few threads whose maximum reaches the bound are read again
//                   (L2) and their elements that reach it (about k of them) go to a shared buffer; the penalised
//                   history ids join them;
//                5. the best k of the buffer, sorted, are the slice's answer (rank by counting; if many equal
//                   values overflow the buffer, everything is offered again with compaction, so any input is
//                   handled exactly);
//                6. the last block of a row to finish (a ticket, no waiting) merges the slices' lists and does
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
#include <type_traits>
#include <mutex>
#include <vector>

namespace fnsb {


constexpr int kMaxMergeKeys = 8192;   // k_finalize holds the lists of one row in shared memory
constexpr int kMaxSlices = 128;
constexpr int kEpochElems = 16;       // elements per thread and group (a slice is at most 16 groups of a 256-thread
                                      // block's elements, or 32 of a 512-thread block's: 128 flag bits per thread)
constexpr int kMaxWarps = 16;
constexpr int kRankSelectMax = 384;   // candidate sets up to this size are ranked by counting

struct SelectArgs {
    const void * logits;
    int64_t row_stride;
    int vocab;
    int id_base;
    const uint32_t * masks;
    int64_t mask_stride;
    const int32_t * mask_rows;  // null, or per row: which row of `masks` holds its mask (rows may share one)
    const int32_t * history;
    int64_t history_stride;
    const int32_t * history_len;
    const int32_t * draft;  // verification windows: [windows][n_draft]; row = window * (n_draft + 1) + column
    int n_draft;
    const fns_b200_params * params;  // per window (per row when n_draft == 0); null: p0
    fns_b200_params p0;
    int k_cap;
    int slices;
    int slice_len;   // a multiple of threads * 16 elements
    int cap;         // candidate buffer entries (>= 4 * k_cap)
    int trigger;     // compact when the buffer holds this many
    int own_cap;     // entries of the list of owned history ids (a multiple of 4), 0: no penalties
    int list_cap;    // entries of the work list of the second pass
    int seg_cap;     // segments of a slice (32 vectors each), a multiple of 4
    int n_stages;    // k_ring: stages of 8,192 elements that cover the row
    int ring_depth;  // k_ring: stages of shared memory that the copies rotate through
    int ring_off;    // k_ring: where the ring starts in the block's shared memory
    int own_off;     // k_ring: where the list of owned history ids starts
    int hist_cap;    // k_cluster: history ids per row that are staged in shared memory (a multiple of 4)
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
    uint32_t n_own;       // history ids of the slice that the mask allows, each once
    uint32_t n_vl;        // cursor of the work list
    uint32_t n_seg;       // segments with an allowed element
    int keep;
    int is_last;
    __align__(16) float warp_bound[kMaxWarps];  // per warp: a value that r of its lanes have reached
    uint32_t warp_top[kMaxWarps];               // per warp: its largest thread maximum (as an order word)
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
// end, merged into sorted[0 .. k): the selection rounds of k_sample (src/kernels.cu:680-695).  Returns the number
// of candidates (< k when fewer tokens are allowed, src/kernels.cu:698-699); sorted[nk .. k_cap) = 0.
//   1. Witnesses: the first few keys of every list, at least k in all.  The k-th largest witness (found by
//      counting, every witness against every other) is a bar that k keys reach, so the best k keys of the union
//      all reach it.
//   2. Every key that reaches the bar moves to a scratch list (`spare`, room for spare_len keys).  The lists are
//      sorted, so these are a prefix of each: little more than k keys unless one list holds most of the best.
//   3. The scratch list is ranked by counting; ranks below k are the answer, in order.
// If there are too few witnesses or the scratch list overflows, a radix selection over all keys does the job.
// All NT threads; block synchronised on entry and exit.
template <int NT>
__device__ int merge_lists(uint64_t * buf, int lists, int len, uint64_t * sel, uint64_t * sorted, uint64_t * spare,
                           int spare_len, SelectScratch & sc, int k, int k_cap) {
    const int tid = threadIdx.x;
    const int total = lists * len;
    int depth = (k + lists - 1) / lists + 2;
    if (depth > len) depth = len;
    const int n_wit = lists * depth;
    for (int j = tid; j < k_cap; j += NT) sorted[j] = 0ull;
    if (tid == 0) {
        sc.count = 0u;
        sc.or_hi = 0u;  // the bar, as two words
        sc.or_lo = 0u;
    }
    __syncthreads();
    // (the witnesses are first copied side by side, so that the counting loop is one flat, unrolled walk)
    uint64_t * wit = spare;  // n_wit <= spare_len is checked below; the scratch list is written only afterwards
    const bool flat = n_wit <= spare_len;
    if (flat)
        for (int i = tid; i < n_wit; i += NT) wit[i] = buf[(i / depth) * len + (i % depth)];
    __syncthreads();
    for (int i = tid; i < n_wit; i += NT) {
        const uint64_t key = buf[(i / depth) * len + (i % depth)];
        if (key == 0ull) continue;
        int rank = 0;
        if (flat) {
#pragma unroll 8
            for (int j = 0; j < n_wit; ++j) rank += wit[j] > key ? 1 : 0;
        } else {
            for (int l = 0; l < lists; ++l)
                for (int d = 0; d < depth; ++d) rank += buf[l * len + d] > key ? 1 : 0;
        }
        if (rank == k - 1) {
            sc.or_hi = (uint32_t) (key >> 32);
            sc.or_lo = (uint32_t) key;
        }
    }
    __syncthreads();
    const uint64_t bar = ((uint64_t) sc.or_hi << 32) | sc.or_lo;  // 0: fewer than k witnesses
    for (int i = tid; i < total; i += NT) {
        const uint64_t key = buf[i];
        if (key != 0ull && key >= bar) {
            const uint32_t at = atomicAdd(&sc.count, 1u);
            if (at < (uint32_t) spare_len) spare[at] = key;
        }
    }
    __syncthreads();
    const int n = (int) sc.count;
    int nk;
    if (n <= spare_len) {
        nk = block_rank_select<NT>(spare, n, k, sorted);
        __syncthreads();
        return nk;
    }
    // the long way: squeeze out the empty slots (the order does not matter to the selection), then select
    __syncthreads();
    if (tid == 0) sc.count = 0u;
    __syncthreads();
    for (int base = 0; base < total; base += NT) {
        const int i = base + tid;
        const uint64_t key = i < total ? buf[i] : 0ull;
        __syncthreads();
        if (key != 0ull) buf[atomicAdd(&sc.count, 1u)] = key;
        __syncthreads();
    }
    const int m = (int) sc.count;
    __syncthreads();
    const uint64_t tau = block_kth_key<NT>(buf, m, k, sc);
    nk = block_take<NT>(buf, m, k, tau, sel, sc);
    block_rank_sort<NT>(sel, nk, sorted);
    __syncthreads();
    return nk;
}

// The one-warp part of the draw for at most 64 candidates: pj[j] = exp(v_j - v_0) and acc[j] = exp((v_j - v_0) / T)
// are in shared memory, the uniform in sc.hist.  Lane 0 walks the running sums left to right, as the reference adds
// (src/kernels.cu:702-719); every lane then holds candidates j = lane and lane + 32, and the three decisions (top-p
// cut, min-p cut, inverse-CDF hit) are the first set bits of ballots.  Called by the 32 threads of warp 0.
__device__ __forceinline__ void draw_warp(const uint64_t * sorted, int nk, double * pj, double * acc, double * qj,
                                          SelectScratch & sc, const fns_b200_params & p, int32_t * out_token) {
    const int tid = threadIdx.x;
    const int lane = tid, hi = tid + 32;
    double sum = 0.0;
    if (lane == 0) {
        double run = 0.0;
        int j = 0;
        for (; j + 4 <= nk; j += 4) {
            double a4[4], w4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                a4[u] = pj[j + u];
                w4[u] = acc[j + u];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                sum += a4[u];
                run += w4[u];
                acc[j + u] = run;
            }
        }
        for (; j < nk; ++j) {
            sum += pj[j];
            run += acc[j];
            acc[j] = run;
        }
    }
    __syncwarp();
    sum = __shfl_sync(kFull, sum, 0);
    const double p0 = lane < nk ? pj[lane] : 0.0, p1 = hi < nk ? pj[hi] : 0.0;
    if (lane < nk) qj[lane] = p0 / sum;
    if (hi < nk) qj[hi] = p1 / sum;
    __syncwarp();
    if (lane == 0) {
        double run = 0.0;
        int j = 0;
        for (; j + 4 <= nk; j += 4) {
            double q4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) q4[u] = qj[j + u];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                run += q4[u];
                qj[j + u] = run;
            }
        }
        for (; j < nk; ++j) {
            run += qj[j];
            qj[j] = run;
        }
    }
    __syncwarp();
    auto first_of = [&](bool lo_bit, bool hi_bit, int none) -> int {  // index of the first candidate with the property
        const uint32_t b0 = __ballot_sync(kFull, lo_bit), b1 = __ballot_sync(kFull, hi_bit);
        return b0 ? __ffs(b0) - 1 : (b1 ? 31 + __ffs(b1) : none);
    };
    const int cut = first_of(lane < nk && qj[lane] >= (double) p.top_p, hi < nk && qj[hi] >= (double) p.top_p, nk - 1) + 1;
    int keep = cut;
    if (p.min_p > 0.0f) {
        const int low = first_of(lane >= 1 && lane < nk && !(p0 >= (double) p.min_p), hi < nk && !(p1 >= (double) p.min_p), nk);
        keep = low < keep ? low : keep;
    }
    const double wsum = acc[keep - 1];
    const double u = reinterpret_cast<volatile double *>(&sc.hist[0])[1] * wsum;
    const int pick = first_of(lane < keep && u < acc[lane], hi < keep && u < acc[hi], keep - 1);
    if (lane == 0) *out_token = key_id(sorted[pick]);
}

// The tail of k_sample (src/kernels.cu:698-720) over the nk sorted candidates: candidate softmax, top-p / min-p
// cut, temperature weights, Philox draw.  exp and the quotients are per-element and run in parallel; for up to 64
// candidates the three running sums keep the reference's left-to-right order (draw_warp: `sum` and the weight
// prefix - which is both wsum and the acc of the inverse-CDF walk - side by side, then `cum`).  qj aliases the
// selection staging (k_cap doubles).  All NT threads; block synchronised on entry.  p.counter is the counter of
// this row.
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
    if (nk <= 64 && NT >= 160) {
        // The usual case, at most 64 candidates: after the exponentials (threads 0-63 and 64-127, side by side, the
        // uniform on thread 128) ONE warp does the rest without another block barrier.  Lane 0 walks the running
        // sums left to right, as the reference adds; every lane then holds candidates j = lane and lane + 32, and
        // the three decisions (top-p cut, min-p cut, inverse-CDF hit) are the first set bits of ballots.
        if (tid < 128) {
            const int j = tid & 63;
            if (j < nk) {
                const double d = (double) key_value(sorted[j]) - v0;
                if (tid < 64) pj[j] = exp(d);
                else acc[j] = exp(d / p.temperature);
            }
        } else if (tid == 128) {
            reinterpret_cast<volatile double *>(&sc.hist[0])[1] = philox_uniform(p.seed, p.counter);
        }
        __syncthreads();
        if (tid >= 32) return;
        draw_warp(sorted, nk, pj, acc, qj, sc, p, out_token);
        return;
    }
    // More candidates (only with k_cap > 64, which the reference does not have: there the summation order is ours to
    // choose).  The two exponentials of a candidate go to different halves of the block; the two running sums - the
    // candidate probabilities and the temperature weights - are made together by a blocked scan: every thread adds
    // up its own few consecutive entries, a warp scan joins the threads, the warps' totals join the warps.
    {
        const bool second = tid >= NT / 2;
        for (int j = second ? tid - NT / 2 : tid; j < nk; j += NT / 2) {
            const double d = (double) key_value(sorted[j]) - v0;
            if (second) acc[j] = exp(d / p.temperature);
            else pj[j] = exp(d);
        }
    }
    if (tid == 0) reinterpret_cast<volatile double *>(&sc.hist[0])[1] = philox_uniform(p.seed, p.counter);
    __syncthreads();
    {
        constexpr int kWarpsT = NT / 32;
        double * warp_p = reinterpret_cast<double *>(&sc.hist[16]);   // [kWarpsT] totals of the warps' probabilities
        double * warp_w = warp_p + kWarpsT;                            // [kWarpsT] ... of their weights
        static_assert(16 + 4 * kWarpsT <= 256, "the warps' totals fit the scratch histogram");
        const int per = (nk + NT - 1) / NT;  // consecutive entries per thread
        const int j0 = tid * per;
        double sp = 0.0, sw = 0.0;
        for (int j = j0; j < j0 + per && j < nk; ++j) {
            sp += pj[j];
            sw += acc[j];
            qj[j] = sp;   // running sums inside the thread's stretch; the offsets follow
            acc[j] = sw;
        }
        double ip = sp, iw = sw;  // inclusive over the lanes of the warp
        const int lane_t = tid & 31, warp_t = tid >> 5;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double tp = __shfl_up_sync(kFull, ip, o), tw = __shfl_up_sync(kFull, iw, o);
            if (lane_t >= o) {
                ip += tp;
                iw += tw;
            }
        }
        if (lane_t == 31) {
            warp_p[warp_t] = ip;
            warp_w[warp_t] = iw;
        }
        __syncthreads();
        double op = ip - sp, ow = iw - sw;  // what precedes this thread's stretch
        for (int w = 0; w < warp_t; ++w) {
            op += warp_p[w];
            ow += warp_w[w];
        }
        for (int j = j0; j < j0 + per && j < nk; ++j) {
            qj[j] += op;
            acc[j] += ow;
        }
        __syncthreads();
        const double sum = qj[nk - 1];
        for (int j = tid; j < nk; j += NT) qj[j] = qj[j] / sum;  // the running probability
    }
    volatile uint32_t * first_cut = &sc.hist[8];   // first j + 1 whose running probability reaches top_p
    volatile uint32_t * first_low = &sc.hist[9];   // first j >= 1 whose probability is below min_p
    volatile uint32_t * first_hit = &sc.hist[10];  // first j whose running weight exceeds the draw
    if (tid == 0) {
        *first_cut = (uint32_t) nk;
        *first_low = (uint32_t) nk;
        *first_hit = 0xffffffffu;
    }
    __syncthreads();
    // `cum >= top_p` first holds at the smallest such j (the sums never decrease); min_p keeps the longest prefix of
    // the rest whose probabilities reach it
    for (int j = tid; j < nk; j += NT) {
        if (qj[j] >= (double) p.top_p) atomicMin(const_cast<uint32_t *>(first_cut), (uint32_t) j + 1u);
        if (p.min_p > 0.0f && j >= 1 && !(pj[j] >= (double) p.min_p)) atomicMin(const_cast<uint32_t *>(first_low), (uint32_t) j);
    }
    __syncthreads();
    const int keep = (int) min(*first_cut, *first_low);
    const double wsum = acc[keep - 1];
    const double u = reinterpret_cast<volatile double *>(&sc.hist[0])[1] * wsum;
    for (int j = tid; j < keep; j += NT)
        if (u < acc[j]) atomicMin(const_cast<uint32_t *>(first_hit), (uint32_t) j);
    __syncthreads();
    if (tid == 0) {
        const uint32_t hit = *first_hit;
        *out_token = key_id(sorted[hit == 0xffffffffu ? keep - 1 : (int) hit]);
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

// The running bound of pass 1 (every thread of the block calls it at the same point).  A warp splits into
// groups of `lanes_per_group` lanes, takes each group's largest thread maximum and publishes the smallest of
// them: as many different lanes as there are groups have reached it.  The bound is the minimum over the warps
// (greedy: the maximum).  Only the first call waits for every warp's share; later calls read what is there, which
// is valid because a warp's value never decreases.
template <int NT>
__device__ __forceinline__ float block_bound(float tmax, float thr_v, int lanes_per_group, bool wait, bool greedy,
                                          SelectShared & sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float v = tmax;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float other = __shfl_xor_sync(kFull, v, o);
        v = o < lanes_per_group ? fmaxf(v, other) : fminf(v, other);
    }
    if (lane == 0) *(volatile float *) &sh.warp_bound[warp] = v;
    if (wait) __syncthreads();
    const volatile float * wb = sh.warp_bound;
    float b = wb[0];
#pragma unroll
    for (int w = 1; w < NT / 32; ++w) b = greedy ? fmaxf(b, wb[w]) : fminf(b, wb[w]);
    return fmaxf(thr_v, b);  // -inf (a warp that has seen nothing yet) leaves the bound alone
}

// 4-byte asynchronous copy global -> shared (no register is held while the load is in flight).
__device__ __forceinline__ void copy_word_async(uint32_t * dst_shared, const void * src_global) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t) __cvta_generic_to_shared(dst_shared)),
                 "l"(src_global)
                 : "memory");
}
__device__ __forceinline__ void copy_word_wait() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
// The 32-bit word that holds element p[0], and the element's value out of that word.
__device__ __forceinline__ const void * word_of(const float * p) { return p; }
__device__ __forceinline__ const void * word_of(const __nv_bfloat16 * p) {
    return reinterpret_cast<const void *>(reinterpret_cast<uintptr_t>(p) & ~(uintptr_t) 3);
}
__device__ __forceinline__ float value_in_word(uint32_t w, const float *) { return __uint_as_float(w); }
__device__ __forceinline__ float value_in_word(uint32_t w, const __nv_bfloat16 * p) {
    return __uint_as_float((reinterpret_cast<uintptr_t>(p) & 2) ? (w & 0xffff0000u) : (w << 16));
}

// DIRECT: the plan promises at most two groups per slice (slice_len <= 2 * NT * 16): both stay in registers until
// the bound is final and the candidates are taken straight from there (no running bound, no flags, nothing read
// twice).  The slices of a single row are like that.
template <typename T, int VEC, int NT, bool DIRECT>
__global__ void __launch_bounds__(NT, 1024 / NT) k_select(const SelectArgs a) {
    constexpr int NV = kEpochElems / VEC;                    // vectors per thread per group
    constexpr int FPE = NV < 4 ? NV : 4;                     // flag bits per thread and group
    constexpr int VPF = NV / FPE;                            // vectors per flag bit (a "group")
    constexpr int TS = 2 * NT;                               // slots of the occurrence-count table
    constexpr int kTShift = NT == 512 ? 22 : 23;             // 32 - log2(TS)
    constexpr uint32_t kNoKey = 0xffffffffu;
    constexpr int kWarps = NT / 32;
    constexpr uint32_t kVecBits = VEC == 32 ? 0xffffffffu : (1u << VEC) - 1u;
    static_assert(32 * FPE <= 128, "two 64-bit flag words hold the longest slice");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.y, slice = blockIdx.x;
    const int W = a.n_draft + 1, win = row / W, col = row - win * W;
    const int lo = slice * a.slice_len;
    const int n_s = max(0, min(a.vocab, lo + a.slice_len) - lo);
    uint64_t * out = a.cand + ((size_t) row * a.slices + slice) * a.k_cap;

    // shared memory: candidate buffer | selection staging | sorted | p, acc (fp64) | slice bit set |
    // owned history ids: offsets, logit words | mask-to-addend table
    uint64_t * buf = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t * sel = buf + a.cap;
    uint64_t * sorted = sel + a.k_cap;
    double * pj = reinterpret_cast<double *>(sorted + a.k_cap);
    double * acc = pj + a.k_cap;
    uint32_t * eff = reinterpret_cast<uint32_t *>(acc + a.k_cap);
    uint32_t * own = eff + a.slice_len / 32 + 8;  // (8 zero words follow the bit set: the bits of the list's padding)
    uint32_t * oval = own + a.own_cap;
    float4 * lut = reinterpret_cast<float4 *>(oval + a.own_cap);
    uint32_t * vlist = reinterpret_cast<uint32_t *>(lut + 16);  // [list_cap] work list of the second pass: vectors to read again
    uint32_t * tkey = vlist + a.list_cap;                       // [TS] in-slice offsets whose occurrences are counted
    uint32_t * tcnt = tkey + TS;                                // [TS]
    uint32_t * taint = tcnt + TS;                               // [NT] per thread: its largest history logit
    uint16_t * seglist = reinterpret_cast<uint16_t *>(taint + NT);  // [seg_cap] segments with an allowed element
    uint16_t * segpos = seglist + a.seg_cap;                    // [seg_cap] segment -> its place in the list
    SelectShared & sh = *reinterpret_cast<SelectShared *>(segpos + a.seg_cap);

    const T * x = reinterpret_cast<const T *>(a.logits) + (size_t) row * a.row_stride + lo;
    const uint32_t id0 = (uint32_t) (a.id_base + lo);
    // Launched with programmatic stream serialisation: this block may start while the previous kernel of the stream
    // still drains, and the next kernel's blocks may take the places of blocks that have exited (they wait here
    // too).  Nothing is read from global memory before the previous kernel has finished.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const uint32_t * mrow = a.masks ? a.masks + (size_t) (a.mask_rows ? a.mask_rows[row] : row) * a.mask_stride + (lo >> 5) : nullptr;

    // Everything whose address is known is requested before anything is waited for: the row's parameters, its
    // history length, the first history ids and the mask words.
    const int32_t * hrow = a.history ? a.history + (size_t) win * a.history_stride : nullptr;
    const int32_t * drow = a.draft ? a.draft + (size_t) win * a.n_draft : nullptr;
    fns_b200_params p = a.params ? a.params[win] : a.p0;
    int n_hist = (a.history && a.history_len) ? a.history_len[win] : 0;
    int32_t ids0[4] = {-1, -1, -1, -1};
    if (hrow && a.own_cap > 0) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = u * NT + tid;
            if (j < (int) a.history_stride) ids0[u] = hrow[j];
        }
    }

    // 1. The slice's bit set: bit e = element lo + e is allowed.  Bits past the end of the row are 0, so the
    // streaming loop needs no bounds handling.  Every warp also counts its allowed elements; the block adds these
    // up after the barrier, without atomics.
    const int words = (n_s + 31) >> 5;
    if (tid == 0) {
        sh.n_cand = 0u;
        sh.thr_key = 0ull;
        sh.n_own = 0u;
        sh.n_vl = 0u;
        sh.n_seg = 0u;
    }
    for (int i = tid; i < TS; i += NT) {
        tkey[i] = kNoKey;
        tcnt[i] = 0u;
    }
    taint[tid] = 0u;
    if (tid < 8) eff[a.slice_len / 32 + tid] = 0u;
    if (tid < 16) {  // addend per mask nibble: 0 keeps an element, -inf removes it from every maximum
        lut[tid] = make_float4((tid & 1) ? 0.0f : -INFINITY, (tid & 2) ? 0.0f : -INFINITY, (tid & 4) ? 0.0f : -INFINITY,
                               (tid & 8) ? 0.0f : -INFINITY);
    }
    __syncthreads();
    {
        // The bit set, the number of allowed elements, and the list of SEGMENTS that have one.  A segment is what
        // one warp loads with one instruction: 32 consecutive vectors, WPS mask words; here every thread takes
        // whole segments (one 16-byte load of mask words where the row of masks allows it).  Pass 1 walks the
        // list, so excluded stretches of the row cost nothing and every warp gets the same share; an entry also
        // says whether the whole segment is allowed (then nobody looks at the bit set again).
        constexpr int WPS = VEC;  // mask words per segment
        constexpr int SU = 4;     // segments per thread requested together
        const int slice_segs = a.slice_len / (32 * VEC);
        const uint32_t below = (1u << lane) - 1u;
        const uint32_t tail = (n_s & 31) ? (1u << (n_s & 31)) - 1u : 0xffffffffu;
        const bool wide = WPS >= 4 && mrow && (reinterpret_cast<uintptr_t>(mrow) & 15u) == 0;
#pragma unroll 1
        for (int s0 = 0; s0 < slice_segs; s0 += NT * SU) {  // one round for slices up to 2048 * NT / 512 segments
            uint32_t mw[SU][WPS];
#pragma unroll
            for (int u = 0; u < SU; ++u) {  // independent loads, all in flight together
                const int w0 = (s0 + u * NT + tid) * WPS;
                if constexpr (WPS >= 4) {
                    if (wide && w0 + WPS <= words) {
#pragma unroll
                        for (int q = 0; q < WPS; q += 4) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(mrow + w0 + q);
                            mw[u][q] = v.x;
                            mw[u][q + 1] = v.y;
                            mw[u][q + 2] = v.z;
                            mw[u][q + 3] = v.w;
                        }
                        continue;
                    }
                }
#pragma unroll
                for (int q = 0; q < WPS; ++q) mw[u][q] = w0 + q < words ? (mrow ? mrow[w0 + q] : 0xffffffffu) : 0u;
            }
            uint32_t lead[SU], whole[SU];
            int n_mine = 0;
#pragma unroll
            for (int u = 0; u < SU; ++u) {
                const int seg = s0 + u * NT + tid;
                uint32_t any = 0u, all = 0xffffffffu;
                if (seg < slice_segs) {
#pragma unroll
                    for (int q = 0; q < WPS; ++q) {
                        if (seg * WPS + q == words - 1) mw[u][q] &= tail;
                        any |= mw[u][q];
                        all &= mw[u][q];
                        eff[seg * WPS + q] = mw[u][q];
                    }
                }
                lead[u] = __ballot_sync(kFull, any != 0u);
                whole[u] = __ballot_sync(kFull, any != 0u && all == 0xffffffffu);
                n_mine += __popc(lead[u]);
            }
            uint32_t at = 0u;
            if (lane == 0 && n_mine) at = atomicAdd(&sh.n_seg, (uint32_t) n_mine);
            at = __shfl_sync(kFull, at, 0);
#pragma unroll
            for (int u = 0; u < SU; ++u) {
                if ((lead[u] >> lane) & 1u) {
                    const uint32_t seg = (uint32_t) (s0 + u * NT + tid);
                    const uint32_t pos = at + (uint32_t) __popc(lead[u] & below);
                    seglist[pos] = (uint16_t) (seg | (((whole[u] >> lane) & 1u) << 15));
                    segpos[seg] = (uint16_t) pos;
                }
                at += (uint32_t) __popc(lead[u]);
            }
        }
    }
    const int k = p.temperature <= 0.0f ? 1 : clamp_k(p.top_k, a.k_cap);
    const bool any_pen = p.repetition != 1.0f || p.presence != 0.0f || p.frequency != 0.0f;
    const bool use_hist = any_pen && a.own_cap > 0 && n_s > 0;
    n_hist = n_hist < 0 ? 0 : (n_hist > (int) a.history_stride ? (int) a.history_stride : n_hist);
    const int n_pen = n_hist + (a.draft ? col : 0);
    uint64_t best = 0ull;      // k == 1: this thread's best key
    __syncthreads();
    const int n_seg = (int) sh.n_seg;
    const int n_groups = (n_seg + kWarps * NV - 1) / (kWarps * NV);  // a group: NV consecutive list entries per warp
    // the last group is filled up with a segment behind the slice, whose bits (the zero words after the bit set)
    // exclude everything: no loop below has to ask where the list ends
    for (int i = n_seg + tid; i < n_groups * kWarps * NV; i += NT) seglist[i] = (uint16_t) (a.slice_len / (32 * VEC));

    // 2. Penalties.  Every history id (plus the draft prefix of a verification column) that lies in the slice
    // clears its bit in the bit set, so the streaming pass never sees it and pays nothing for penalties.  The
    // thread that finds the bit still set owns the id: ids that the mask excludes have no owner, and of several
    // occurrences of one id exactly one thread wins.  Owners append the id to a list (one reservation per warp
    // and round) and start an asynchronous copy of its logit into shared memory; its penalised value is offered
    // as a candidate after pass 1, when a bound exists that most of them fail.  The occurrence count (frequency
    // penalty) is looked up only for the few that could pass the bound.  Traffic: 4 bytes per history id (every
    // slice reads the list; it stays in L2).
    int n_own = 0;
    uint32_t t_base = 0u, t_pre = 0u, t_mine = 0u;  // this thread's list slots of the first round
    // A history logit may become its thread's maximum in a group that is streamed without the bit set.  Such a
    // maximum must not count as a witness for the bound, so every owner records the logit in taint[] of the thread
    // that streams the element: a thread whose maximum does not exceed its taint is left out of the bound.
    auto publish_taint = [&](uint32_t slot) {
        const uint32_t off = own[slot];
        const float raw = value_in_word(oval[slot], x + off);
        const uint32_t vec = off / VEC;  // streamed by lane vec % 32 of the warp that the segment's list place gives
        if (is_finite(raw)) atomicMax(&taint[((segpos[vec >> 5] / NV) % kWarps) * 32 + (vec & 31u)], order_word(raw));
    };
    if (use_hist && n_pen > 0) {
        const uint32_t below = (1u << lane) - 1u;
        for (int j0 = 0; j0 < n_pen; j0 += NT * 4) {
            int32_t ids[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {  // four independent loads in flight
                const int j = j0 + u * NT + tid;
                if (j0 == 0 && hrow) ids[u] = j < n_hist ? ids0[u] : (j < n_pen ? drow[j - n_hist] : -1);
                else ids[u] = j < n_hist ? hrow[j] : (j < n_pen ? drow[j - n_hist] : -1);
            }
            uint32_t offs[4], pre[4], total = 0u;
            bool mine[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                offs[u] = (uint32_t) (ids[u] - a.id_base - lo);
                mine[u] = false;
                if (offs[u] < (uint32_t) n_s && ids[u] >= a.id_base) {
                    const uint32_t bit = 1u << (offs[u] & 31);
                    // (the plain read first: excluded ids and repeats, the common case under a mask, cost no atomic)
                    if (eff[offs[u] >> 5] & bit) mine[u] = (atomicAnd(&eff[offs[u] >> 5], ~bit) & bit) != 0u;  // (a stale 1 is settled by the atomic)
                }
                const uint32_t b = __ballot_sync(kFull, mine[u]);
                pre[u] = total + (uint32_t) __popc(b & below);
                total += (uint32_t) __popc(b);
            }
            if (total == 0u) continue;  // uniform per warp
            uint32_t base = 0u;
            if (lane == 0) base = atomicAdd(&sh.n_own, total);
            base = __shfl_sync(kFull, base, 0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (!mine[u]) continue;
                own[base + pre[u]] = offs[u];
                copy_word_async(&oval[base + pre[u]], word_of(x + offs[u]));
            }
            if (j0 == 0) {
                t_base = base;
                t_pre = pre[0] | (pre[1] << 8) | (pre[2] << 16) | (pre[3] << 24);  // each < 128
                t_mine = (mine[0] ? 1u : 0u) | (mine[1] ? 2u : 0u) | (mine[2] ? 4u : 0u) | (mine[3] ? 8u : 0u);
            } else {  // a long history: no point in hiding this latency
                copy_word_wait();
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (mine[u]) publish_taint(base + pre[u]);
            }
        }
    }
    __syncthreads();
    if (use_hist) n_own = (int) sh.n_own;
    // The row's ragged end: the elements of a last, partial vector are taken out of the bit set here, so that the
    // vector loads below never reach past the row; each becomes a key that is offered with the other candidates.
    uint64_t rag_key = 0ull;
    if (VEC > 1 && (n_s % VEC) != 0) {
        if (tid < (n_s % VEC)) {
            const int e = n_s - (n_s % VEC) + tid;
            const uint32_t bit = 1u << (e & 31);
            if (atomicAnd(&eff[e >> 5], ~bit) & bit) {
                const float xi = to_float(x[e]);
                if (is_finite(xi)) rag_key = make_key(xi, id0 + (uint32_t) e);
            }
        }
        __syncthreads();
    }

    // 3. Pass 1 over the listed segments: maxima only.  A group gives every warp NV segments, that is every thread
    // NV vectors (16 elements); two groups are in flight (the loads of the next one are issued before the current
    // one is reduced).  In a segment that is allowed as a whole nobody looks at the bit set; elsewhere a vector
    // whose elements the bit set excludes is not loaded, and excluded elements of a loaded vector get -inf added (a
    // table lookup by the vector's mask nibble), so the maxima need no branches.  Every thread keeps the maximum
    // of what it has seen; a vector group whose maximum reaches the running bound sets a flag bit and is read
    // again in pass 2.  The bound needs no buffer: if r lanes of EVERY warp hold a maximum >= v (r * warps >= k),
    // the slice has at least k elements >= v, so nothing below v can be among its best k.  A warp splits into r
    // groups of lanes (r a power of two), takes each group's maximum and publishes the smallest of them: r
    // different lanes have reached it.  The bound is the minimum over the warps (for k = 1: the maximum).  It is
    // made after the first group, refreshed after the second and the fourth, and tightened at the end (flags are
    // cheap: only the few threads that hold a candidate ever look at theirs; under a mask that leaves some lanes
    // without an element for long there is simply no running bound, and everything is flagged).
    const int r_need = (k + kWarps - 1) / kWarps;  // lanes per warp that must hold a value above the bound
    const bool bounded = r_need <= 32;             // otherwise every group is flagged
    int lanes_per_group = 32;                      // 32 / (r_need rounded up to a power of two)
    while (lanes_per_group > 1 && (32 / lanes_per_group) < r_need) lanes_per_group >>= 1;
    float tmax = -INFINITY;                        // this thread's maximum so far
    float thr_v = -FLT_MAX;                        // the bound: x < thr_v cannot be a candidate
    uint64_t f0 = 0ull, f1 = 0ull;                 // flag bit g * FPE + j: vector group j of list group g reached the bound
    int done = 0;
    uint32_t taint_w = 0u;  // this thread's taint, read when the first bound is made
    int next_refresh = 0;   // the bound is refreshed after this many groups (the same in all lanes of a warp)
    auto clean_max = [&]() -> float { return (tmax > -INFINITY && order_word(tmax) > taint_w) ? tmax : -INFINITY; };
    // This warp's NV list entries of group g (consecutive places: consecutive segments, one read).
    const uint16_t * my_entries = seglist + warp * NV;
    auto entries_of = [&](int g, uint32_t (&en)[NV]) {
        const uint16_t * at = my_entries + g * (kWarps * NV);
        if constexpr (NV == 4) {
            const uint2 v = *reinterpret_cast<const uint2 *>(at);
            en[0] = v.x & 0xffffu;
            en[1] = v.x >> 16;
            en[2] = v.y & 0xffffu;
            en[3] = v.y >> 16;
        } else if constexpr (NV == 2) {
            const uint32_t v = *reinterpret_cast<const uint32_t *>(at);
            en[0] = v & 0xffffu;
            en[1] = v >> 16;
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i) en[i] = at[i];
        }
    };
    const T * x_lane = x + lane * VEC;                           // this lane's vector of segment 0
    const uint32_t * eff_lane = eff + ((lane * VEC) >> 5);       // the word with its bits, and where they start
    const int eff_shift = (lane * VEC) & 31;
    auto vector_bits = [&](uint32_t seg) -> uint32_t { return (eff_lane[seg * VEC] >> eff_shift) & kVecBits; };
    auto vector_at = [&](uint32_t seg) -> const T * { return x_lane + seg * (32u * VEC); };
    // Requests the NV vectors of group g.  Returns whether all of them lie in segments that are allowed as a whole
    // (the same answer in every lane of the warp): then mb is not even written.
    auto issue = [&](int g, float (&xv)[NV][VEC], uint32_t (&mb)[NV]) -> bool {
        uint32_t en[NV];
        entries_of(g, en);
        uint32_t all = 0x8000u;
#pragma unroll
        for (int i = 0; i < NV; ++i) all &= en[i];
        if (all) {
#pragma unroll
            for (int i = 0; i < NV; ++i) load_vec<T, VEC>(vector_at(en[i] & 0x7fffu), xv[i]);
            return true;
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const uint32_t seg = en[i] & 0x7fffu;
            mb[i] = (en[i] & 0x8000u) ? kVecBits : vector_bits(seg);
            if (mb[i]) load_vec<T, VEC>(vector_at(seg), xv[i]);
        }
        return false;
    };
    // The maxima of the NV vectors of a group (vmx) and of the whole group (returned; +inf if an allowed element is).
    auto group_max = [&](float (&xv)[NV][VEC], uint32_t (&mb)[NV], bool plain, float (&vmx)[NV]) -> float {
        float emax = -INFINITY;
        if (plain) {  // every element counts (history ids too: see taint)
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                float m = xv[i][0];
#pragma unroll
                for (int j = 1; j < VEC; ++j) m = fmaxf(m, xv[i][j]);
                vmx[i] = m;
                emax = fmaxf(emax, m);
            }
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                float m = -INFINITY;
                if constexpr (VEC == 1) {
                    m = mb[i] ? xv[i][0] : -INFINITY;
                } else {
                    // a vector that was not loaded holds stale values: stale - inf is -inf or NaN, and NaN never wins
#pragma unroll
                    for (int q = 0; q < VEC / 4; ++q) {
                        const float4 t = lut[(mb[i] >> (4 * q)) & 15u];
                        m = fmaxf(m, fmaxf(fmaxf(xv[i][4 * q] + t.x, xv[i][4 * q + 1] + t.y),
                                           fmaxf(xv[i][4 * q + 2] + t.z, xv[i][4 * q + 3] + t.w)));
                    }
                }
                vmx[i] = m;
                emax = fmaxf(emax, m);
            }
        }
        return emax;
    };
    auto reduce = [&](int ep, float (&xv)[NV][VEC], uint32_t (&mb)[NV], bool plain) {
        float vmx[NV];
        float emax = group_max(xv, mb, plain, vmx);
        constexpr int EPW = 64 / FPE;  // groups per flag word
        if (__builtin_expect(!(emax <= FLT_MAX), 0)) {
            // +inf among the allowed elements: never a candidate (src/kernels.cu:629-639).  The group is left to
            // pass 2, which looks at every element, and adds nothing to this thread's maximum.
            const uint64_t every = (1ull << FPE) - 1ull;
            if (ep < EPW) f0 |= every << (ep * FPE);
            else f1 |= every << ((ep - EPW) * FPE);
            emax = -INFINITY;
        }
        tmax = fmaxf(tmax, emax);
        if (__builtin_expect(bounded && done == next_refresh, 0))
        {
            if (done == 0 && n_own > 0) {  // uniform: the owners have published their taint before their first reduce
                __syncthreads();
                taint_w = taint[tid];
            }
            thr_v = block_bound<NT>(clean_max(), thr_v, lanes_per_group, done == 0, k == 1, sh);
            next_refresh = done == 0 ? 1 : (done == 1 ? 3 : -1);  // after groups 1, 2 and 4, then not before the end
        }
        ++done;
        if (__builtin_expect(emax >= thr_v, 0)) {
            uint64_t hb = 0ull;  // the vector groups of this group that reach the bound
#pragma unroll
            for (int g = 0; g < FPE; ++g) {
                bool q = false;
#pragma unroll
                for (int u = 0; u < VPF; ++u) q = q || vmx[g * VPF + u] >= thr_v;
                hb |= (q ? 1ull : 0ull) << g;
            }
            if (ep < EPW) f0 |= hb << (ep * FPE);
            else f1 |= hb << ((ep - EPW) * FPE);
        }
    };
    // The final bound (every thread of the block calls it at the same point).  After the lane-group bound it is
    // tightened to (nearly) the k-th largest of the threads' maxima: k threads that have reached a value are k
    // elements that have, and a count over the block is one barrier.  The search runs bit by bit below the highest
    // bit in which the bound so far and the block's maximum differ.
    auto tighten = [&](float cmax) {
        copy_word_wait();  // this thread's logit copies have landed; the barriers below show them to the others
        const uint32_t wt = cmax > -INFINITY ? order_word(cmax) : 0u;  // this thread's witness as an order word
        if (bounded && done > 0) {
            const uint32_t top = __reduce_max_sync(kFull, wt);
            if (lane == 0) sh.warp_top[warp] = top;
            thr_v = block_bound<NT>(cmax, thr_v, lanes_per_group, true, k == 1, sh);  // (its barrier also covers warp_top)
            if (k > 1 && k <= NT) {
                uint32_t hi_w = sh.warp_top[0];
#pragma unroll
                for (int w = 1; w < kWarps; ++w) hi_w = max(hi_w, sh.warp_top[w]);
                const uint32_t lo_w = order_word(thr_v);
                if (hi_w > lo_w) {
                    const int split = 31 - __clz((int) (lo_w ^ hi_w));
                    uint32_t bw = split == 31 ? 0u : (lo_w & ~((2u << split) - 1u));  // the common prefix: <= lo_w, so valid
                    const int stop = split > 10 ? split - 10 : 0;
#pragma unroll 1
                    for (int bit = split; bit >= stop; --bit) {
                        const uint32_t cand = bw | (1u << bit);
                        if (__syncthreads_count(wt >= cand) >= k) bw = cand;
                    }
                    if (bw > lo_w) thr_v = word_value(bw);
                }
            }
        } else {
            __syncthreads();
        }
        thr_v += 0.0f;  // -0.0 -> +0.0: one key pattern for both zeros
    };
    float xa[NV][VEC], xb[NV][VEC];  // the two groups in flight
    uint32_t ma[NV], mb[NV];
    bool pa = false, pb = false;
    if constexpr (DIRECT) {
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int j = 0; j < VEC; ++j) xa[i][j] = xb[i][j] = 0.0f;
        if (n_groups > 0) pa = issue(0, xa, ma);
        if (n_groups > 1) pb = issue(1, xb, mb);
        if (t_mine) {
            copy_word_wait();
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if ((t_mine >> u) & 1u) publish_taint(t_base + ((t_pre >> (8 * u)) & 255u));
        }
        if (n_own > 0) {  // uniform
            __syncthreads();
            taint_w = taint[tid];
        }
        auto take_max = [&](int g, float (&xv)[NV][VEC], uint32_t (&mv)[NV], bool plain) {
            float vmx[NV];
            float emax = group_max(xv, mv, plain, vmx);
            if (!(emax <= FLT_MAX)) {  // +inf among the allowed elements: the largest finite one, the slow way
                emax = -INFINITY;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const uint32_t bits = vector_bits(my_entries[g * (kWarps * NV) + i] & 0x7fffu);
                    if (bits) emax = fmaxf(emax, vector_max<VEC>(xv[i], bits));
                }
            }
            tmax = fmaxf(tmax, emax);
        };
        if (n_groups > 0) take_max(0, xa, ma, pa);
        if (n_groups > 1) take_max(1, xb, mb, pb);
        done = n_groups;
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
            for (int j = 0; j < VEC; ++j) xa[i][j] = xb[i][j] = 0.0f;
        if (n_groups > 0) pa = issue(0, xa, ma);
#pragma unroll 1
        for (int g = 0; g < n_groups; g += 2) {
            if (g + 1 < n_groups) pb = issue(g + 1, xb, mb);
            if (g == 0 && t_mine) {  // with two groups requested: the history logits of this thread's ids, for the taint
                copy_word_wait();
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if ((t_mine >> u) & 1u) publish_taint(t_base + ((t_pre >> (8 * u)) & 255u));
            }
            reduce(g, xa, ma, pa);
            if (g + 1 >= n_groups) break;
            if (g + 2 < n_groups) pa = issue(g + 2, xa, ma);
            reduce(g + 1, xb, mb, pb);
        }
    }
    tighten(clean_max());
    if (!(tmax >= thr_v)) f0 = f1 = 0ull;  // nothing of this thread can be a candidate: its flags are void

    // 4. The candidates.  Three sources are compared with the final bound and what passes is appended to the
    // buffer: the ragged end, the penalised history ids, and the flagged groups of pass 1 (read again).  With the
    // tightened bound little more than k keys arrive, so the first attempt does not watch the buffer at all: an
    // append that finds it full is dropped, and the cursor running past the end afterwards says so.  Only then
    // (many equal values, k near the buffer size) is everything offered again the careful way: every group
    // flagged, the block voting after every round on whether to compact (which also raises the bar) and
    // repeating the appends that failed.
    uint64_t thr_key = (uint64_t) order_word(thr_v) << 32;
    auto penalised = [&](float v, float cnt) -> float {  // each step rounded on its own: no fused multiply-add
        v = v > 0.0f ? __fdiv_rn(v, p.repetition) : __fmul_rn(v, p.repetition);
        v = __fsub_rn(v, __fmul_rn(p.frequency, cnt));
        return __fsub_rn(v, p.presence);
    };
    auto pop_flag = [&]() -> int {
        if (f0) {
            const int b = __ffsll((long long) f0) - 1;
            f0 &= f0 - 1ull;
            return b;
        }
        if (f1) {
            const int b = __ffsll((long long) f1) - 1;
            f1 &= f1 - 1ull;
            return 64 + b;
        }
        return -1;
    };
    for (int attempt = 0; attempt < 2; ++attempt) {
        const bool careful = attempt == 1;
        // (a) the ragged end
        if (rag_key != 0ull) {
            if (k == 1) best = rag_key > best ? rag_key : best;
            else if (rag_key >= thr_key) push(rag_key, buf, sh, a.cap);  // at most VEC - 1 keys, first in the buffer
        }
        // (b) Every owned history id with its penalised value (the bound came from the other elements alone, which
        // can only make it lower than the true k-th best: still a valid bar).  One list entry per thread and round.
        // The value with ONE occurrence is computed first; with a frequency penalty >= 0 more occurrences can only
        // lower it, so an id's occurrences are counted only if that value reaches the bound: such ids enter a
        // small hash table, the block walks the history once and counts the hits, and the owners read their counts
        // back (and empty their slots for the next round).
        if (n_own > 0) {
            const bool counts = p.frequency != 0.0f;
            const bool count_all = p.frequency < 0.0f;  // then more occurrences raise the value
            for (int j0 = 0; j0 < n_own; j0 += NT) {
                const int j = j0 + tid;
                uint32_t off = 0u;
                float raw = 0.0f, v = -INFINITY;
                bool live = j < n_own;
                if (live) {
                    off = own[j];
                    raw = value_in_word(oval[j], x + off);
                    v = penalised(raw, 1.0f);
                    live = count_all || v >= thr_v;
                }
                if (counts && __syncthreads_or(live)) {
                    uint32_t slot = 0u;
                    if (live) {  // owned ids are distinct: every insert claims an empty slot
                        slot = (off * 2654435761u) >> kTShift;
                        while (atomicCAS(&tkey[slot], kNoKey, off) != kNoKey) slot = (slot + 1u) & (TS - 1);
                    }
                    __syncthreads();
                    for (int t = tid; t < n_pen; t += NT) {
                        const int32_t id = t < n_hist ? hrow[t] : drow[t - n_hist];
                        const uint32_t o = (uint32_t) (id - a.id_base - lo);
                        if (o >= (uint32_t) n_s || id < a.id_base) continue;
                        uint32_t h = (o * 2654435761u) >> kTShift;
                        for (uint32_t kx = tkey[h]; kx != kNoKey; kx = tkey[h]) {  // at most NT keys in 2 * NT slots
                            if (kx == o) {
                                atomicAdd(&tcnt[h], 1u);
                                break;
                            }
                            h = (h + 1u) & (TS - 1);
                        }
                    }
                    __syncthreads();
                    if (live) {
                        v = penalised(raw, (float) tcnt[slot]);
                        tkey[slot] = kNoKey;
                        tcnt[slot] = 0u;
                    }
                }
                uint64_t key = 0ull;
                if (live && is_finite(v)) key = make_key(v, id0 + off);
                bool full = false;
                if (key != 0ull) {
                    if (k == 1) best = key > best ? key : best;
                    else if (key >= thr_key) full = !push(key, buf, sh, a.cap);
                }
                if (careful && k > 1 && n_own + VEC > a.trigger) {  // uniform: only a long list can fill the buffer
                    while (__syncthreads_or(full || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                        compact<NT>(buf, sel, k, a.cap, sh);
                        const uint64_t tk = sh.thr_key;
                        if (tk > thr_key) { thr_key = tk; thr_v = key_floor_value(tk); }
                        if (full && (key < thr_key || push(key, buf, sh, a.cap))) full = false;
                        if (!__syncthreads_or(full)) break;
                    }
                }
            }
        }
        // (c) The flagged groups.  Their vectors go on a work list that the whole block then shares: one vector per
        // thread and round, read again (from L1 / L2, or HBM when a large batch has pushed the row out).  The
        // careful way walks every group instead, one per round, with a vote after each.
        bool listed = true;
        if (DIRECT && !careful) {
            if constexpr (DIRECT) {
            auto offer_group = [&](int g, float (&xv)[NV][VEC]) {
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        const uint32_t seg = my_entries[g * (kWarps * NV) + i] & 0x7fffu;
                        const uint32_t bits = vector_bits(seg);  // (the bit set: history ids are out, also in a whole segment)
                        if (!bits) continue;
                        const uint32_t e = ((seg << 5) + (uint32_t) lane) * VEC;
#pragma unroll
                        for (int j = 0; j < VEC; ++j) {
                            if (!(((bits >> j) & 1u) && xv[i][j] >= thr_v && xv[i][j] <= FLT_MAX)) continue;
                            const uint64_t key = make_key(xv[i][j], id0 + e + (uint32_t) j);
                            if (k == 1) best = key > best ? key : best;
                            else if (key >= thr_key) push(key, buf, sh, a.cap);
                        }
                    }
                };
                if (n_groups > 0) offer_group(0, xa);
                if (n_groups > 1) offer_group(1, xb);
            }
        } else if (!careful) {
            // one reservation per warp: a prefix sum over the lanes' flag counts
            const int mine_n = (__popcll(f0) + __popcll(f1)) * VPF;
            int upto = mine_n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(kFull, upto, o);
                if (lane >= o) upto += t;
            }
            const int warp_n = __shfl_sync(kFull, upto, 31);
            uint32_t at = 0u;
            if (lane == 31 && warp_n) at = atomicAdd(&sh.n_vl, (uint32_t) warp_n);
            at = __shfl_sync(kFull, at, 31) + (uint32_t) (upto - mine_n);
            while ((f0 | f1) != 0ull) {
                const int b = pop_flag();
                const int ep = b / FPE, g = b - ep * FPE;
#pragma unroll
                for (int u = 0; u < VPF; ++u) {
                    const uint32_t seg = my_entries[ep * (kWarps * NV) + g * VPF + u] & 0x7fffu;
                    if (at < (uint32_t) a.list_cap) vlist[at] = (seg << 5) + (uint32_t) lane;
                    ++at;
                }
            }
            __syncthreads();
            const int n_work = (int) sh.n_vl;
            listed = n_work <= a.list_cap;  // uniform; a list that does not fit sends the slice the careful way
#pragma unroll 1
            for (int i = tid; i < n_work && listed; i += NT) {
                const int e = (int) vlist[i] * VEC;
                const uint32_t bits = (eff[e >> 5] >> (e & 31)) & kVecBits;
                if (!bits) continue;
                float xv[VEC];
                load_vec<T, VEC>(x + e, xv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    if (!(((bits >> j) & 1u) && xv[j] >= thr_v && xv[j] <= FLT_MAX)) continue;
                    const uint64_t key = make_key(xv[j], id0 + (uint32_t) (e + j));
                    if (k == 1) best = key > best ? key : best;
                    else if (key >= thr_key) push(key, buf, sh, a.cap);
                }
            }
        } else {
#pragma unroll 1
            for (int g = 0; g < n_groups; ++g) {
                uint32_t bits[NV], lost = 0u;  // lost: elements of this round that found the buffer full
                int e0[NV];                    // first element of each vector of this round
                float xv[NV][VEC];
                uint32_t en[NV];
                entries_of(g, en);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const uint32_t seg = en[i] & 0x7fffu;
                    e0[i] = (int) (((seg << 5) + (uint32_t) lane) * VEC);
                    bits[i] = vector_bits(seg);
                    if (bits[i]) load_vec<T, VEC>(x + e0[i], xv[i]);
                }
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (!bits[i]) continue;
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        if (!(((bits[i] >> j) & 1u) && xv[i][j] >= thr_v && xv[i][j] <= FLT_MAX)) continue;
                        const uint64_t key = make_key(xv[i][j], id0 + (uint32_t) (e0[i] + j));
                        if (k == 1) best = key > best ? key : best;
                        else if (key >= thr_key && !push(key, buf, sh, a.cap)) lost |= 1u << (i * VEC + j);
                    }
                }
                if (k == 1) continue;  // greedy: nothing is buffered, so nothing can overflow
                while (__syncthreads_or(lost != 0u || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                    compact<NT>(buf, sel, k, a.cap, sh);
                    const uint64_t tk = sh.thr_key;
                    if (tk > thr_key) { thr_key = tk; thr_v = key_floor_value(tk); }
                    uint32_t still = 0u;
                    for (uint32_t q = lost; q; q &= q - 1u) {
                        const int b = __ffs(q) - 1;
                        int e = b % VEC;
#pragma unroll
                        for (int i = 0; i < NV; ++i)
                            if (i == b / VEC) e += e0[i];
                        const uint64_t key = make_key(to_float(x[e]), id0 + (uint32_t) e);
                        if (key >= thr_key && !push(key, buf, sh, a.cap)) still |= 1u << b;
                    }
                    lost = still;
                    if (!__syncthreads_or(lost != 0u)) break;
                }
            }
        }
        __syncthreads();
        if (attempt == 1 || (listed && (k == 1 || sh.n_cand <= (uint32_t) a.cap))) break;  // uniform: all is in
        // The buffer or the work list overflowed: start again from an empty buffer, the careful way.
        __syncthreads();
        if (tid == 0) sh.n_cand = 0u;
        best = 0ull;
        __syncthreads();
    }
    __syncthreads();

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
            draw_tail<NT>(sorted, got, pj, acc, reinterpret_cast<double *>(sel), sh.sc, p, a.k_cap, tok, oc);
            return;
        }
    }

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
        return;
    }
    // the slices' lists, each sorted, side by side in the buffer: [slices][k]
    for (int i = tid; i < a.slices * k; i += NT) {
        const int l = i / k, j = i - l * k;
        buf[i] = __ldcg(lists + (size_t) l * a.k_cap + j);
    }
    __syncthreads();
    const int nk = merge_lists<NT>(buf, a.slices, k, sel, sorted, reinterpret_cast<uint64_t *>(pj), 2 * a.k_cap, sh.sc, k, a.k_cap);
    draw_tail<NT>(sorted, nk, pj, acc, reinterpret_cast<double *>(sel), sh.sc, p, a.k_cap, tok, oc);
}

}  // namespace fnsb

#include "fns_ring.cuh"
#include "fns_cluster.cuh"

namespace fnsb {

// ---- finalize as a kernel of its own -------------------------------------------------------------------------
constexpr int kFinalThreads = 512;

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
    // many short lists: witnesses and counting; a few long ones (vocabulary shards): merged pairwise, every key
    // finding its place in the sibling list by a binary search, a merged list keeping its best k
    int nk;
    if (a.list_len > 64 && a.lists <= 8 && k <= a.list_len) {  // (then a merged run is never longer than list_len: the halves fit)
        // A few long sorted lists (vocabulary shards).  First a bound: with q = ceil(k / lists), at least k keys reach
        // the smallest of the lists' q-th keys, so nothing below it can be among the best k - for shards of a
        // shuffled vocabulary that leaves a fraction of the keys.
        uint32_t * n_of = &sh.sc.hist[0];  // [lists] keys of a list that reach the bound; [8]: their sum
        const int L = a.lists, len = a.list_len;
        if (tid == 0) {
            const int q = (k + L - 1) / L;
            uint64_t m = ~0ull;
            for (int l = 0; l < L; ++l) {
                const uint64_t key = q - 1 < len ? buf[(size_t) l * len + q - 1] : 0ull;
                m = key < m ? key : m;
            }
            *reinterpret_cast<uint64_t *>(&sh.sc.hist[10]) = m;  // (0: a list is shorter than q keys - no bound)
        }
        for (int j = tid; j < a.k_cap; j += kFinalThreads) sorted[j] = 0ull;
        __syncthreads();
        const uint64_t m = *reinterpret_cast<const uint64_t *>(&sh.sc.hist[10]);
        if (tid < L) {  // the keys of list tid that reach the bound (empty slots are 0 and sort last)
            const uint64_t * lst = buf + (size_t) tid * len;
            const uint64_t floor_key = m > 1ull ? m : 1ull;
            int lo = 0, hi = len;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (lst[mid] >= floor_key) lo = mid + 1;
                else hi = mid;
            }
            n_of[tid] = (uint32_t) lo;
        }
        __syncthreads();
        // Then the lists' heads are merged pairwise, level by level; a merged run keeps its best k; every thread
        // produces four consecutive keys of a merged run at a time (merge_chunk).  Run descriptors (start, length,
        // first chunk) live in shared memory, two sets that take turns.
        uint32_t * desc = &sh.sc.hist[16];  // [2][3][8]: per set the runs' start | length | index of the first chunk
        uint64_t * spare = reinterpret_cast<uint64_t *>(&sh + 1);  // [(lists + 1) / 2 * list_len + k_cap]
        if (tid == 0) {
            uint32_t all = 0u;
            for (int l = 0; l < 8; ++l) {
                desc[l] = (uint32_t) (l * len);
                desc[8 + l] = l < L ? n_of[l] : 0u;
                all += desc[8 + l];
            }
            sh.sc.count = all;
        }
        __syncthreads();
        const int total = (int) sh.sc.count;
        uint64_t * src = buf, * dst = spare;
        int runs = L, set = 0;
#pragma unroll 1
        while (runs > 1) {
            const uint32_t * st = desc + set * 24, * nn = st + 8;
            uint32_t * ost = desc + (set ^ 1) * 24, * onn = ost + 8, * ofirst = ost + 16;
            const int out_runs = (runs + 1) >> 1;
            if (tid == 0) {  // the merged runs: side by side at a distance of k
                uint32_t chunks = 0u;
                for (int r = 0; r < 8; ++r) {
                    const uint32_t both = r < out_runs ? nn[2 * r] + (2 * r + 1 < runs ? nn[2 * r + 1] : 0u) : 0u;
                    ost[r] = (uint32_t) (r * k);
                    onn[r] = both < (uint32_t) k ? both : (uint32_t) k;
                    ofirst[r] = chunks;
                    chunks += (onn[r] + 3u) >> 2;
                }
                sh.sc.bucket = chunks;
            }
            __syncthreads();
            const int chunks = (int) sh.sc.bucket;
#pragma unroll 1
            for (int c = tid; c < chunks; c += kFinalThreads) {
                int r = 0;
#pragma unroll
                for (int t = 1; t < 4; ++t) r += t < out_runs && (uint32_t) c >= ofirst[t] ? 1 : 0;
                const int d0 = (c - (int) ofirst[r]) << 2;
                const bool pair = 2 * r + 1 < runs;
                merge_chunk<4>(src + st[2 * r], (int) nn[2 * r], src + (pair ? st[2 * r + 1] : 0u), pair ? (int) nn[2 * r + 1] : 0, d0,
                               (int) onn[r], dst + ost[r]);
            }
            __syncthreads();
            uint64_t * t = src;
            src = dst;
            dst = t;
            runs = out_runs;
            set ^= 1;
        }
        {
            const uint32_t * st = desc + set * 24, * nn = st + 8;
            const int have = (int) nn[0];
            for (int j = tid; j < have && j < k; j += kFinalThreads) sorted[j] = src[st[0] + j];
        }
        __syncthreads();
        nk = total < k ? total : k;
    } else if (a.list_len > 64 && k <= a.list_len) {  // (then a merged list is never longer than list_len: the halves fit)
        uint64_t * spare = reinterpret_cast<uint64_t *>(&sh + 1);  // [lists * list_len / 2 + k]
        int len = 0;
        const uint64_t * res = merge_runs<kFinalThreads>(buf, spare, a.lists, a.list_len, k, &len);
        if (tid == 0) sh.sc.count = 0u;
        __syncthreads();
        const int take = len < k ? len : k;
        for (int j = tid; j < a.k_cap; j += kFinalThreads) {
            const uint64_t key = j < take ? res[j] : 0ull;
            sorted[j] = key;
            if (key != 0ull && (j + 1 == take || res[j + 1] == 0ull)) sh.sc.count = (uint32_t) j + 1u;  // the last candidate
        }
        __syncthreads();
        nk = (int) sh.sc.count;
    } else {
        nk = merge_lists<kFinalThreads>(buf, a.lists, a.list_len, sel, sorted, reinterpret_cast<uint64_t *>(pj), 2 * a.k_cap,
                                        sh.sc, k, a.k_cap);
    }
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
    bool logits_in_host_memory;  // the next call's logits are page-locked host memory (set by the engine glue)
    bool cluster_ok;             // a cluster of 16 CTAs of k_cluster can be resident on this device
    int cluster_rows;            // calls of up to this many rows take k_cluster: as many clusters as the device holds at once
    int cluster_rows_unmasked;   // ... and without a mask up to twice that (two waves of clusters still beat k_ring)
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
    int threads, slices, slice_len, cap, trigger, own_cap, vec, list_cap, seg_cap;
    size_t smem_select;
    bool cluster; // k_cluster (small batches)
    bool ring;    // k_ring instead of k_select
    int n_stages, ring_depth, ring_off, own_off, hist_cap;
};

int round_up(int x, int m) { return (x + m - 1) / m * m; }

int fail(fns_b200_sampler * s, int code, const char * what) {
    if (s) std::snprintf(s->msg, sizeof s->msg, "%s", what);
    return code;
}
int fail_cuda(fns_b200_sampler * s, cudaError_t e, const char * where) {
    if (s) std::snprintf(s->msg, sizeof s->msg, "%s: %s", where, cudaGetErrorString(e));
    return FNS_B200_ERR_CUDA;
}

// Launch geometry.  A block has 512 threads (two fit an SM).  From five rows on a row is one slice: setup, history
// and draw are paid once per row and there is nothing to merge; this measured faster than any cut at every batch
// size from 5 to 1024 rows.  Up to four rows are cut into slices of one group per thread (8,192 elements), so that
// many SMs share the row, and the last block to finish merges the slices' lists.  A slice is a whole number of
// threads * 16 elements and at most 16 (256 threads) or 32 (512 threads) of them; the slices' lists of one row must
// fit the merge (kMaxMergeKeys).
bool make_plan_for(const fns_b200_sampler * s, int dtype, int vocab, int rows, int hist_bound, bool aligned, bool whole_rows,
                   Plan & pl) {
    const int k_cap = s->k_cap;
    pl.threads = s->force_threads > 0 ? s->force_threads : (s->force_slices > 0 ? 256 : 512);
    const int epoch = pl.threads * kEpochElems;
    const int max_slice_len = (pl.threads == 256 ? 16 : 32) * epoch;
    const int min_slices = (vocab + max_slice_len - 1) / max_slice_len;
    int max_slices = kMaxMergeKeys / k_cap;
    if (max_slices > kMaxSlices) max_slices = kMaxSlices;
    if (min_slices > max_slices) return false;
    int want;
    if (s->force_slices > 0) want = s->force_slices;
    else if (whole_rows) want = 1;
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
    pl.cap = round_up(pl.cap, 2);  // what follows the buffer stays 16-byte aligned
    pl.own_cap = 0;
    if (hist_bound > 0) pl.own_cap = round_up(hist_bound < pl.slice_len ? hist_bound : pl.slice_len, 4);
    pl.list_cap = pl.threads * 8;  // vectors the second pass can take; more than that sends the slice the careful way
    pl.seg_cap = round_up(pl.slice_len / (32 * pl.vec) + 1, 256);  // room for the padding of the last group (<= 256 entries)
    pl.smem_select = (size_t) pl.cap * 8 + (size_t) k_cap * 8 * 4 + (size_t) pl.slice_len / 8 + 32 + (size_t) pl.own_cap * 8 +
                     16 * 16 + (size_t) pl.list_cap * 4 + (size_t) pl.threads * 20 + (size_t) pl.seg_cap * 4 + sizeof(SelectShared) + 16;
    return pl.smem_select <= 200 * 1024;
}

// k_ring: one block per row, the row streamed through a ring of shared-memory stages by bulk copies.  Two blocks
// share an SM when the ring, the bit set and the cell maxima fit twice; a call with no more rows than SMs gives
// every block an SM of its own and a deeper ring.
bool make_ring_plan(const fns_b200_sampler * s, int dtype, int vocab, int rows, int hist_bound, Plan & pl) {
    const int k_cap = s->k_cap;
    const size_t esz = dtype == FNS_B200_BF16 ? 2 : 4;
    pl.ring = true;
    pl.threads = kRingThreads;
    pl.slices = 1;
    pl.slice_len = vocab;
    pl.vec = (int) (16 / esz);
    pl.n_stages = (vocab + kStageElems - 1) / kStageElems;
    if (pl.n_stages > kMaxRingStages) return false;
    pl.cap = round_up(4 * k_cap > 2048 ? 4 * k_cap : 2048, 2);
    pl.trigger = pl.cap / 2;
    pl.own_cap = hist_bound > 0 ? round_up(hist_bound < vocab ? hist_bound : vocab, 4) : 0;
    pl.list_cap = 4096;
    pl.seg_cap = 0;
    const size_t sh_bytes = (sizeof(SelectShared) + 15) & ~(size_t) 15;
    size_t fixed = 128 + sh_bytes + kMaxRingStages * 4 + (size_t) pl.n_stages * 1024;  // ... | chunk map, stage list | bit set
    fixed += (size_t) pl.n_stages * 1024;  // cell maxima
    pl.own_off = (int) fixed;
    fixed += (size_t) pl.own_cap * 4;
    pl.ring_off = (int) ((fixed + 127) & ~(size_t) 127);
    const size_t tail = (size_t) pl.cap * 8 + (size_t) pl.list_cap * 4 + (size_t) k_cap * 8 * 4 + (size_t) pl.own_cap * 4 +
                        (size_t) kRingThreads * 2 * 8;
    const size_t stage = (size_t) kStageElems * esz;
    // an SM has 228 KB of shared memory and every resident block costs 1 KB on top of what it asks for
    const size_t two_per_sm = 115200, one_per_sm = 225 * 1024;
    auto depth_for = [&](size_t budget) -> int {
        if ((size_t) pl.ring_off + tail > budget || (size_t) pl.ring_off + 2 * stage > budget) return 0;
        const size_t d = (budget - pl.ring_off) / stage;
        return (int) (d > (size_t) kMaxRingDepth ? kMaxRingDepth : d);
    };
    int depth = rows > s->sm_count ? depth_for(two_per_sm) : 0;
    if (depth < 2) depth = depth_for(one_per_sm);
    if (depth < 2) return false;
    if (depth > pl.n_stages) depth = pl.n_stages < 2 ? 2 : pl.n_stages;
    pl.ring_depth = depth;
    const size_t ring_bytes = (size_t) depth * stage;
    pl.smem_select = pl.ring_off + (ring_bytes > tail ? ring_bytes : tail);
    return true;
}

// k_cluster: one cluster of 16 CTAs per row for small batches (make_plan says how small).
bool make_cluster_plan(const fns_b200_sampler * s, int dtype, int vocab, int hist_bound, Plan & pl) {
    const int k_cap = s->k_cap;
    const size_t esz = dtype == FNS_B200_BF16 ? 2 : 4;
    if (k_cap > kClusterMaxK || !s->cluster_ok) return false;
    pl.cluster = true;
    pl.ring = false;
    pl.threads = kClusterThreads;
    pl.slices = kClusterCtas;
    pl.slice_len = round_up((vocab + kClusterCtas - 1) / kClusterCtas, 128);
    pl.vec = (int) (16 / esz);
    pl.cap = kClusterBuf;
    pl.trigger = kClusterLocal / 2;
    pl.own_cap = hist_bound > 0 ? round_up(hist_bound < pl.slice_len ? hist_bound : pl.slice_len, 4) : 0;
    pl.list_cap = 0;
    pl.seg_cap = 0;
    const size_t cs_bytes = (sizeof(ClusterShared) + 127) & ~(size_t) 127;
    pl.smem_select = cs_bytes + (size_t) pl.slice_len / 8 + (size_t) pl.slice_len * esz + (size_t) (hist_bound + 4) * 4 + (size_t) pl.own_cap * 4 +
                     (size_t) kClusterThreads * 2 * 8 + (size_t) (kClusterLocal + k_cap) * 8 + (size_t) (kClusterBuf + k_cap) * 8 +
                     (size_t) k_cap * 8 * 3;
    return pl.smem_select <= 112 * 1024;  // sixteen of them must be resident together (two fit an SM)
}

// Whole rows (from five rows on) go to k_ring when the call has no mask - every byte of the rows has to move, and
// the copy engine moves it best - and whenever k_cap exceeds the 512 thread maxima that k_select's bound is made of.
// Masked calls with k_cap <= 512 stay with k_select: its per-vector skipping and its loads in registers serve a
// batch better in which a few dense rows stream next to many sparse ones.
bool make_plan(const fns_b200_sampler * s, int dtype, int vocab, int rows, int hist_bound, bool aligned, bool masked, Plan & pl) {
    const bool whole_rows = s->force_threads <= 0 && s->force_slices <= 0 && rows > 4;  // (else: sliced rows, if no cluster takes them)
    pl.ring = false;
    pl.cluster = false;
    if (s->force_threads <= 0 && s->force_slices <= 0 && rows <= (masked ? s->cluster_rows : s->cluster_rows_unmasked) && aligned &&
        !s->logits_in_host_memory &&
        make_cluster_plan(s, dtype, vocab, hist_bound, pl))
        return true;
    pl.cluster = false;
    if (whole_rows && aligned && !s->logits_in_host_memory && (!masked || s->k_cap > kRingThreads) &&
        make_ring_plan(s, dtype, vocab, rows, hist_bound, pl))
        return true;
    pl.ring = false;
    if (whole_rows && make_plan_for(s, dtype, vocab, rows, hist_bound, aligned, true, pl)) return true;
    return make_plan_for(s, dtype, vocab, rows, hist_bound, aligned, false, pl);  // (a long history may not fit a whole row)
}

size_t final_smem(int lists, int list_len, int k_cap) {
    // all keys | staging, sorted, p, acc | scratch | (long lists) the other half of the pairwise merge
    const size_t spare = list_len > 64 ? ((size_t) (lists + 1) / 2 * list_len + k_cap) * 8 : 0;
    return (size_t) lists * list_len * 8 + (size_t) k_cap * 8 * 4 + sizeof(FinalShared) + 16 + spare;
}

// Every kernel that a sampling call can launch opts in to large dynamic shared memory, once per device, before the
// first launch on it.  Doing all of them together also loads all of them: with lazy module loading the first use
// of a kernel allocates device memory, which must not happen later (inside a stream capture, or in a process
// whose arena has taken the whole device).
template <typename K>
cudaError_t opt_in(K kern, int bytes) { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); }

template <typename T, int VEC>
cudaError_t opt_in_select() {
    cudaError_t e = opt_in(k_select<T, VEC, 512, false>, 200 * 1024);
    if (e == cudaSuccess) e = opt_in(k_select<T, VEC, 512, true>, 200 * 1024);
    if (e == cudaSuccess) e = opt_in(k_select<T, VEC, 256, false>, 200 * 1024);
    if (e == cudaSuccess) e = opt_in(k_select<T, VEC, 256, true>, 200 * 1024);
    return e;
}

cudaError_t configure_kernels_once() {  // call with the device current
    static std::mutex lock;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> hold(lock);
    if (configured[dev]) return cudaSuccess;
    e = opt_in_select<float, 4>();
    if (e == cudaSuccess) e = opt_in_select<float, 1>();
    if (e == cudaSuccess) e = opt_in_select<__nv_bfloat16, 8>();
    if (e == cudaSuccess) e = opt_in_select<__nv_bfloat16, 1>();
    if (e == cudaSuccess) e = opt_in(k_ring<float>, 226 * 1024);
    if (e == cudaSuccess) e = opt_in(k_ring<__nv_bfloat16>, 226 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_ring<float>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_ring<__nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = opt_in(k_finalize, 200 * 1024);
    if (e == cudaSuccess) e = opt_in(k_cluster<float>, 112 * 1024);
    if (e == cudaSuccess) e = opt_in(k_cluster<__nv_bfloat16>, 112 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_cluster<float>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_cluster<__nv_bfloat16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess) configured[dev] = true;
    return e;
}

template <typename T, int VEC, int NT, bool DIRECT>
cudaError_t launch_select_d(const SelectArgs & a, int rows, size_t smem, cudaStream_t st) {
    auto kern = k_select<T, VEC, NT, DIRECT>;
    const cudaError_t ce = configure_kernels_once();
    if (ce != cudaSuccess) return ce;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned) a.slices, (unsigned) rows);
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the prologue overlaps the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

template <typename T, int VEC, int NT>
cudaError_t launch_select_t(const SelectArgs & a, int rows, size_t smem, cudaStream_t st) {
    return a.slice_len <= 2 * NT * kEpochElems ? launch_select_d<T, VEC, NT, true>(a, rows, smem, st)
                                                : launch_select_d<T, VEC, NT, false>(a, rows, smem, st);
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

template <typename T>
cudaError_t launch_ring_t(const SelectArgs & a, int rows, size_t smem, cudaStream_t st) {
    auto kern = k_ring<T>;
    const cudaError_t ce = configure_kernels_once();
    if (ce != cudaSuccess) return ce;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned) rows);
    cfg.blockDim = dim3(kRingThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the prologue overlaps the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

template <typename T>
cudaError_t launch_cluster_t(const SelectArgs & a, int rows, size_t smem, cudaStream_t st) {
    const cudaError_t ce = configure_kernels_once();
    if (ce != cudaSuccess) return ce;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kClusterCtas, (unsigned) rows);
    cfg.blockDim = dim3(kClusterThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kClusterCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the prologue overlaps the previous kernel's tail
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, k_cluster<T>, a);
}

// Whether sixteen CTAs of k_cluster with their largest shared-memory request fit the device as one cluster.
int clusters_that_fit_device() {  // clusters of k_cluster (at its largest shared-memory size) resident at once
    if (configure_kernels_once() != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kClusterCtas, 1);
    cfg.blockDim = dim3(kClusterThreads);
    cfg.dynamicSmemBytes = 112 * 1024;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kClusterCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, k_cluster<float>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

cudaError_t launch_final(const FinalArgs & a, int rows, cudaStream_t st) {
    const size_t smem = final_smem(a.lists, a.list_len, a.k_cap);
    const cudaError_t ce = configure_kernels_once();
    if (ce != cudaSuccess) return ce;
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
               int32_t id_base, const uint32_t * masks, int64_t mask_stride, const int32_t * mask_rows, const int32_t * history,
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
    if (!make_plan(s, dtype, vocab, rows, hist_bound, aligned, masks != nullptr, pl)) return fail(s, FNS_B200_ERR_CAPACITY, "no launch plan fits (vocab too large for k_cap)");
    if (!pl.cluster && (size_t) rows * pl.slices * s->k_cap > s->cand_entries) return fail(s, FNS_B200_ERR_CAPACITY, "workspace too small for this call");
    SelectArgs a{};
    a.logits = logits;
    a.row_stride = row_stride;
    a.vocab = vocab;
    a.id_base = id_base;
    a.masks = masks;
    a.mask_stride = mask_stride;
    a.mask_rows = masks ? mask_rows : nullptr;
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
    a.own_cap = pl.own_cap;
    a.list_cap = pl.list_cap;
    a.seg_cap = pl.seg_cap;
    a.n_stages = pl.n_stages;
    a.ring_depth = pl.ring_depth;
    a.ring_off = pl.ring_off;
    a.own_off = pl.own_off;
    a.hist_cap = pl.cluster ? (int) ((history ? history_stride : 0) / 4 * 4) : 0;
    a.cand = s->cand;
    a.tickets = s->tickets;
    a.out_tokens = out_tokens;
    a.out_cands = out_cands;
    a.err = s->err;
    const bool prof = s->prof_on && (size_t) (s->prof_calls + 1) * 3 <= s->prof_ev.size();
    if (prof) cudaEventRecord(s->prof_ev[(size_t) s->prof_calls * 3], st);
    cudaError_t e;
    if (pl.cluster) e = dtype == FNS_B200_BF16 ? launch_cluster_t<__nv_bfloat16>(a, rows, pl.smem_select, st)
                                               : launch_cluster_t<float>(a, rows, pl.smem_select, st);
    else if (!pl.ring) e = launch_select(a, pl.threads, dtype, pl.vec, rows, pl.smem_select, st);
    else if (dtype == FNS_B200_BF16) e = launch_ring_t<__nv_bfloat16>(a, rows, pl.smem_select, st);
    else e = launch_ring_t<float>(a, rows, pl.smem_select, st);
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
    s->logits_in_host_memory = false;
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
    if (configure_kernels_once() != cudaSuccess) {
        delete s;
        return FNS_B200_ERR_CUDA;
    }
    const int clusters = clusters_that_fit_device();
    s->cluster_ok = clusters >= 4;  // four rows at once
    // Measured on B200 (V = 151,936 fp32, 12 clusters resident): under masks the cluster kernel wins up to 12 rows
    // (17 us against 22 us for one block per row) and ties at 16; without masks it wins up to 24 rows (24 against 28 us).
    s->cluster_rows = clusters < 12 ? clusters : 12;
    s->cluster_rows_unmasked = 2 * clusters < 24 ? 2 * clusters : 24;
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
        return fail(s, FNS_B200_ERR_DEVICE, flag == 3 ? "a bulk copy into shared memory never completed" : "kernel error flag set");
    }
    return FNS_B200_OK;
}


int fns_b200_hint_host_logits(fns_b200_sampler * s, int on) {
    if (!s) return FNS_B200_ERR_ARG;
    s->logits_in_host_memory = on != 0;
    return FNS_B200_OK;
}

int fns_b200_set_slices(fns_b200_sampler * s, int slices) {
    if (!s || slices < 0 || slices > kMaxSlices) return FNS_B200_ERR_ARG;
    s->force_slices = slices;
    return FNS_B200_OK;
}

int fns_b200_set_cluster_rows(fns_b200_sampler * s, int rows) {
    if (!s || rows < 0) return FNS_B200_ERR_ARG;
    s->cluster_rows = rows;
    s->cluster_rows_unmasked = rows;
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
    if (!make_plan(s, dtype, vocab, rows, history_bound, true, true, pl)) return FNS_B200_ERR_CAPACITY;
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
    int rc = run_select(s, logits, dtype, row_stride, vocab, rows, 0, masks, mask_stride_words, nullptr, history, history_stride,
                        history_len, nullptr, 0, params, nullptr, out_tokens, nullptr, (cudaStream_t) stream, pl);
    return rc;
}

int fns_b200_sample_rows_shared_masks(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab,
                                      int rows, const uint32_t * masks, int64_t mask_stride_words, const int32_t * mask_rows,
                                      const int32_t * history, int64_t history_stride, const int32_t * history_len,
                                      const fns_b200_params * params, int32_t * out_tokens, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_tokens || !params || !masks || !mask_rows) return fail(s, FNS_B200_ERR_ARG, "out_tokens, params, masks or mask_rows null");
    DeviceGuard g(s->device);
    Plan pl;
    return run_select(s, logits, dtype, row_stride, vocab, rows, 0, masks, mask_stride_words, mask_rows, history, history_stride,
                      history_len, nullptr, 0, params, nullptr, out_tokens, nullptr, (cudaStream_t) stream, pl);
}

int fns_b200_sample_one(fns_b200_sampler * s, const void * logits, int dtype, int vocab, const uint32_t * mask,
                        const int32_t * history, int history_len, const fns_b200_params * params_host,
                        int32_t * out_token, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_token || !params_host) return fail(s, FNS_B200_ERR_ARG, "out_token or params_host null");
    if (history && history_len > 0) return fail(s, FNS_B200_ERR_ARG, "sample_one takes no history: use sample_rows");
    DeviceGuard g(s->device);
    Plan pl;
    int rc = run_select(s, logits, dtype, vocab, vocab, 1, 0, mask, (vocab + 31) / 32, nullptr, nullptr, 0, nullptr, nullptr, 0,
                        nullptr, params_host, out_token, nullptr, (cudaStream_t) stream, pl);
    return rc;
}

int fns_b200_sample_one_with_history(fns_b200_sampler * s, const void * logits, int dtype, int vocab, const uint32_t * mask,
                                     const int32_t * history, int64_t history_stride, const int32_t * history_len,
                                     const fns_b200_params * params_host, int32_t * out_token, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_token || !params_host) return fail(s, FNS_B200_ERR_ARG, "out_token or params_host null");
    DeviceGuard g(s->device);
    Plan pl;
    return run_select(s, logits, dtype, vocab, vocab, 1, 0, mask, (vocab + 31) / 32, nullptr, history, history_stride, history_len,
                      nullptr, 0, nullptr, params_host, out_token, nullptr, (cudaStream_t) stream, pl);
}

int fns_b200_select_rows(fns_b200_sampler * s, const void * logits, int dtype, int64_t row_stride, int vocab, int rows,
                         int32_t id_base, const uint32_t * masks, int64_t mask_stride_words,
                         const int32_t * history, int64_t history_stride, const int32_t * history_len,
                         const fns_b200_params * params, fns_b200_cand * out_cands, void * stream) {
    if (!s) return FNS_B200_ERR_ARG;
    if (!out_cands || !params) return fail(s, FNS_B200_ERR_ARG, "out_cands or params null");
    DeviceGuard g(s->device);
    Plan pl;
    int rc = run_select(s, logits, dtype, row_stride, vocab, rows, id_base, masks, mask_stride_words, nullptr, history,
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
    int rc = run_select(s, logits, dtype, row_stride, vocab, rows, 0, masks, mask_stride_words, nullptr, history, history_stride,
                        history_len, draft, n_draft, params, nullptr, out_tokens, nullptr, (cudaStream_t) stream, pl);
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
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) return fail_text(FNS_B200_ERR_CUDA, cudaGetErrorString(e));
            // every kernel this entry point can ever launch is loaded and configured now, whatever the shape of
            // this first call: later calls of other shapes (other dtype, row count or alignment) find nothing to set up
            e = configure_kernels_once();
            if (e != cudaSuccess) return fail_text(FNS_B200_ERR_CUDA, cudaGetErrorString(e));
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
    const int rc = run_select(&s, logits, dtype, row_stride, vocab, rows, 0, masks, mask_stride_words, nullptr, history,
                              history_stride, history_len, nullptr, 0, params, nullptr, out_tokens, nullptr,
                              (cudaStream_t) stream, pl);
    if (rc != FNS_B200_OK) return fail_text(rc, s.msg);
    return FNS_B200_OK;
}
