// fns_device.cuh - device helpers of the sampler: order-preserving keys, the reference's Philox variant, and
// the block-wide exact top-k selection over 64-bit keys in shared memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "fns_internal.h"

namespace fnsb {

constexpr unsigned kFull = 0xffffffffu;

// ---- keys ---------------------------------------------------------------------------------------------
// The reference orders candidates by value descending, then index ascending, with float compares
// (src/kernels.cu:594, :637-638), and never selects a non-finite value (:629-639).  A candidate becomes one
// 64-bit key whose unsigned order IS that total order: high word = monotone image of the float (-0.0 folded
// onto +0.0, which the float compare ties), low word = ~id (smaller id -> larger key).  Keys of distinct
// elements are distinct, and key 0 never occurs (the high word of a finite float is >= 0x00800000), so 0 marks
// an empty slot.
__device__ __forceinline__ uint32_t order_word(float x) {
    uint32_t b = __float_as_uint(x);
    if (b == 0x80000000u) b = 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float word_value(uint32_t w) {
    return __uint_as_float((w & 0x80000000u) ? (w & 0x7fffffffu) : ~w);
}
__device__ __forceinline__ bool is_finite(float x) { return fabsf(x) <= FLT_MAX; }  // false for NaN and +-inf
__device__ __forceinline__ uint64_t make_key(float x, uint32_t id) {
    return ((uint64_t) order_word(x) << 32) | (uint32_t) ~id;
}
__device__ __forceinline__ float key_value(uint64_t key) { return word_value((uint32_t) (key >> 32)); }
__device__ __forceinline__ int32_t key_id(uint64_t key) { return (int32_t) ~(uint32_t) key; }
// Largest float v with make_key(x, id) >= key  =>  x >= v, for any key (also one whose low bits were zeroed).
__device__ __forceinline__ float key_floor_value(uint64_t key) {
    uint32_t w = (uint32_t) (key >> 32);
    if (w < 0x00800000u) w = 0x00800000u;  // order word of -FLT_MAX
    return word_value(w);
}

__device__ __forceinline__ fns_b200_cand key_to_cand(uint64_t key) {
    fns_b200_cand c;
    if (key == 0) {
        c.value = -FLT_MAX;
        c.id = FNS_B200_EMPTY_ID;
    } else {
        c.value = key_value(key);
        c.id = key_id(key);
    }
    return c;
}
__device__ __forceinline__ uint64_t cand_to_key(fns_b200_cand c) {
    return (c.id == FNS_B200_EMPTY_ID || c.id < 0 || !is_finite(c.value)) ? 0ull : make_key(c.value, (uint32_t) c.id);
}

// ---- Philox ---------------------------------------------------------------------------------------------
// The reference's generator (src/kernels.cu:652-665): state (counter lo, counter hi, seed lo, seed hi), ten
// rounds, round index xored into the first word, no key schedule; u = (word >> 8) * 2^-24 in [0, 1).
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t counter) {
    uint32_t c0 = (uint32_t) counter, c1 = (uint32_t) (counter >> 32);
    uint32_t c2 = (uint32_t) seed, c3 = (uint32_t) (seed >> 32);
#pragma unroll
    for (uint32_t i = 0; i < 10; ++i) {
        const uint32_t hi0 = __umulhi(0x9E3779B9u, c0), lo0 = 0x9E3779B9u * c0;
        const uint32_t hi1 = __umulhi(0xBB67AE85u, c2), lo1 = 0xBB67AE85u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ i, n2 = hi0 ^ c3;
        c0 = n0;
        c1 = lo1;
        c2 = n2;
        c3 = lo0;
    }
    return (float) (c0 >> 8) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ int clamp_k(int top_k, int k_cap) { return (top_k <= 0 || top_k > k_cap) ? k_cap : top_k; }

// ---- block-wide selection ---------------------------------------------------------------------------------
struct SelectScratch {
    uint32_t hist[256];
    uint32_t or_hi, or_lo, and_hi, and_lo;
    uint32_t bucket, need, bucket_count, count;
};

// tau such that exactly min(k, n) of the DISTINCT, NON-ZERO keys buf[0 .. n) are >= tau (0 when n <= k).
// MSB-first radix select, 8 bits per pass, starting below the bits that all keys share (the keys that reach a
// compaction lie in a narrow value range, so their leading bits agree and a histogram over them would put
// every atomic on one bin).  It stops as soon as the pivot bucket is taken whole; tau then has zero low bits.
// Called by all NT threads of the block with uniform arguments; ends with the block synchronised.
template <int NT>
__device__ uint64_t block_kth_key(const uint64_t * buf, int n, int k, SelectScratch & sc) {
    const int tid = threadIdx.x, lane = tid & 31;
    if (n <= k) return 0ull;
    if (tid == 0) {
        sc.or_hi = sc.or_lo = 0u;
        sc.and_hi = sc.and_lo = 0xffffffffu;
    }
    __syncthreads();
    {
        uint32_t oh = 0, ol = 0, ah = 0xffffffffu, al = 0xffffffffu;
        for (int i = tid; i < n; i += NT) {
            const uint64_t key = buf[i];
            oh |= (uint32_t) (key >> 32);
            ol |= (uint32_t) key;
            ah &= (uint32_t) (key >> 32);
            al &= (uint32_t) key;
        }
        oh = __reduce_or_sync(kFull, oh);
        ol = __reduce_or_sync(kFull, ol);
        ah = __reduce_and_sync(kFull, ah);
        al = __reduce_and_sync(kFull, al);
        if (lane == 0) {
            atomicOr(&sc.or_hi, oh);
            atomicOr(&sc.or_lo, ol);
            atomicAnd(&sc.and_hi, ah);
            atomicAnd(&sc.and_lo, al);
        }
    }
    __syncthreads();
    const uint64_t all_or = ((uint64_t) sc.or_hi << 32) | sc.or_lo, all_and = ((uint64_t) sc.and_hi << 32) | sc.and_lo;
    const uint64_t varying = all_or ^ all_and;
    if (varying == 0ull) return all_and;  // n > k >= 1 equal keys cannot happen with distinct keys; harmless
    int remaining = 64 - __clzll((long long) varying);                      // bits still undecided: [0, remaining)
    uint64_t pmask = remaining == 64 ? 0ull : ~((1ull << remaining) - 1ull);  // bits already decided
    uint64_t prefix = all_and & pmask;
    int need = k;
    while (remaining > 0) {
        const int bits = remaining < 8 ? remaining : 8;
        const int shift = remaining - bits;
        const uint32_t dmask = (1u << bits) - 1u;
        for (int i = tid; i < 256; i += NT) sc.hist[i] = 0u;
        __syncthreads();
        for (int i = tid; i < n; i += NT) {
            const uint64_t key = buf[i];
            if ((key & pmask) == prefix) atomicAdd(&sc.hist[(uint32_t) (key >> shift) & dmask], 1u);
        }
        __syncthreads();
        if (tid < 32) {
            uint32_t c[8], s = 0;
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                c[b] = sc.hist[lane * 8 + b];
                s += c[b];
            }
            uint32_t incl = s;  // keys in the bins of lanes >= this one
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_down_sync(kFull, incl, o);
                if (lane + o < 32) incl += t;
            }
            uint32_t above = incl - s;  // keys in the bins of higher lanes
            if (above < (uint32_t) need && (uint32_t) need <= incl) {  // the pivot bin is one of this lane's
                bool found = false;
#pragma unroll
                for (int b = 7; b >= 0; --b) {
                    if (!found) {
                        if (above + c[b] >= (uint32_t) need) {
                            sc.bucket = (uint32_t) (lane * 8 + b);
                            sc.need = (uint32_t) need - above;
                            sc.bucket_count = c[b];
                            found = true;
                        } else {
                            above += c[b];
                        }
                    }
                }
            }
        }
        __syncthreads();
        prefix |= (uint64_t) sc.bucket << shift;
        pmask |= (uint64_t) dmask << shift;
        need = (int) sc.need;
        remaining = shift;
        if (sc.bucket_count == (uint32_t) need) break;
    }
    __syncthreads();  // sc.* is reused by the next call
    return prefix;
}

// Moves the keys >= tau of buf[0 .. n) (at most k of them) to sel[0 .. ), and returns how many.  sc.count is the
// cursor.  Ends with the block synchronised.
template <int NT>
__device__ int block_take(const uint64_t * buf, int n, int k, uint64_t tau, uint64_t * sel, SelectScratch & sc) {
    const int tid = threadIdx.x;
    if (tid == 0) sc.count = 0u;
    __syncthreads();
    for (int i = tid; i < n; i += NT) {
        const uint64_t key = buf[i];
        if (key >= tau) {
            const uint32_t pos = atomicAdd(&sc.count, 1u);
            if (pos < (uint32_t) k) sel[pos] = key;
        }
    }
    __syncthreads();
    const int got = (int) min(sc.count, (uint32_t) k);
    __syncthreads();
    return got;
}

// out[rank] = key for the m distinct keys of sel, rank = number of larger keys: descending order = the total
// order.  out may be shared or global.  No synchronisation inside.
template <int NT>
__device__ void block_rank_sort(const uint64_t * sel, int m, uint64_t * out) {
    for (int i = threadIdx.x; i < m; i += NT) {
        const uint64_t key = sel[i];
        int rank = 0;
#pragma unroll 8
        for (int j = 0; j < m; ++j) rank += sel[j] > key ? 1 : 0;
        out[rank] = key;
    }
}

// For small n: out[rank] = key for every key whose rank (number of larger keys) is below k: the best k in the
// total order, with no barrier and no scratch.  Every key is compared with every other, so only worth it while
// n * n / NT stays small.  Returns min(n, k); out must not alias buf.
template <int NT>
__device__ int block_rank_select(const uint64_t * buf, int n, int k, uint64_t * out) {
    for (int i = threadIdx.x; i < n; i += NT) {
        const uint64_t key = buf[i];
        int rank = 0;
#pragma unroll 8
        for (int j = 0; j < n; ++j) rank += buf[j] > key ? 1 : 0;
        if (rank < k) out[rank] = key;
    }
    return n < k ? n : k;
}

}  // namespace fnsb
