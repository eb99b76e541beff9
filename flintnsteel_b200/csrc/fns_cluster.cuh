// fns_cluster.cuh - k_cluster: the select + draw kernel for small batches (launch-to-token latency): as many rows as
// the device holds clusters at once, and without masks twice that.
// Included by fns_sampler.cu after the shared helpers (push, compact, draw_tail, merge_lists, ...).
//
// One thread-block cluster of 16 CTAs per row; a CTA owns one sixteenth of the row.  The slice comes into shared
// memory with ONE bulk asynchronous copy (cp.async.bulk, own-GPU global memory, no multicast) and stays there: the
// maxima pass and the candidate pass both read shared memory, nothing is read twice from global memory, and the
// history ids' logits are simply looked up in the slice.  The CTAs meet in distributed shared memory, not in global
// memory:
//   1. every warp writes the two largest of its threads' maxima into CTA 0 (256 witnesses: distinct elements);
//      cluster barrier; every CTA reads the witnesses and ranks them by counting: the k-th largest is a bound that
//      at least k elements of the row reach
//   2. every CTA offers the elements of its slice that reach the bound, and its penalised history ids, straight into
//      CTA 0's candidate buffer (one remote reservation per warp); cluster barrier
//   3. CTA 0 ranks the (about k + a few) keys and draws
// If the buffer overflows (equal values, or a mask that leaves too few witnesses for a bound), every CTA reduces its
// slice to its own best k by the careful walk with compaction, the lists meet in CTA 0 and are merged there: any
// input is handled exactly.  No spin waits anywhere: the only waits are the hardware cluster barrier and one
// bounded mbarrier wait for the bulk copy.
#pragma once

namespace fnsb {

constexpr int kClusterCtas = 16;
constexpr int kClusterThreads = 256;
constexpr int kClusterRegion = 128;   // keys a CTA may send to CTA 0 directly; more (from any CTA) means the careful way
constexpr int kClusterBuf = kClusterCtas * kClusterRegion;
constexpr int kClusterLocal = 2048;   // keys of a CTA's own buffer (careful way; in CTA 0 also the regions side by side)
constexpr int kClusterMaxK = 128;     // 256 witnesses give a bound for k up to this
constexpr int kClusterRankMax = 640;  // CTA 0 ranks up to this many keys by counting (n * n / 256 compares per thread)

struct ClusterShared {
    SelectShared s;
    uint64_t bar;                 // the mbarrier of the slice's bulk copy
    uint64_t hbar;                // ... and of the history ids' 
    uint32_t region_n[kClusterCtas];  // CTA 0: how many candidates every CTA sent
    uint32_t bound_word;          // order word of the bound (0: none)
    uint32_t local_bound[kClusterCtas];  // second chance: the bound that each CTA could make of its own threads' maxima
    __align__(16) uint32_t wit[kClusterCtas * 16];  // the witnesses, two per warp of the cluster (every CTA gets a copy)
};

// The k-th largest of 256 order words in shared memory (0 = no value; words below 0x00800000 stand for no finite
// element), for one warp: every lane takes eight words, the bits in which the words differ are found first, and the
// search decides up to 14 bits from the highest of them downwards, two bits per step with three warp-wide counts that
// do not wait for one another; it stops early once at most four words too many remain.  Returns a word that at least
// k of them reach (not always the largest such), or 0 when there are fewer than k.  The same value in every lane.
__device__ __forceinline__ uint32_t warp_kth_of_256(const uint32_t * w256, int k) {
    const int lane = threadIdx.x & 31;
    uint32_t w8[8];
    {
        const uint4 lo4 = *reinterpret_cast<const uint4 *>(&w256[lane * 8]), hi4 = *reinterpret_cast<const uint4 *>(&w256[lane * 8 + 4]);
        w8[0] = lo4.x; w8[1] = lo4.y; w8[2] = lo4.z; w8[3] = lo4.w;
        w8[4] = hi4.x; w8[5] = hi4.y; w8[6] = hi4.z; w8[7] = hi4.w;
    }
    uint32_t wo = 0u, wa = 0xffffffffu, have = 0u;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        if (w8[q] < 0x00800000u) w8[q] = 0u;  // (no finite element behind it)
        else {
            wo |= w8[q];
            wa &= w8[q];
            ++have;
        }
    }
    wo = __reduce_or_sync(kFull, wo);
    wa = __reduce_and_sync(kFull, wa);
    have = __reduce_add_sync(kFull, have);
    uint32_t bw = 0u;
    if (have >= (uint32_t) k) {  // else: fewer than k words, no bound
        const uint32_t varying = wo & ~wa;
        bw = varying ? (wa & ~((2u << (31 - __clz((int) varying))) - 1u)) : wa;  // the common prefix: a valid bound
        if (varying) {
            const int top = 31 - __clz((int) varying);
            const int stop = top > 13 ? top - 13 : 0;
#pragma unroll 1
            for (int bit = top; bit >= stop; bit -= 2) {
                const uint32_t b1 = 1u << bit, b0 = bit > stop ? 1u << (bit - 1) : 0u;
                uint32_t c1 = 0u, c10 = 0u, c0 = 0u;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    c1 += w8[q] >= (bw | b1) ? 1u : 0u;
                    c10 += w8[q] >= (bw | b1 | b0) ? 1u : 0u;
                    c0 += w8[q] >= (bw | b0) ? 1u : 0u;
                }
                c1 = __reduce_add_sync(kFull, c1);
                c10 = __reduce_add_sync(kFull, c10);
                c0 = __reduce_add_sync(kFull, c0);
                uint32_t tot = 0xffffffffu;
                if (c10 >= (uint32_t) k) bw |= b1 | b0, tot = c10;
                else if (c1 >= (uint32_t) k) bw |= b1, tot = c1;
                else if (c0 >= (uint32_t) k) bw |= b0, tot = c0;
                if (tot <= (uint32_t) k + 4u) break;  // close enough: at most four words too many
            }
        }
    }
    return bw >= 0x00800000u ? bw : 0u;
}

template <typename T>
__global__ void __launch_bounds__(kClusterThreads, 1) k_cluster(const SelectArgs a) {
    namespace cg = cooperative_groups;
    constexpr int NT = kClusterThreads, kWarps = NT / 32;
    constexpr int VEC = 16 / (int) sizeof(T);
    constexpr uint32_t kVecBits = (1u << VEC) - 1u;
    constexpr int TS = 2 * NT;
    constexpr int kTShift = 23;  // 32 - log2(TS)
    constexpr uint32_t kNoKey = 0xffffffffu;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rank = (int) cluster.block_rank();
    const int row = blockIdx.y;
    const int W = a.n_draft + 1, win = row / W, col = row - win * W;
    const int lo = rank * a.slice_len;
    const int n_s = max(0, min(a.vocab, lo + a.slice_len) - lo);
    const int words = (n_s + 31) >> 5;

    // shared memory: ClusterShared | slice bit set | slice data | owned history ids | occurrence table | own buffer,
    // staging (careful way) | CTA 0: cluster buffer, staging, sorted, p, acc
    ClusterShared & cs = *reinterpret_cast<ClusterShared *>(smem_raw);
    SelectShared & sh = cs.s;
    constexpr size_t kCsBytes = (sizeof(ClusterShared) + 127) & ~(size_t) 127;
    uint32_t * eff = reinterpret_cast<uint32_t *>(smem_raw + kCsBytes);                 // [slice_len / 32]
    T * data = reinterpret_cast<T *>(eff + a.slice_len / 32);                           // [slice_len]
    int32_t * hid = reinterpret_cast<int32_t *>(data + a.slice_len);                    // [hist_cap] the row's history ids
    uint32_t * own = reinterpret_cast<uint32_t *>(hid + a.hist_cap);                    // [own_cap]
    uint32_t * tkey = own + a.own_cap;                                                  // [TS]
    uint32_t * tcnt = tkey + TS;                                                        // [TS]
    uint64_t * lbuf = reinterpret_cast<uint64_t *>(tcnt + TS);                          // [kClusterLocal]
    uint64_t * lsel = lbuf + kClusterLocal;                                             // [k_cap]
    uint64_t * gbuf = lsel + a.k_cap;                                                   // [kClusterBuf] (CTA 0's is used)
    uint64_t * gsel = gbuf + kClusterBuf;                                               // [k_cap]
    uint64_t * sorted = gsel + a.k_cap;                                                 // [k_cap]
    double * pj = reinterpret_cast<double *>(sorted + a.k_cap);                         // [k_cap]
    double * acc = pj + a.k_cap;                                                        // [k_cap]
    ClusterShared * cs0 = cluster.map_shared_rank(&cs, 0);
    uint64_t * gbuf0 = cluster.map_shared_rank(gbuf, 0);

    if (tid == 0) {
        mbar_init(&cs.bar, 1u);
        mbar_init(&cs.hbar, 1u);
        mbar_init_fence();
        sh.n_cand = 0u;
        sh.thr_key = 0ull;
        sh.n_own = 0u;
        cs.bound_word = 0u;
    }
    for (int i = tid; i < TS; i += NT) {
        tkey[i] = kNoKey;
        tcnt[i] = 0u;
    }
    // 1. the slice's bit set.  Without a mask it depends on nothing in global memory and is made here, ahead of the wait.
    const uint32_t tail_bits = (n_s & 31) ? (1u << (n_s & 31)) - 1u : 0xffffffffu;
    if (!a.masks)
        for (int w = tid; w < a.slice_len / 32; w += NT) eff[w] = w < words ? (w == words - 1 ? tail_bits : 0xffffffffu) : 0u;
    __syncthreads();
    // Launched with programmatic stream serialisation: nothing is read from global memory before the previous
    // kernel of the stream has finished; what precedes this line overlaps its tail.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // (the row's parameters and the first mask words first: their latency passes while the copies are being issued)
    fns_b200_params p = a.params ? a.params[win] : a.p0;
    int n_hist = (a.history && a.history_len) ? a.history_len[win] : 0;
    const uint32_t * mrow = a.masks ? a.masks + (size_t) (a.mask_rows ? a.mask_rows[row] : row) * a.mask_stride + (lo >> 5) : nullptr;
    constexpr int kMaskRegs = 4;  // mask words a thread fetches ahead (slices of up to 32,768 elements: all of them)
    uint32_t mreg[kMaskRegs];
    if (mrow) {
#pragma unroll
        for (int q = 0; q < kMaskRegs; ++q) mreg[q] = tid + q * NT < words ? mrow[tid + q * NT] : 0u;
    }
    const T * x = reinterpret_cast<const T *>(a.logits) + (size_t) row * a.row_stride + lo;
    const uint32_t id0 = (uint32_t) (a.id_base + lo);
    const int32_t * hrow = a.history ? a.history + (size_t) win * a.history_stride : nullptr;
    const int32_t * drow = a.draft ? a.draft + (size_t) win * a.n_draft : nullptr;
    // The slice: whole 16-byte vectors by one bulk copy, a ragged end by plain loads.  The row's history ids come into
    // shared memory with one more bulk copy (when the list is 16-byte aligned): every later walk over them - the
    // scatter, the occurrence count - reads shared memory.  The two copies are issued by threads of different warps.
    const uint32_t bulk_bytes = ((uint32_t) n_s * (uint32_t) sizeof(T)) & ~15u;
    const bool hist_staged = hrow && a.own_cap > 0 && a.hist_cap > 0 && (reinterpret_cast<uintptr_t>(hrow) & 15u) == 0;
    if (tid == 0) {
        if (bulk_bytes) bulk_load(data, x, bulk_bytes, &cs.bar);
        mbar_arrive_expect(&cs.bar, bulk_bytes);
    } else if (tid == 32) {
        const uint32_t hb = hist_staged ? (uint32_t) a.hist_cap * 4u : 0u;  // (hist_cap: the stride rounded down to 4 ids)
        if (hb) bulk_load(hid, hrow, hb, &cs.hbar);
        mbar_arrive_expect(&cs.hbar, hb);
    }
    for (int e = (int) (bulk_bytes / sizeof(T)) + tid; e < n_s; e += NT) data[e] = x[e];
    if (mrow) {
#pragma unroll
        for (int q = 0; q < kMaskRegs; ++q) {
            const int w = tid + q * NT;
            if (w < a.slice_len / 32) eff[w] = w == words - 1 ? mreg[q] & tail_bits : mreg[q];
        }
        for (int w = tid + kMaskRegs * NT; w < a.slice_len / 32; w += NT) {
            uint32_t m = w < words ? mrow[w] : 0u;
            if (w == words - 1) m &= tail_bits;
            eff[w] = m;
        }
    }
    const int k = p.temperature <= 0.0f ? 1 : clamp_k(p.top_k, a.k_cap);
    const bool any_pen = p.repetition != 1.0f || p.presence != 0.0f || p.frequency != 0.0f;
    const bool use_hist = any_pen && a.own_cap > 0 && n_s > 0;
    n_hist = n_hist < 0 ? 0 : (n_hist > (int) a.history_stride ? (int) a.history_stride : n_hist);
    const int n_pen = n_hist + (a.draft ? col : 0);
    if (mrow) __syncthreads();

    // 2. history ids of the slice clear their bits; the thread that clears a bit owns the id
    auto pen_id = [&](int j) -> int32_t {  // id j of the row's history followed by the window's draft prefix
        if (j >= n_hist) return j < n_pen ? drow[j - n_hist] : -1;
        return (hist_staged && j < a.hist_cap) ? hid[j] : hrow[j];
    };
    if (use_hist && n_pen > 0) {
        if (hist_staged && !mbar_wait(&cs.hbar, 0u) && a.err) atomicExch(a.err, 3);
        // Sixteen ids per thread at a time, as four vectors of four from shared memory.  The steps are kept apart - all
        // loads, all range tests, all reads of the bit set, then the atomics - because an atomic in between would keep
        // the compiler from moving the later loads ahead of it, and the ids would be handled one after the other.
        const bool vec_ok = hist_staged && n_hist <= a.hist_cap;  // every history id is in shared memory
        auto claim = [&](auto hb, int j0) {
            constexpr int HB = decltype(hb)::value;
            int32_t id[HB];
#pragma unroll
            for (int q = 0; q < HB / 4; ++q) {
                const int jb = j0 + q * 4 * NT + tid * 4;
                if (vec_ok && jb + 4 <= n_hist) {
                    const int4 v = *reinterpret_cast<const int4 *>(hid + jb);
                    id[4 * q] = v.x; id[4 * q + 1] = v.y; id[4 * q + 2] = v.z; id[4 * q + 3] = v.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) id[4 * q + e] = jb + e < n_pen ? pen_id(jb + e) : -1;
                }
            }
            uint32_t offv[HB], wv[HB], inr = 0u, won = 0u;  // bit u of won: this thread owns id[u]
#pragma unroll
            for (int u = 0; u < HB; ++u) {
                offv[u] = (uint32_t) (id[u] - a.id_base - lo);
                if (offv[u] < (uint32_t) n_s && id[u] >= a.id_base) inr |= 1u << u;
            }
#pragma unroll
            for (int u = 0; u < HB; ++u) wv[u] = ((inr >> u) & 1u) ? eff[offv[u] >> 5] : 0u;
#pragma unroll
            for (int u = 0; u < HB; ++u) {
                const uint32_t bit = 1u << (offv[u] & 31);
                // (the plain read came first: ids that the mask excludes, and repeats, cost no atomic; a stale 1 is settled
                // by the atomic itself, and a 0 stays 0)
                if ((wv[u] & bit) && (atomicAnd(&eff[offv[u] >> 5], ~bit) & bit)) won |= 1u << u;
            }
            const uint32_t mine_n = (uint32_t) __popc(won);
            if (__ballot_sync(kFull, mine_n != 0u) == 0u) return;
            uint32_t upto = mine_n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(kFull, upto, o);
                if (lane >= o) upto += t;
            }
            uint32_t at = 0u;
            if (lane == 31) at = atomicAdd(&sh.n_own, upto);
            at = __shfl_sync(kFull, at, 31) + upto - mine_n;
#pragma unroll
            for (int u = 0; u < HB; ++u)
                if ((won >> u) & 1u) own[at++] = offv[u];
        };
        int j0 = 0;
#pragma unroll 1
        for (; n_pen - j0 > 4 * NT; j0 += 16 * NT) claim(std::integral_constant<int, 16>{}, j0);
        if (j0 < n_pen) claim(std::integral_constant<int, 4>{}, j0);  // (a short list, or a short rest: one vector per thread)
    }
    __syncthreads();
    const int n_own = use_hist ? (int) sh.n_own : 0;

    // 3. the maxima of the threads over the slice in shared memory
    const bool arrived = mbar_wait(&cs.bar, 0u);
    if (!arrived && a.err) atomicExch(a.err, 3);
    __syncthreads();  // (the ragged end written by plain stores is visible too)
    const int n_vec = (n_s + VEC - 1) / VEC;
    auto vec_bits = [&](int v) -> uint32_t { return (eff[(v * VEC) >> 5] >> ((v * VEC) & 31)) & kVecBits; };
    auto vec_load = [&](int v, float (&xv)[VEC]) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(data + (size_t) v * VEC);
        if constexpr (sizeof(T) == 4) {
            xv[0] = __uint_as_float(raw.x);
            xv[1] = __uint_as_float(raw.y);
            xv[2] = __uint_as_float(raw.z);
            xv[3] = __uint_as_float(raw.w);
        } else {
            const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                xv[2 * q] = __uint_as_float(w4[q] << 16);
                xv[2 * q + 1] = __uint_as_float(w4[q] & 0xffff0000u);
            }
        }
    };
    // (every thread also keeps which of its vectors holds its maximum, and the largest value of its other vectors: the
    // candidate pass then re-reads one vector per thread, the others only if they can matter)
    float tmax = -INFINITY, tmax2 = -INFINITY;
    int vmax_at = tid;
#pragma unroll 4
    for (int v = tid; v < n_vec; v += NT) {
        const uint32_t bits = vec_bits(v);
        float xv[VEC];
        vec_load(v, xv);
        float vm = -INFINITY;
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            if (((bits >> j) & 1u) && fabsf(xv[j]) <= FLT_MAX) vm = fmaxf(vm, xv[j]);  // finite and allowed (src/kernels.cu:629-639)
        if (vm > tmax) {
            tmax2 = tmax;
            tmax = vm;
            vmax_at = v;
        } else {
            tmax2 = fmaxf(tmax2, vm);
        }
    }
    // the two largest thread maxima of every warp go to CTA 0: 2 * 8 * 16 witnesses, all different elements
    {
        uint32_t w = tmax > -INFINITY ? order_word(tmax) : 0u;
        const uint32_t w1 = __reduce_max_sync(kFull, w);
        const uint32_t holders = __ballot_sync(kFull, w == w1);
        if (lane == __ffs(holders) - 1) w = 0u;
        const uint32_t w2 = __reduce_max_sync(kFull, w);
        // every CTA receives the witnesses (lane l stores into CTA l / 2): the bound search then reads its own memory
        cluster.map_shared_rank(&cs, lane >> 1)->wit[(rank * kWarps + warp) * 2 + (lane & 1)] = (lane & 1) ? w2 : w1;
    }
    cluster.sync();

    // 4. the bound: the k-th largest witness, found by one warp of every CTA in its own copy of the witnesses.
    if (warp == 0) {
        const uint32_t bw = warp_kth_of_256(cs.wit, k);
        if (lane == 0) cs.bound_word = bw;
    }
    __syncthreads();
    if (cs.bound_word == 0u) {  // (the same in every CTA: all searched the same witnesses)
        // Fewer than k witnesses.  Under a mask whose allowed ids lie in a few slices that is no proof that the row has
        // fewer than k candidates: a CTA whose own threads hold k maxima makes a bound of them, every CTA gets every
        // such bound, and the largest is the row's.  (Two warps' witnesses per CTA were all that it could send above.)
        uint32_t * w256 = reinterpret_cast<uint32_t *>(lbuf);  // (the CTA's buffer is not in use yet)
        w256[tid] = tmax > -INFINITY ? order_word(tmax) : 0u;
        __syncthreads();
        if (warp == 0) {
            const uint32_t mine = warp_kth_of_256(w256, k);
            if (lane < kClusterCtas) cluster.map_shared_rank(&cs, lane)->local_bound[rank] = mine;
        }
        cluster.sync();
        uint32_t best = 0u;
#pragma unroll
        for (int r = 0; r < kClusterCtas; ++r) best = max(best, cs.local_bound[r]);
        __syncthreads();  // (w256 is the candidate buffer again)
        if (tid == 0) cs.bound_word = best;
        __syncthreads();
    }
    const bool no_bound = cs.bound_word == 0u;  // (the same in every CTA of the cluster)
    float thr_v = cs.bound_word ? word_value(cs.bound_word) + 0.0f : -FLT_MAX;
    uint64_t thr_key = (uint64_t) order_word(thr_v) << 32;
    auto penalised = [&](float v, float cnt) -> float {  // each step rounded on its own: no fused multiply-add
        v = v > 0.0f ? __fdiv_rn(v, p.repetition) : __fmul_rn(v, p.repetition);
        v = __fsub_rn(v, __fmul_rn(p.frequency, cnt));
        return __fsub_rn(v, p.presence);
    };
    // the owned history ids: penalised value, occurrences counted only for those that could pass (see k_select)
    const bool counts = p.frequency != 0.0f, count_all = p.frequency < 0.0f;
    auto history_key = [&](int j) -> uint64_t {  // every thread of the block calls it in the same round; j may be past the list
        uint32_t off = 0u;
        float raw = 0.0f, v = -INFINITY;
        bool live = j < n_own;
        if (live) {
            off = own[j];
            raw = to_float(data[off]);
            v = penalised(raw, 1.0f);
            live = count_all || v >= thr_v;
        }
        if (counts && __syncthreads_or(live)) {
            // usually one or two ids need their occurrences: they go on a short list and every history id is compared
            // with the list; only a longer list takes the table
            uint32_t * few = sh.sc.hist;  // [0]: cursor, [1 .. 8]: offsets, [9 .. 16]: counts
            if (tid < 17) few[tid] = 0u;
            __syncthreads();
            uint32_t place = 0xffffffffu;
            if (live) place = atomicAdd(&few[0], 1u);
            __syncthreads();
            const uint32_t n_few = few[0];
            if (n_few <= 8u) {
                if (live) few[1 + place] = off;
                __syncthreads();
                uint32_t fo[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) fo[q] = (uint32_t) q < n_few ? few[1 + q] : 0xffffffffu;
                const bool vec_ok = hist_staged && n_hist <= a.hist_cap;
#pragma unroll 2
                for (int t0 = tid * 4; t0 < n_pen; t0 += 4 * NT) {  // four ids per thread and round; matches first, atomics after
                    int32_t id4[4];
                    if (vec_ok && t0 + 4 <= n_hist) {
                        const int4 v = *reinterpret_cast<const int4 *>(hid + t0);
                        id4[0] = v.x; id4[1] = v.y; id4[2] = v.z; id4[3] = v.w;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) id4[e] = t0 + e < n_pen ? pen_id(t0 + e) : -1;
                    }
                    uint32_t hits = 0u;  // bit 8 e + q: id e is the list's entry q
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t o = id4[e] >= a.id_base ? (uint32_t) (id4[e] - a.id_base - lo) : 0xfffffffeu;
#pragma unroll
                        for (int q = 0; q < 8; ++q) hits |= o == fo[q] ? 1u << (8 * e + q) : 0u;
                    }
                    for (; hits; hits &= hits - 1u) atomicAdd(&few[9 + ((__ffs(hits) - 1) & 7)], 1u);
                }
                __syncthreads();
                if (live) v = penalised(raw, (float) few[9 + place]);
                __syncthreads();
            } else {
                uint32_t slot = 0u;
                if (live) {
                    slot = (off * 2654435761u) >> kTShift;
                    while (atomicCAS(&tkey[slot], kNoKey, off) != kNoKey) slot = (slot + 1u) & (TS - 1);
                }
                __syncthreads();
#pragma unroll 1
                for (int t = tid; t < n_pen; t += NT) {
                    const int32_t id = pen_id(t);
                    const uint32_t o = (uint32_t) (id - a.id_base - lo);
                    if (o >= (uint32_t) n_s || id < a.id_base) continue;
                    uint32_t h = (o * 2654435761u) >> kTShift;
                    for (uint32_t kx = tkey[h]; kx != kNoKey; kx = tkey[h]) {
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
        }
        return (live && is_finite(v)) ? make_key(v, id0 + off) : 0ull;
    };

    // 5. everything that reaches the bound is gathered in this CTA's own buffer first (shared-memory atomics are
    // cheap), then sent to CTA 0 in one piece: one remote reservation per CTA, so the latency of distributed shared
    // memory is paid once.
    auto offer_local = [&](uint64_t key) {  // every lane of the warp calls it; key 0 = nothing to offer
        const bool has = key != 0ull && key >= thr_key;
        const uint32_t b = __ballot_sync(kFull, has);
        if (b == 0u) return;
        uint32_t base = 0u;
        if (lane == 0) base = atomicAdd(&sh.n_cand, (uint32_t) __popc(b));
        base = __shfl_sync(kFull, base, 0);
        const uint32_t at = base + (uint32_t) __popc(b & ((1u << lane) - 1u));
        if (has && at < (uint32_t) kClusterLocal) lbuf[at] = key;
    };
    {
        for (int j0 = 0; j0 < n_own; j0 += NT) offer_local(history_key(j0 + tid));
        // The elements that reach the bound: one reservation per round of the warp, whatever the number of hits.
        auto offer_vec = [&](uint32_t hit, const float (&xv)[VEC], int v) {  // every lane calls it; hit: elements of vector v to offer
            uint32_t total = 0u, pos[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                const uint32_t b = __ballot_sync(kFull, (hit >> j) & 1u);
                pos[j] = total + (uint32_t) __popc(b & ((1u << lane) - 1u));
                total += (uint32_t) __popc(b);
            }
            if (total == 0u) return;
            uint32_t base = 0u;
            if (lane == 0) base = atomicAdd(&sh.n_cand, total);
            base = __shfl_sync(kFull, base, 0);
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (((hit >> j) & 1u) && base + pos[j] < (uint32_t) kClusterLocal) lbuf[base + pos[j]] = make_key(xv[j], id0 + (uint32_t) (v * VEC + j));
        };
        auto hits_of = [&](int v, float (&xv)[VEC]) -> uint32_t {
            const uint32_t bits = v < n_vec ? vec_bits(v) : 0u;
            uint32_t hit = 0u;
            if (bits) {
                vec_load(v, xv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) hit |= (((bits >> j) & 1u) && xv[j] >= thr_v && xv[j] <= FLT_MAX) ? 1u << j : 0u;
            }
            return hit;
        };
        // A thread whose maximum reaches the bound offers the hits of that vector: one round for the whole warp.  Only a
        // thread with a second vector that reaches the bound has all its vectors looked at.
        const bool holder = tmax >= thr_v;
        if (__any_sync(kFull, holder)) {
            float xv[VEC];
            offer_vec(holder ? hits_of(vmax_at, xv) : 0u, xv, vmax_at);
            // (its other vectors are taken by the lanes of the warp, one each: thread t owns vectors t, t + NT, ...)
            for (uint32_t rest = __ballot_sync(kFull, holder && tmax2 >= thr_v); rest; rest &= rest - 1u) {
                const int src = __ffs(rest) - 1;
                const int done = __shfl_sync(kFull, vmax_at, src);
#pragma unroll 1
                for (int q0 = 0; warp * 32 + src + q0 * NT < n_vec; q0 += 32) {
                    const int v = warp * 32 + src + (q0 + lane) * NT;
                    offer_vec(v != done ? hits_of(v, xv) : 0u, xv, v);
                }
            }
        }
        __syncthreads();
        // every CTA has its own region of CTA 0's buffer: plain remote stores, no reservation, no round trip
        uint32_t n_loc = sh.n_cand;
        const uint64_t * src = lbuf;
        if (no_bound && n_loc <= (uint32_t) kClusterLocal) {
            // No bound (a sparse mask left too few witnesses, and no CTA had k maxima of its own): every allowed id of
            // the row is a candidate.  Every CTA sends its own best k, sorted, at a distance of k: CTA 0 ranks their
            // union as it comes while that is small, and merges sixteen sorted lists when it is not.
            uint64_t * dst = gbuf0 + (size_t) rank * k;
            int got;
            if (n_loc <= (uint32_t) kRankSelectMax) {
                got = block_rank_select<NT>(lbuf, (int) n_loc, k, dst);
            } else {
                const uint64_t tau = block_kth_key<NT>(lbuf, (int) n_loc, k, sh.sc);
                got = block_take<NT>(lbuf, (int) n_loc, k, tau, lsel, sh.sc);
                block_rank_sort<NT>(lsel, got, dst);
            }
            for (int j = got + tid; j < k; j += NT) dst[j] = 0ull;
            if (tid == 0) cs0->region_n[rank] = (uint32_t) got;
        } else {
            if (n_loc > (uint32_t) kClusterRegion && n_loc <= (uint32_t) kClusterLocal) {
                // More than a region holds, but all of it is here: only this CTA's best k can matter, and k fits a region.
                int got;
                if (n_loc <= (uint32_t) kRankSelectMax) {
                    got = block_rank_select<NT>(lbuf, (int) n_loc, k, lsel);
                } else {
                    const uint64_t tau = block_kth_key<NT>(lbuf, (int) n_loc, k, sh.sc);
                    got = block_take<NT>(lbuf, (int) n_loc, k, tau, lsel, sh.sc);
                }
                __syncthreads();
                n_loc = (uint32_t) got;
                src = lsel;
            }
            if (tid == 0) cs0->region_n[rank] = n_loc;  // (still more than a region holds: the careful way follows)
            for (uint32_t i = tid; i < n_loc && i < (uint32_t) kClusterRegion; i += NT) gbuf0[(size_t) rank * kClusterRegion + i] = src[i];
        }
        __syncthreads();
        if (tid == 0) sh.n_cand = 0u;  // (the careful way starts from an empty buffer)
    }
    cluster.sync();

    // 6. CTA 0 finishes.  If its buffer overflowed, every CTA first reduces its slice to its own best k.
    uint32_t n_glob = 0u, n_most = 0u;
#pragma unroll
    for (int r = 0; r < kClusterCtas; ++r) {
        const uint32_t n = cs0->region_n[r];
        n_glob += n < (uint32_t) kClusterRegion ? n : (uint32_t) kClusterRegion;
        n_most = n > n_most ? n : n_most;
    }
    const bool careful = n_most > (uint32_t) kClusterRegion;  // the same answer in every CTA of the cluster
    if (careful) {
        // the careful walk: every vector offered to the CTA's own buffer, with a vote after every round
        thr_key = 0ull;
        thr_v = -FLT_MAX;
        const int trigger = kClusterLocal / 2;
        auto settle = [&](uint64_t key, bool & lost) {
            while (__syncthreads_or(lost || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) trigger)) {
                compact<NT>(lbuf, lsel, k, kClusterLocal, sh);
                const uint64_t tk = sh.thr_key;
                if (tk > thr_key) {
                    thr_key = tk;
                    thr_v = key_floor_value(tk);
                }
                if (lost && (key < thr_key || push(key, lbuf, sh, kClusterLocal))) lost = false;
                if (!__syncthreads_or(lost)) break;
            }
        };
        for (int j0 = 0; j0 < n_own; j0 += NT) {
            const uint64_t key = history_key(j0 + tid);
            bool lost = key != 0ull && key >= thr_key && !push(key, lbuf, sh, kClusterLocal);
            settle(key, lost);
        }
        for (int v0 = 0; v0 < n_vec; v0 += NT) {
            const int v = v0 + tid;
            const uint32_t bits = v < n_vec ? vec_bits(v) : 0u;
            float xv[VEC];
            if (bits) vec_load(v, xv);
#pragma unroll 1
            for (int j = 0; j < VEC; ++j) {  // one element per thread and vote
                uint64_t key = 0ull;
                if (((bits >> j) & 1u) && xv[j] >= thr_v && xv[j] <= FLT_MAX) key = make_key(xv[j], id0 + (uint32_t) (v * VEC + j));
                bool lost = key != 0ull && key >= thr_key && !push(key, lbuf, sh, kClusterLocal);
                settle(key, lost);
            }
        }
        __syncthreads();
        // the CTA's best k, sorted, into its place of CTA 0's buffer: [16][k]
        const int n = (int) min(sh.n_cand, (uint32_t) kClusterLocal);
        uint64_t * dst = gbuf0 + (size_t) rank * k;
        int got;
        if (n <= kRankSelectMax) {
            got = block_rank_select<NT>(lbuf, n, k, dst);
        } else {
            const uint64_t tau = block_kth_key<NT>(lbuf, n, k, sh.sc);
            got = block_take<NT>(lbuf, n, k, tau, lsel, sh.sc);
            block_rank_sort<NT>(lsel, got, dst);
        }
        for (int j = got + tid; j < k; j += NT) dst[j] = 0ull;
        cluster.sync();
    }
    if (rank == 0) {
        p.counter += (uint64_t) col;  // column c of a window draws with counter + c (src/engine.cu:756)
        int32_t * tok = a.out_tokens ? a.out_tokens + row : nullptr;
        fns_b200_cand * oc = a.out_cands ? a.out_cands + (size_t) row * a.k_cap : nullptr;
        int nk;
        if (careful || (no_bound && n_glob > (uint32_t) kClusterRankMax)) {  // sixteen sorted lists of k
            nk = merge_lists<NT>(gbuf, kClusterCtas, k, gsel, sorted, reinterpret_cast<uint64_t *>(pj), 2 * a.k_cap, sh.sc, k, a.k_cap);
        } else {
            // the regions side by side in the CTA's own buffer (sixteen threads per region), then the ordinary ranking
            const int n = (int) n_glob;
            {
                const int r = tid >> 4;
                uint32_t before = 0u;
                for (int q = 0; q < r; ++q) before += cs.region_n[q];
                const uint32_t cnt = cs.region_n[r];
                const int apart = no_bound ? k : kClusterRegion;  // (without a bound the CTAs sent lists of k)
                for (uint32_t i = (uint32_t) (tid & 15); i < cnt; i += 16u) lbuf[before + i] = gbuf[(size_t) r * apart + i];
                for (int j = tid; j < a.k_cap; j += NT) sorted[j] = 0ull;
                __syncthreads();
            }
            if (n <= kClusterRankMax) {
                nk = block_rank_select<NT>(lbuf, n, k, sorted);
            } else {
                const uint64_t tau = block_kth_key<NT>(lbuf, n, k, sh.sc);
                nk = block_take<NT>(lbuf, n, k, tau, gsel, sh.sc);
                block_rank_sort<NT>(gsel, nk, sorted);
            }
            __syncthreads();
        }
        draw_tail<NT>(sorted, nk, pj, acc, reinterpret_cast<double *>(gsel), sh.sc, p, a.k_cap, tok, oc);
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
}

}  // namespace fnsb
