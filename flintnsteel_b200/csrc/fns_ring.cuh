// fns_ring.cuh - k_ring: the select + draw kernel for whole rows in device memory (one 512-thread block per row).
// Included by fns_sampler.cu after the shared helpers (push, compact, draw_tail, ...).
//
// The row is moved by the copy engine, not by the threads: 1-D bulk asynchronous copies (cp.async.bulk, own-GPU
// global memory only, no multicast) fill a ring of stages in shared memory, each stage guarded by an mbarrier whose
// transaction count is the bytes under way.  The threads hold no row data in registers and the copies need nothing
// that the block computes, so the first stages are in flight while the block still builds its bit set and scatters
// the history.  A stage is 8,192 elements: 16 consecutive elements (a "cell") per thread.  Under a grammar mask a
// stage is copied in 512-element chunks (one warp's cells) and chunks without an allowed id are not copied at all.
// The kernel is launched with programmatic stream serialisation: its prologue overlaps the previous kernel's tail.
//
//   prefix   bit set = mask AND in-range (shared memory), chunk map, list of stages that have an allowed id;
//            every history id clears its bit and is listed once: its owner keeps it in a register and picks its logit
//            out of the ring when the stage passes (no gather from global memory)
//   stream   per stage and thread: the maximum of the cell's allowed elements.  The last warp to leave a stage
//            refills its slot with the stage `depth` places ahead; no block barrier is needed to run the ring.
//            Each maximum is kept as the upper 16 bits of its order word (rounded down) in shared memory, the
//            thread's own maximum in a register.  No flags, no running bound, no block barrier inside the loop:
//            taking candidates on the spot under a running bound was measured and is slower (the insertions
//            diverge inside the loop that feeds the ring).
//   bound    k <= 512: (nearly) the k-th largest thread maximum, found by one warp that holds sixteen maxima per lane
//            and decides two bits per step; larger k: the k-th largest of the threads' three best cell maxima, found
//            by counting with one block barrier per bit
//   pass 2   the cells that reach the bound (about k of them) are read again from L2 / HBM, element by element,
//            and the keys that reach the bound go to the candidate buffer together with the penalised history ids;
//            if equal values overflow the list or the buffer, every cell is offered again with votes and
//            compaction, so any input is handled exactly
//   select   the best k in the total order (up to 384 keys ranked by counting, more sorted by merging: runs of four
//            ordered in registers, then merge-path levels), then the draw (draw_tail)
#pragma once

namespace fnsb {

constexpr int kRingThreads = 512;
constexpr int kCell = 16;                           // elements per thread and stage
constexpr int kStageElems = kRingThreads * kCell;   // 8,192
constexpr int kChunkElems = 32 * kCell;             // 512: what one warp takes of a stage; the copy granule under a mask
constexpr int kMaxRingDepth = 8;
constexpr int kMaxRingStages = 64;                  // rows up to 524,288 elements

__device__ __forceinline__ uint32_t smem_addr(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
// Makes the initialised barriers visible to the copy engine (the async proxy).
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void async_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect(uint64_t * bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t * bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0u;
}
// Waits for the phase of the given parity.  Bounded: gives up after about half a second of polling and says so.
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try(bar, parity))
        if (clock64() - t0 > (1ll << 30)) return false;
    return true;
}
// bytes (a multiple of 16) from global to shared memory, counted on `bar` when they have landed
__device__ __forceinline__ void bulk_load(void * dst_shared, const void * src_global, uint32_t bytes, uint64_t * bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                     smem_addr(dst_shared)),
                 "l"(src_global), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// A bound for k beyond the thread count, from more witnesses per thread: every thread takes the three largest of
// its own cell maxima (cells are disjoint, so 3 * NT >= k different elements stand behind them), and the block finds
// the k-th largest of these 3 * NT values bit by bit from the top: one count per bit (three compares, a warp sum,
// one shared-memory add per warp, one barrier; three counters take turns so that none is cleared while it is read).
// At least k cells reach the result; a thread with more than three such cells adds a few more.  0 when there are
// fewer than k witnesses.  Cell of thread t in stage s at v[s * NT + t].
template <int NT>
__device__ uint32_t block_kth_witness(const uint16_t * v, int n_stages, int k, SelectScratch & sc) {
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t t0 = 0u, t1 = 0u, t2 = 0u;  // this thread's three largest cell maxima, t0 >= t1 >= t2
#pragma unroll 4
    for (int s = 0; s < n_stages; ++s) {
        const uint32_t x = v[s * NT + tid];
        const uint32_t a = max(t0, x), b = min(t0, x);
        const uint32_t c = max(t1, b), d = min(t1, b);
        t0 = a;
        t1 = c;
        t2 = max(t2, d);
    }
    if (tid < 3) sc.hist[tid] = 0u;
    __syncthreads();
    uint32_t prefix = 0u;
#pragma unroll 1
    for (int step = 0; step < 16; ++step) {
        const uint32_t cand = prefix | (0x8000u >> step);
        uint32_t cnt = (t0 >= cand ? 1u : 0u) + (t1 >= cand ? 1u : 0u) + (t2 >= cand ? 1u : 0u);
        cnt = __reduce_add_sync(kFull, cnt);
        uint32_t * slot = &sc.hist[step % 3];
        if (lane == 0 && cnt) atomicAdd(slot, cnt);
        __syncthreads();
        if (*(volatile uint32_t *) slot >= (uint32_t) k) prefix = cand;
        if (tid == 0) sc.hist[(step + 2) % 3] = 0u;  // the counter of step + 2: its readers of step - 1 are past this barrier
    }
    __syncthreads();
    return prefix;
}

// Merges sorted runs pairwise until one is left: `runs` runs of L keys each at a[r * L] (each descending, empty
// slots = 0 last), every key finding its place in the merged pair by a binary search in the sibling run (keys are
// distinct).  A merged run keeps its best `keep` keys only.  a and b alternate as source and destination; returns
// the buffer that holds the result and sets *len to its length.  All NT threads; block synchronised on entry and exit.
template <int NT>
__device__ uint64_t * merge_runs(uint64_t * a, uint64_t * b, int runs, int L, int keep, int * len) {
    while (runs > 1) {
        const int Lout = 2 * L < keep ? 2 * L : keep;
        const int out_runs = (runs + 1) >> 1;
        for (int i = threadIdx.x; i < out_runs * Lout; i += NT) b[i] = 0ull;
        __syncthreads();
        for (int idx = threadIdx.x; idx < runs * L; idx += NT) {
            const int r = idx / L, i = idx - r * L;
            const uint64_t key = a[idx];
            if (key == 0ull) continue;
            int pos = i;
            if ((r ^ 1) < runs) {  // (the last of an odd number of runs moves on as it is)
                const uint64_t * sib = a + (size_t) (r ^ 1) * L;
                int lo = 0, hi = L;
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (sib[mid] > key) lo = mid + 1;
                    else hi = mid;
                }
                pos += lo;
            }
            if (pos < Lout) b[(size_t) (r >> 1) * Lout + pos] = key;
        }
        __syncthreads();
        uint64_t * t = a;
        a = b;
        b = t;
        runs = out_runs;
        L = Lout;
    }
    *len = L;
    return a;
}

// C consecutive outputs, d0 .. d0 + C - 1, of the merge of two descending runs A[0 .. na) and B[0 .. nb) (distinct keys;
// an empty slot is 0 and sorts last): a binary search along the diagonal d0 finds how many of the first d0 outputs come
// from A, then the outputs are taken one by one.  Outputs at or beyond `limit` are not produced.
template <int C>
__device__ __forceinline__ void merge_chunk(const uint64_t * A, int na, const uint64_t * B, int nb, int d0, int limit,
                                            uint64_t * out) {
    int lo = d0 - nb > 0 ? d0 - nb : 0, hi = d0 < na ? d0 : na;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (A[mid] > B[d0 - mid - 1]) lo = mid + 1;
        else hi = mid;
    }
    int i = lo, j = d0 - lo;
    uint64_t x = i < na ? A[i] : 0ull, y = j < nb ? B[j] : 0ull;
#pragma unroll
    for (int t = 0; t < C; ++t) {
        if (d0 + t >= limit) break;
        const bool from_a = x > y || j >= nb;
        out[d0 + t] = from_a ? x : y;
        if (from_a) {
            ++i;
            x = i < na ? A[i] : 0ull;
        } else {
            ++j;
            y = j < nb ? B[j] : 0ull;
        }
    }
}

// Merges `runs` sorted runs of 1 << lg keys each (a power of two of them, side by side in a) pairwise until one is
// left, a merged run keeping its best `keep` keys (a power of two): every thread produces four consecutive keys of a
// merged run at a time.  a and b alternate as source and destination; returns the buffer that holds the result.
// All NT threads; block synchronised on entry and exit.
template <int NT>
__device__ uint64_t * merge_levels_pow2(uint64_t * a, uint64_t * b, int runs, int lg, int keep) {
    while (runs > 1) {
        const int L = 1 << lg;
        const int lg_out = 2 * L > keep ? lg : lg + 1;  // (a merged run of 2 L keys is cut back to keep = L)
        const int Lout = 1 << lg_out;
        const int chunks = ((runs >> 1) << lg_out) >> 2;
        for (int c = threadIdx.x; c < chunks; c += NT) {
            const int r = (c << 2) >> lg_out, d0 = (c << 2) & (Lout - 1);
            const uint64_t * A = a + ((size_t) (2 * r) << lg);
            merge_chunk<4>(A, L, A + L, L, d0, Lout, b + ((size_t) r << lg_out));
        }
        __syncthreads();
        uint64_t * t = a;
        a = b;
        b = t;
        runs >>= 1;
        lg = lg_out;
    }
    return a;
}

// Sorts a[0 .. m) (m a power of two, in shared memory) into descending order: a bitonic network, one barrier per
// step.  All NT threads; block synchronised on entry and exit.
template <int NT>
__device__ void block_sort_desc(uint64_t * a, int m) {
    for (int size = 2; size <= m; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < (m >> 1); i += NT) {
                const int lo = 2 * i - (i & (stride - 1));  // the pair (lo, lo + stride)
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const uint64_t x = a[lo], y = a[hi];
                if ((x < y) == desc) {
                    a[lo] = y;
                    a[hi] = x;
                }
            }
            __syncthreads();
        }
    }
}



constexpr int kRegOwn = 4;  // owned history ids that a thread keeps in registers (4 * 512 per row)

template <typename T>
__global__ void __launch_bounds__(kRingThreads, 2) k_ring(const SelectArgs a) {
    constexpr int NT = kRingThreads, kWarps = NT / 32;
    constexpr int VEC = 16 / (int) sizeof(T);   // elements per 16-byte vector
    constexpr int NVEC = kCell / VEC;           // vectors per cell
    constexpr uint32_t kVecBits = (1u << VEC) - 1u;
    constexpr int TS = 2 * NT;
    constexpr int kTShift = 22;                 // 32 - log2(TS)
    constexpr uint32_t kNoKey = 0xffffffffu;
    constexpr uint32_t kStageBytes = kStageElems * sizeof(T);
    constexpr uint32_t kChunkBytes = kChunkElems * sizeof(T);
    constexpr int kStageWords = kStageElems / 32;  // 256 mask words per stage
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x;
    const int W = a.n_draft + 1, win = row / W, col = row - win * W;
    const int V = a.vocab, n_stages = a.n_stages, depth = a.ring_depth;

    // shared memory: barriers, slot counters | SelectShared | chunk map | stage list | bit set | cell maxima |
    // owned history ids | ring, which later holds: candidate buffer | staging | sorted | p, acc | history logits |
    // occurrence table | work list
    uint64_t * full = reinterpret_cast<uint64_t *>(smem_raw);                    // [kMaxRingDepth]
    uint32_t * slot_done = reinterpret_cast<uint32_t *>(full + kMaxRingDepth);   // [kMaxRingDepth]
    SelectShared & sh = *reinterpret_cast<SelectShared *>(smem_raw + 128);
    constexpr size_t kShBytes = (sizeof(SelectShared) + 15) & ~(size_t) 15;
    uint16_t * chunk_bits = reinterpret_cast<uint16_t *>(smem_raw + 128 + kShBytes);  // [kMaxRingStages] bit c: chunk c of the stage has an allowed id
    uint16_t * stage_list = chunk_bits + kMaxRingStages;                         // [kMaxRingStages]
    uint32_t * eff = reinterpret_cast<uint32_t *>(stage_list + kMaxRingStages);  // [n_stages * 256]
    const uint16_t * eff16 = reinterpret_cast<const uint16_t *>(eff);            // the 16 bits of a cell
    uint16_t * cmax = reinterpret_cast<uint16_t *>(eff + n_stages * kStageWords);  // [n_stages * NT]
    uint32_t * own = reinterpret_cast<uint32_t *>(smem_raw + a.own_off);         // [own_cap]
    unsigned char * ring = smem_raw + a.ring_off;

    const T * x = reinterpret_cast<const T *>(a.logits) + (size_t) row * a.row_stride;
    const uint32_t id0 = (uint32_t) a.id_base;

    // What the copy of one stage moves: whole 16-byte vectors only (a ragged end is fetched with plain loads).
    auto issue_stage = [&](int s, int slot, uint32_t cb) {
        const int rem = V - s * kStageElems;
        const uint32_t avail = ((uint32_t) (rem < kStageElems ? rem : kStageElems) * (uint32_t) sizeof(T)) & ~15u;
        unsigned char * dst = ring + (size_t) slot * kStageBytes;
        const unsigned char * src = reinterpret_cast<const unsigned char *>(x + (size_t) s * kStageElems);
        uint32_t total = 0u;
        if (cb == 0xffffu) {
            if (avail) bulk_load(dst, src, avail, &full[slot]);
            total = avail;
        } else {
            for (uint32_t q = cb; q; q &= q - 1u) {
                const uint32_t off = (uint32_t) (__ffs(q) - 1) * kChunkBytes;
                if (off >= avail) break;
                const uint32_t n = avail - off < kChunkBytes ? avail - off : kChunkBytes;
                bulk_load(dst + off, src + off, n, &full[slot]);
                total += n;
            }
        }
        mbar_arrive_expect(&full[slot], total);
    };

    if (tid < kWarps) sh.warp_top[tid] = 0u;
    if (tid == 0) {
        for (int d = 0; d < depth; ++d) {
            mbar_init(&full[d], 1u);
            slot_done[d] = 0u;
        }
        mbar_init_fence();
        sh.n_cand = 0u;
        sh.thr_key = 0ull;
        sh.n_own = 0u;
        sh.n_vl = 0u;
        sh.n_seg = 0u;
    }
    // 1. The bit set (bit e: element e is allowed and inside the row), the chunk map and the list of stages that have
    // an allowed id.  A chunk is 16 words = 4 neighbouring lanes, so a warp covers 8 chunks of one stage and writes
    // their bits as one byte: no atomics.  (Doing this ahead of the dependency wait for rows without a mask was
    // measured: it slows the previous kernel's tail on the same SM by more than it saves.)
    auto build_bits = [&](const uint32_t * mrow) {
        {
            const int words = (V + 31) >> 5;
            const int eff_words = n_stages * kStageWords;
            const uint32_t tail = (V & 31) ? (1u << (V & 31)) - 1u : 0xffffffffu;
            const bool wide = mrow && (reinterpret_cast<uintptr_t>(mrow) & 15u) == 0;
            constexpr int IT = 4;  // rounds whose loads are all issued before the first is used (rows up to 262,144)
            auto fetch = [&](int w0, uint32_t (&m)[4]) {
                if (!mrow) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) m[q] = w0 + q < words ? 0xffffffffu : 0u;
                } else if (wide && w0 + 4 <= words) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(mrow + w0);
                    m[0] = v.x;
                    m[1] = v.y;
                    m[2] = v.z;
                    m[3] = v.w;
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) m[q] = w0 + q < words ? mrow[w0 + q] : 0u;
                }
            };
            auto settle = [&](int w0, uint32_t (&m)[4]) {  // (every lane of the warp is here: eff_words is a multiple of 128)
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (w0 + q == words - 1) m[q] &= tail;
                *reinterpret_cast<uint4 *>(eff + w0) = make_uint4(m[0], m[1], m[2], m[3]);
                const uint32_t b = __ballot_sync(kFull, (m[0] | m[1] | m[2] | m[3]) != 0u);
                if (lane == 0) {
                    uint32_t c8 = 0u;
#pragma unroll
                    for (int c = 0; c < 8; ++c) c8 |= ((b >> (4 * c)) & 15u) ? (1u << c) : 0u;
                    reinterpret_cast<uint8_t *>(chunk_bits)[w0 >> 7] = (uint8_t) c8;  // byte = 128 words = half a stage
                }
            };
            uint32_t mw[IT][4];
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int w0 = (it * NT + tid) * 4;
                if (w0 < eff_words) fetch(w0, mw[it]);
            }
#pragma unroll
            for (int it = 0; it < IT; ++it) {
                const int w0 = (it * NT + tid) * 4;
                if (w0 < eff_words) settle(w0, mw[it]);
            }
            for (int w0 = (IT * NT + tid) * 4; w0 < eff_words; w0 += NT * 4) {
                uint32_t m[4];
                fetch(w0, m);
                settle(w0, m);
            }
        }
        {
            uint4 * z = reinterpret_cast<uint4 *>(cmax);
            for (int i = tid; i < n_stages * NT / 8; i += NT) z[i] = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    auto list_stages = [&](const uint32_t * mrow) {  // warp 0; with a mask the first copies start here
        if (warp == 0) {
            const uint32_t below = (1u << lane) - 1u;
            int base = 0;
            for (int s0 = 0; s0 < n_stages; s0 += 32) {
                const int s = s0 + lane;
                const bool live = s < n_stages && chunk_bits[s] != 0u;
                const uint32_t b = __ballot_sync(kFull, live);
                if (live) stage_list[base + __popc(b & below)] = (uint16_t) s;
                base += __popc(b);
            }
            if (lane == 0) sh.n_seg = (uint32_t) base;
            __syncwarp();
            if (lane == 0 && mrow)
                for (int u = 0; u < depth && u < base; ++u) issue_stage(stage_list[u], u, chunk_bits[stage_list[u]]);
        }
    };
    // Launched with programmatic stream serialisation: this block may start while the previous kernel of the stream
    // still drains, and the next kernel's blocks may take the places of blocks that have exited (they wait here
    // too).  Nothing is read from global memory before the previous kernel has finished.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const uint32_t * mrow = a.masks ? a.masks + (size_t) (a.mask_rows ? a.mask_rows[row] : row) * a.mask_stride : nullptr;
    // without a mask every chunk is wanted: the first stages start now
    if (tid == 0 && !mrow)
        for (int u = 0; u < depth && u < n_stages; ++u) issue_stage(u, u, 0xffffu);
    // Everything whose address is known is requested before anything is waited for.
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
    build_bits(mrow);
    const int k = p.temperature <= 0.0f ? 1 : clamp_k(p.top_k, a.k_cap);
    const bool any_pen = p.repetition != 1.0f || p.presence != 0.0f || p.frequency != 0.0f;
    const bool use_hist = any_pen && a.own_cap > 0;
    n_hist = n_hist < 0 ? 0 : (n_hist > (int) a.history_stride ? (int) a.history_stride : n_hist);
    const int n_pen = n_hist + (a.draft ? col : 0);
    __syncthreads();
    list_stages(mrow);

    // 2. Penalties: every history id (plus the draft prefix of a verification column) clears its bit, so the
    // streaming pass never counts it; the thread that finds the bit still set owns the id and lists it once.
    if (use_hist && n_pen > 0) {
        const uint32_t below = (1u << lane) - 1u;
        for (int j0 = 0; j0 < n_pen; j0 += NT * 4) {
            int32_t ids[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * NT + tid;
                if (j0 == 0 && hrow) ids[u] = j < n_hist ? ids0[u] : (j < n_pen ? drow[j - n_hist] : -1);
                else ids[u] = j < n_hist ? hrow[j] : (j < n_pen ? drow[j - n_hist] : -1);
            }
            // (the steps are kept apart - plain reads of the bit set, then the atomics, then the votes - because an atomic
            // in between would keep the compiler from moving the later reads ahead of it)
            uint32_t offs[4], seen[4], pre[4], total = 0u;
            bool mine[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                offs[u] = (uint32_t) (ids[u] - a.id_base);
                seen[u] = (offs[u] < (uint32_t) V && ids[u] >= a.id_base) ? eff[offs[u] >> 5] : 0u;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t bit = 1u << (offs[u] & 31);
                // (a plain read came first: a stale 1 is settled by the atomic itself, and a 0 stays 0)
                mine[u] = (seen[u] & bit) && (atomicAnd(&eff[offs[u] >> 5], ~bit) & bit) != 0u;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t b = __ballot_sync(kFull, mine[u]);
                pre[u] = total + (uint32_t) __popc(b & below);
                total += (uint32_t) __popc(b);
            }
            if (total == 0u) continue;  // uniform per warp
            uint32_t base = 0u;
            if (lane == 0) base = atomicAdd(&sh.n_own, total);
            base = __shfl_sync(kFull, base, 0);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (mine[u]) own[base + pre[u]] = offs[u];
        }
    }
    // The row's ragged end (less than one 16-byte vector): out of the bit set, offered as keys of their own.
    uint64_t rag_key = 0ull;
    if ((V % VEC) != 0 && tid < (V % VEC)) {
        const int e = V - (V % VEC) + tid;
        const uint32_t bit = 1u << (e & 31);
        if (atomicAnd(&eff[e >> 5], ~bit) & bit) {
            const float xi = to_float(x[e]);
            if (is_finite(xi)) rag_key = make_key(xi, id0 + (uint32_t) e);
        }
    }
    __syncthreads();
    const int n_own = use_hist ? (int) sh.n_own : 0;
    const int n_live = (int) sh.n_seg;
    // The first 4 * NT owned ids stay in registers, one per thread and round: their logits are picked out of the ring
    // when their stage passes through, so no history id costs a gather from global memory.
    uint32_t my_off[kRegOwn], my_val[kRegOwn];
#pragma unroll
    for (int r = 0; r < kRegOwn; ++r) {
        const int j = r * NT + tid;
        my_off[r] = j < n_own ? own[j] : 0xffffffffu;
        my_val[r] = 0u;
    }

    // 3. The streaming pass.
    float tmax = -INFINITY;     // this thread's maximum so far
    uint64_t best = 0ull;       // k == 1: this thread's best key
    bool gave_up = false;
    {
        const int f = (lane >> (NVEC == 4 ? 1 : 2)) & (NVEC - 1);  // the order in which a lane takes its vectors: no bank conflicts
        // The cell of this thread in the slot: its maximum over the allowed, finite elements (-inf if none).
        auto scan_cell = [&](const unsigned char * cell, uint32_t bits) -> float {
            float m = -INFINITY;
            float xv[NVEC][VEC];
#pragma unroll
            for (int j = 0; j < NVEC; ++j) {
                const int v = j ^ f;
                const uint4 raw = *reinterpret_cast<const uint4 *>(cell + v * 16);
                if constexpr (sizeof(T) == 4) {
                    xv[j][0] = __uint_as_float(raw.x);
                    xv[j][1] = __uint_as_float(raw.y);
                    xv[j][2] = __uint_as_float(raw.z);
                    xv[j][3] = __uint_as_float(raw.w);
                } else {
                    const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        xv[j][2 * q] = __uint_as_float(w4[q] << 16);
                        xv[j][2 * q + 1] = __uint_as_float(w4[q] & 0xffff0000u);
                    }
                }
                if (bits == 0xffffu) {  // the whole cell is allowed: nothing but maxima (the same in all 16 elements' bits)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) m = fmaxf(m, xv[j][e]);
                } else {
                    const uint32_t vb = bits >> (v * VEC);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) m = fmaxf(m, ((vb >> e) & 1u) ? xv[j][e] : -INFINITY);
                }
            }
            if (__builtin_expect(!(m <= FLT_MAX), 0)) {  // +inf among the allowed: never a candidate (src/kernels.cu:629-639)
                m = -INFINITY;
#pragma unroll
                for (int j = 0; j < NVEC; ++j) {
                    const uint32_t vb = bits >> ((j ^ f) * VEC);
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        if (((vb >> e) & 1u) && xv[j][e] <= FLT_MAX) m = fmaxf(m, xv[j][e]);
                }
            }
            return m;
        };
        int slot = 0;
        uint32_t parity = 0u;
        for (int u = 0; u < n_live; ++u) {
            const int s = stage_list[u];
            const uint32_t bits = eff16[s * NT + tid];
            if (!mbar_wait(&full[slot], parity)) gave_up = true;
            if (n_own > 0) {  // uniform
                const T * stage_base = reinterpret_cast<const T *>(ring + (size_t) slot * kStageBytes);
#pragma unroll
                for (int r = 0; r < kRegOwn; ++r) {
                    if ((int) (my_off[r] >> 13) == s) {  // (kStageElems = 2^13)
                        const T xe = stage_base[my_off[r] & (kStageElems - 1)];
                        if constexpr (sizeof(T) == 4) my_val[r] = __float_as_uint(xe);
                        else my_val[r] = __float_as_uint(__bfloat162float(xe));
                    }
                }
            }
            const unsigned char * cell = ring + (size_t) slot * kStageBytes + (size_t) tid * (kCell * sizeof(T));
            float m = -INFINITY;
            if (bits) m = scan_cell(cell, bits);  // (a chunk that was not copied has no bits)
            if (m > -INFINITY) {
                tmax = fmaxf(tmax, m);
                cmax[s * NT + tid] = (uint16_t) (order_word(m) >> 16);
            }
            // the last warp to leave the stage refills the slot
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                if (atomicAdd(&slot_done[slot], 1u) == (uint32_t) kWarps - 1u) {
                    slot_done[slot] = 0u;
                    if (u + depth < n_live) {
                        async_proxy_fence();
                        const int s2 = stage_list[u + depth];
                        issue_stage(s2, slot, chunk_bits[s2]);
                    }
                }
            }
            if (++slot == depth) {
                slot = 0;
                parity ^= 1u;
            }
        }
    }
    if (gave_up && a.err) atomicExch(a.err, 3);  // a copy never arrived: the result of this row is not valid
    __syncthreads();  // the ring is free: what follows lives there

    uint64_t * buf = reinterpret_cast<uint64_t *>(ring);
    uint64_t * sel = buf + a.cap;
    uint64_t * sorted = sel + a.k_cap;
    double * pj = reinterpret_cast<double *>(sorted + a.k_cap);
    double * acc = pj + a.k_cap;
    uint32_t * oval = reinterpret_cast<uint32_t *>(acc + a.k_cap);  // [own_cap] logit words of the owned ids beyond the registers
    uint32_t * tkey = oval + a.own_cap;                             // [TS] offsets whose occurrences are counted
    uint32_t * tcnt = tkey + TS;                                    // [TS]
    uint32_t * vlist = tcnt + TS;                                   // [list_cap] cells to read again

    for (int i = tid; i < TS; i += NT) {
        tkey[i] = kNoKey;
        tcnt[i] = 0u;
    }
    for (int j = kRegOwn * NT + tid; j < n_own; j += NT) copy_word_async(&oval[j], word_of(x + own[j]));  // (a very long history)
    if ((V % VEC) != 0) {  // an owned id in the row's ragged end never passed through the ring
#pragma unroll
        for (int r = 0; r < kRegOwn; ++r)
            if (my_off[r] != 0xffffffffu && my_off[r] >= (uint32_t) (V - V % VEC)) my_val[r] = __float_as_uint(to_float(x[my_off[r]]));
    }

    // 4. The bound: a value that at least k allowed, unpenalised elements reach.
    float thr_v = -FLT_MAX;
    if (k <= NT) {
        // The k-th largest of the threads' maxima (k == 1: the largest).  One warp does it without block barriers:
        // every lane takes sixteen maxima, the bits in which they differ are found first, and the search decides up
        // to 14 bits from the highest of them downwards, two bits per step with three warp-wide counts that do not
        // wait for one another; it stops early once at most four maxima too many remain.
        uint32_t * wtop = vlist;  // [NT] (the work list is filled later)
        wtop[tid] = tmax > -INFINITY ? order_word(tmax) : 0u;
        __syncthreads();
        if (warp == 0) {
            uint32_t w[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 v = *reinterpret_cast<const uint4 *>(&wtop[lane * 16 + q * 4]);
                w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
            }
            uint32_t wo = 0u, wa = 0xffffffffu, have = 0u, top1 = 0u;
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                if (w[q] != 0u) {
                    wo |= w[q];
                    wa &= w[q];
                    ++have;
                }
                top1 = max(top1, w[q]);
            }
            wo = __reduce_or_sync(kFull, wo);
            wa = __reduce_and_sync(kFull, wa);
            have = __reduce_add_sync(kFull, have);
            uint32_t bw = 0u;
            if (k == 1) {
                bw = __reduce_max_sync(kFull, top1);
            } else if (have >= (uint32_t) k) {  // else: fewer than k threads have seen anything, no bound
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
                        for (int q = 0; q < 16; ++q) {
                            c1 += w[q] >= (bw | b1) ? 1u : 0u;
                            c10 += w[q] >= (bw | b1 | b0) ? 1u : 0u;
                            c0 += w[q] >= (bw | b0) ? 1u : 0u;
                        }
                        c1 = __reduce_add_sync(kFull, c1);
                        c10 = __reduce_add_sync(kFull, c10);
                        c0 = __reduce_add_sync(kFull, c0);
                        uint32_t tot = 0xffffffffu;
                        if (c10 >= (uint32_t) k) bw |= b1 | b0, tot = c10;
                        else if (c1 >= (uint32_t) k) bw |= b1, tot = c1;
                        else if (c0 >= (uint32_t) k) bw |= b0, tot = c0;
                        if (tot <= (uint32_t) k + 4u) break;
                    }
                }
            }
            if (lane == 0) sh.warp_top[0] = bw;
        }
        __syncthreads();
        const uint32_t bw = sh.warp_top[0];
        if (bw != 0u) thr_v = word_value(bw) + 0.0f;  // (-0.0 -> +0.0: one key pattern for both zeros)
        __syncthreads();  // (the work list's words are written next)
    } else {
        static_assert(FNS_B200_MAX_K <= 3 * NT, "three witnesses per thread cover the largest k");
        const uint32_t b = block_kth_witness<NT>(cmax, n_stages, k, sh.sc);
        if (b >= 0x0080u) thr_v = word_value(b << 16);
        thr_v += 0.0f;
    }
    uint64_t thr_key = (uint64_t) order_word(thr_v) << 32;

    // 5. The candidates.
    auto penalised = [&](float v, float cnt) -> float {  // each step rounded on its own: no fused multiply-add
        v = v > 0.0f ? __fdiv_rn(v, p.repetition) : __fmul_rn(v, p.repetition);
        v = __fsub_rn(v, __fmul_rn(p.frequency, cnt));
        return __fsub_rn(v, p.presence);
    };
    {
        // the cells of this thread that reach the bound go on the work list
        const uint32_t b16 = max((uint32_t) (thr_key >> 48), 1u);
        uint64_t qual = 0ull;  // bit s: this thread's cell of stage s reaches the bound (a stage that was not streamed holds zeros)
        if (tmax >= thr_v) {
#pragma unroll 8
            for (int s = 0; s < n_stages; ++s) qual |= (uint64_t) ((uint32_t) cmax[s * NT + tid] >= b16 ? 1u : 0u) << s;
        }
        const int mine_n = __popcll(qual);
        if (__ballot_sync(kFull, mine_n != 0)) {  // one reservation per warp
            int upto = mine_n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(kFull, upto, o);
                if (lane >= o) upto += t;
            }
            uint32_t at = 0u;
            if (lane == 31) at = atomicAdd(&sh.n_vl, (uint32_t) upto);
            at = __shfl_sync(kFull, at, 31) + (uint32_t) (upto - mine_n);
            for (uint64_t q = qual; q; q &= q - 1ull) {
                if (at < (uint32_t) a.list_cap) vlist[at] = (uint32_t) (__ffsll((long long) q) - 1) * NT + (uint32_t) tid;
                ++at;
            }
        }
    }
    copy_word_wait();
    __syncthreads();
    for (int attempt = 0; attempt < 2; ++attempt) {
        const bool careful = attempt == 1;
        // (a) the ragged end
        if (rag_key != 0ull) {
            if (k == 1) best = rag_key > best ? rag_key : best;
            else if (rag_key >= thr_key) push(rag_key, buf, sh, a.cap);
        }
        // (b) the owned history ids with their penalised values; occurrences are counted only for ids whose value
        // with one occurrence reaches the bound (unless more occurrences raise the value)
        if (n_own > 0) {
            const bool counts = p.frequency != 0.0f;
            const bool count_all = p.frequency < 0.0f;  // then more occurrences raise the value
            // the block walks the history once and counts the occurrences of the offsets that sit in the table
            auto count_occurrences = [&]() {
                for (int t = tid; t < n_pen; t += NT) {
                    const int32_t id = t < n_hist ? hrow[t] : drow[t - n_hist];
                    const uint32_t o = (uint32_t) (id - a.id_base);
                    if (o >= (uint32_t) V || id < a.id_base) continue;
                    uint32_t h = (o * 2654435761u) >> kTShift;
                    for (uint32_t kx = tkey[h]; kx != kNoKey; kx = tkey[h]) {  // at most NT keys in 2 * NT slots
                        if (kx == o) {
                            atomicAdd(&tcnt[h], 1u);
                            break;
                        }
                        h = (h + 1u) & (TS - 1);
                    }
                }
            };
            auto table_insert = [&](uint32_t off) -> uint32_t {  // owned ids are distinct: every insert claims an empty slot
                uint32_t slot = (off * 2654435761u) >> kTShift;
                while (atomicCAS(&tkey[slot], kNoKey, off) != kNoKey) slot = (slot + 1u) & (TS - 1);
                return slot;
            };
            const int rounds = (n_own + NT - 1) / NT;
#pragma unroll 1
            for (int r0 = 0; r0 < rounds; r0 += kRegOwn) {  // kRegOwn ids per thread at a time
                uint32_t off[kRegOwn], slot[kRegOwn], live = 0u;
                float raw[kRegOwn], v[kRegOwn];
#pragma unroll
                for (int r = 0; r < kRegOwn; ++r) {
                    const int j = (r0 + r) * NT + tid;
                    off[r] = 0u;
                    raw[r] = 0.0f;
                    v[r] = -INFINITY;
                    slot[r] = 0u;
                    if (j < n_own) {
                        off[r] = r0 == 0 ? my_off[r] : own[j];
                        raw[r] = r0 == 0 ? __uint_as_float(my_val[r]) : value_in_word(oval[j], x + off[r]);
                        v[r] = penalised(raw[r], 1.0f);
                        if (count_all || v[r] >= thr_v) live |= 1u << r;
                    }
                }
                if (counts) {
                    // how many ids need their occurrences (at most kRegOwn per thread that has one): usually a handful,
                    // then one walk serves them all
                    const uint32_t total = (uint32_t) __syncthreads_count(live != 0u) * kRegOwn;
                    if (total != 0u && total <= (uint32_t) NT) {
#pragma unroll
                        for (int r = 0; r < kRegOwn; ++r)
                            if ((live >> r) & 1u) slot[r] = table_insert(off[r]);
                        __syncthreads();
                        count_occurrences();
                        __syncthreads();
#pragma unroll
                        for (int r = 0; r < kRegOwn; ++r) {
                            if ((live >> r) & 1u) {
                                v[r] = penalised(raw[r], (float) tcnt[slot[r]]);
                                tkey[slot[r]] = kNoKey;
                                tcnt[slot[r]] = 0u;
                            }
                        }
                    } else if (total != 0u) {  // more than the table takes at once: round by round
#pragma unroll 1
                        for (int r = 0; r < kRegOwn; ++r) {
                            const bool lv = (live >> r) & 1u;
                            if (!__syncthreads_or(lv)) continue;
                            uint32_t sl = 0u;
                            if (lv) sl = table_insert(off[r]);
                            __syncthreads();
                            count_occurrences();
                            __syncthreads();
                            if (lv) {
                                const float vv = penalised(raw[r], (float) tcnt[sl]);
#pragma unroll
                                for (int q = 0; q < kRegOwn; ++q)
                                    if (q == r) v[q] = vv;
                                tkey[sl] = kNoKey;
                                tcnt[sl] = 0u;
                            }
                        }
                    }
                }
                uint64_t key[kRegOwn];
                uint32_t lost = 0u;
#pragma unroll
                for (int r = 0; r < kRegOwn; ++r) {
                    key[r] = (((live >> r) & 1u) && is_finite(v[r])) ? make_key(v[r], id0 + off[r]) : 0ull;
                    if (key[r] != 0ull) {
                        if (k == 1) best = key[r] > best ? key[r] : best;
                        else if (key[r] >= thr_key && !push(key[r], buf, sh, a.cap)) lost |= 1u << r;
                    }
                }
                if (careful && k > 1 && n_own + VEC > a.trigger) {  // uniform: only a long list can fill the buffer
                    while (__syncthreads_or(lost != 0u || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                        compact<NT>(buf, sel, k, a.cap, sh);
                        const uint64_t tk = sh.thr_key;
                        if (tk > thr_key) {
                            thr_key = tk;
                            thr_v = key_floor_value(tk);
                        }
#pragma unroll
                        for (int r = 0; r < kRegOwn; ++r)
                            if (((lost >> r) & 1u) && (key[r] < thr_key || push(key[r], buf, sh, a.cap))) lost &= ~(1u << r);
                        if (!__syncthreads_or(lost != 0u)) break;
                    }
                }
            }
        }
        // (c) the listed cells, one vector per thread and round, read again.  The careful way walks every cell
        // instead, a round of NT cells at a time, with a vote after each round.
        bool listed = true;
        if (!careful) {
            {
                const int n_work = (int) sh.n_vl;
                listed = n_work <= a.list_cap;  // uniform
                const int total = listed ? n_work * NVEC : 0;
                constexpr int PB = sizeof(T) == 2 ? 4 : 2;  // items per thread whose loads are in flight together (kept as raw 16-byte words)
#pragma unroll 1
                for (int i0 = warp * 32; i0 < total; i0 += PB * NT) {  // (the same rounds for every lane of a warp)
                    uint4 raw[PB];
                    uint32_t bits[PB], e0[PB];
#pragma unroll
                    for (int q = 0; q < PB; ++q) {
                        const int i = i0 + q * NT + lane;
                        bits[q] = 0u;
                        e0[q] = 0u;
                        if (i < total) {
                            const uint32_t cell = vlist[i / NVEC];
                            const int v = i % NVEC;
                            bits[q] = ((uint32_t) eff16[cell] >> (v * VEC)) & kVecBits;
                            e0[q] = cell * kCell + (uint32_t) (v * VEC);
                            if (bits[q]) raw[q] = __ldg(reinterpret_cast<const uint4 *>(x + e0[q]));
                        }
                    }
#pragma unroll
                    for (int q = 0; q < PB; ++q) {
                        uint32_t hit = 0u;  // the elements of this vector that reach the bound
                        float xq[VEC];
                        if (bits[q]) {
                            if constexpr (sizeof(T) == 4) {
                                xq[0] = __uint_as_float(raw[q].x);
                                xq[1] = __uint_as_float(raw[q].y);
                                xq[2] = __uint_as_float(raw[q].z);
                                xq[3] = __uint_as_float(raw[q].w);
                            } else {
                                const uint32_t w4[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    xq[2 * j] = __uint_as_float(w4[j] << 16);
                                    xq[2 * j + 1] = __uint_as_float(w4[j] & 0xffff0000u);
                                }
                            }
#pragma unroll
                            for (int j = 0; j < VEC; ++j)
                                hit |= (((bits[q] >> j) & 1u) && xq[j] >= thr_v && xq[j] <= FLT_MAX) ? 1u << j : 0u;
                        }
                        if (k == 1) {
#pragma unroll
                            for (int j = 0; j < VEC; ++j) {
                                if (!((hit >> j) & 1u)) continue;
                                const uint64_t key = make_key(xq[j], id0 + e0[q] + (uint32_t) j);
                                best = key > best ? key : best;
                            }
                            continue;
                        }
                        if (!__ballot_sync(kFull, hit != 0u)) continue;
                        const uint32_t mine_n = (uint32_t) __popc(hit);  // one reservation per warp
                        uint32_t upto = mine_n;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const uint32_t t = __shfl_up_sync(kFull, upto, o);
                            if (lane >= o) upto += t;
                        }
                        uint32_t at = 0u;
                        if (lane == 31) at = atomicAdd(&sh.n_cand, upto);
                        at = __shfl_sync(kFull, at, 31) + upto - mine_n;
#pragma unroll
                        for (int j = 0; j < VEC; ++j) {
                            if (!((hit >> j) & 1u)) continue;
                            if (at < (uint32_t) a.cap) buf[at] = make_key(xq[j], id0 + e0[q] + (uint32_t) j);
                            ++at;
                        }
                    }
                }
            }
        } else {
#pragma unroll 1
            for (int base = 0; base < n_stages * NT; base += NT) {
                const uint32_t cell = (uint32_t) (base + tid);
                uint32_t lost = 0u;
                const uint32_t c = cmax[cell];
                const uint32_t bits = (c != 0u && c >= (uint32_t) (thr_key >> 48)) ? (uint32_t) eff16[cell] : 0u;
                if (bits) {
#pragma unroll
                    for (int v = 0; v < NVEC; ++v) {
                        const uint32_t vb = (bits >> (v * VEC)) & kVecBits;
                        if (!vb) continue;
                        const uint32_t e = cell * kCell + (uint32_t) (v * VEC);
                        float xv[VEC];
                        load_vec<T, VEC>(x + e, xv);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) {
                            if (!(((vb >> j) & 1u) && xv[j] >= thr_v && xv[j] <= FLT_MAX)) continue;
                            const uint64_t key = make_key(xv[j], id0 + e + (uint32_t) j);
                            if (k == 1) best = key > best ? key : best;
                            else if (key >= thr_key && !push(key, buf, sh, a.cap)) lost |= 1u << (v * VEC + j);
                        }
                    }
                }
                if (k == 1) continue;
                while (__syncthreads_or(lost != 0u || *(volatile uint32_t *) &sh.n_cand >= (uint32_t) a.trigger)) {
                    compact<NT>(buf, sel, k, a.cap, sh);
                    const uint64_t tk = sh.thr_key;
                    if (tk > thr_key) {
                        thr_key = tk;
                        thr_v = key_floor_value(tk);
                    }
                    uint32_t still = 0u;
                    for (uint32_t q = lost; q; q &= q - 1u) {
                        const int b = __ffs(q) - 1;
                        const uint32_t e = cell * kCell + (uint32_t) b;
                        const uint64_t key = make_key(to_float(x[e]), id0 + e);
                        if (key >= thr_key && !push(key, buf, sh, a.cap)) still |= 1u << b;
                    }
                    lost = still;
                    if (!__syncthreads_or(lost != 0u)) break;
                }
            }
        }
        __syncthreads();
        if (attempt == 1 || (listed && (k == 1 || sh.n_cand <= (uint32_t) a.cap))) break;  // uniform: all is in
        // the list or the buffer overflowed (many equal values): again from an empty buffer, the careful way
        __syncthreads();
        if (tid == 0) sh.n_cand = 0u;
        best = 0ull;
        __syncthreads();
    }

    // 6. The best k in the total order, and the draw.
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
            if (tok) *tok = b ? key_id(b) : -1;
            if (oc) oc[0] = key_to_cand(b);
        }
        if (oc)
            for (int j = 1 + tid; j < a.k_cap; j += NT) oc[j] = key_to_cand(0ull);
        return;
    }
    const int n = (int) min(sh.n_cand, (uint32_t) a.cap);
    int got;
    int pow2_runs = 1;  // runs of four keys that cover the buffer's contents, a power of two of them
    while (4 * pow2_runs < n) pow2_runs <<= 1;
    if (n <= kRankSelectMax) {
        got = block_rank_select<NT>(buf, n, k, sorted);
    } else if (8 * pow2_runs <= a.cap) {
        // a long list (k beyond 384): sorted as it is, by merging.  Every thread orders four keys in registers, the
        // runs of four (a power of two of them: empty runs fill up) are merged pairwise in the two halves of the
        // buffer, and the best k of the result are the answer.
        const int half = a.cap / 2;
        const int runs = pow2_runs;
        for (int r = tid; r < runs; r += NT) {
            uint64_t q[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) q[e] = 4 * r + e < n ? buf[4 * r + e] : 0ull;
            auto order = [&](int i, int j) {
                if (q[i] < q[j]) {
                    const uint64_t t = q[i];
                    q[i] = q[j];
                    q[j] = t;
                }
            };
            order(0, 1);
            order(2, 3);
            order(0, 2);
            order(1, 3);
            order(1, 2);
#pragma unroll
            for (int e = 0; e < 4; ++e) buf[4 * r + e] = q[e];
        }
        __syncthreads();
        int keep = 4;  // a merged run keeps the best `keep` keys: the power of two that holds k
        while (keep < k) keep <<= 1;
        const uint64_t * res = merge_levels_pow2<NT>(buf, buf + half, runs, 2, keep);
        got = n < k ? n : k;
        for (int i = tid; i < got; i += NT) sorted[i] = res[i];
    } else {
        const uint64_t tau = block_kth_key<NT>(buf, n, k, sh.sc);
        got = block_take<NT>(buf, n, k, tau, sel, sh.sc);
        if (got <= kRankSelectMax) {
            block_rank_sort<NT>(sel, got, sorted);
        } else {  // (buffer nearly full of keys that all matter: a sorting network over the selected ones)
            int m = 1;
            while (m < got) m <<= 1;
            for (int i = tid; i < m; i += NT) buf[i] = i < got ? sel[i] : 0ull;  // (m <= 2 * k_cap <= cap)
            __syncthreads();
            block_sort_desc<NT>(buf, m);
            for (int i = tid; i < got; i += NT) sorted[i] = buf[i];
        }
    }
    for (int j = got + tid; j < a.k_cap; j += NT) sorted[j] = 0ull;
    __syncthreads();
    draw_tail<NT>(sorted, got, pj, acc, reinterpret_cast<double *>(sel), sh.sc, p, a.k_cap, tok, oc);
}

}  // namespace fnsb
