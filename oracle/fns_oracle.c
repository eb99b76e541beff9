/* fns_oracle.c - CPU restatement of the FlintNSteel logits -> token sampler.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with and the
 * CPU baseline that the benchmark times; the shipped library never links, loads or calls it.
 *
 * Every function cites the reference lines it restates (paths are relative to the
 * NomenAK/FlintNSteel source tree):
 *   - total order and eligibility ......... src/kernels.cu:624-648 (k_topk_part), :605-622 (block_best)
 *   - Philox variant ...................... src/kernels.cu:652-665 (philox_uniform)
 *   - candidate softmax / top-p / draw .... src/kernels.cu:698-720 (tail of k_sample)
 *   - k clamp ............................. src/kernels.cu:778
 *   - presence penalty .................... src/kernels.cu:724-727, :735-742
 *   - host reference distribution ......... tests/sample_check.cu:38-57
 *   - speculative accept rule ............. tools/fns_serve/fns_serve.cpp:492-508,
 *                                           tools/fns_verify/fns_verify.cpp:267-278
 *
 * Parity status.  Pinned: selection order, eligibility, top-p cut, temperature weights, draw and the
 * accept rule, against (a) the known answers of tests/sample_check.cu and (b) outputs of the reference's
 * own kernels recompiled for sm_100a and run on a B200 (fixtures under tests/golden/).
 * PARITY UNPINNED: repetition penalty, frequency penalty, min-p and k > 64.  The reference has no such
 * terms (it has a presence penalty only, and caps k at 64), so the rules below are this project's
 * definition; with repetition = 1, frequency = 0, min_p = 0 and k <= 64 they reduce bit-exactly to the
 * reference.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (no fused multiply-add: the penalty
 * arithmetic is specified as separately rounded fp32 operations).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define FNS_EMPTY_ID 0x7fffffff

typedef struct {
    float temperature; /* <= 0: greedy (src/kernels.cu:701) */
    float top_p;       /* cut on the T=1 candidate softmax (src/kernels.cu:705-710) */
    float min_p;       /* extension; 0 = off */
    float repetition;  /* extension; 1 = off */
    float presence;    /* reference term (src/kernels.cu:726) */
    float frequency;   /* extension; 0 = off */
    int32_t top_k;     /* <= 0 or > k_cap: k_cap (src/kernels.cu:778) */
    int32_t reserved;
    uint64_t seed;
    uint64_t counter;
} fns_oracle_params;

/* src/kernels.cu:652-665.  Four 32-bit words (counter lo, counter hi, seed lo, seed hi); ten rounds;
 * the round index is xored into the first word; no key schedule.  u = (c0 >> 8) * 2^-24. */
uint32_t fns_oracle_philox_word(uint64_t seed, uint64_t counter) {
    uint32_t c0 = (uint32_t) counter, c1 = (uint32_t) (counter >> 32);
    uint32_t c2 = (uint32_t) seed, c3 = (uint32_t) (seed >> 32);
    for (uint32_t i = 0; i < 10; ++i) {
        const uint64_t m0 = (uint64_t) 0x9E3779B9u * c0, m1 = (uint64_t) 0xBB67AE85u * c2;
        const uint32_t n0 = (uint32_t) (m1 >> 32) ^ c1 ^ i, n2 = (uint32_t) (m0 >> 32) ^ c3;
        c1 = (uint32_t) m1;
        c3 = (uint32_t) m0;
        c0 = n0;
        c2 = n2;
    }
    return c0;
}

float fns_oracle_philox_uniform(uint64_t seed, uint64_t counter) {
    return (float) (fns_oracle_philox_word(seed, counter) >> 8) * (1.0f / 16777216.0f);
}

int fns_oracle_clamp_k(int top_k, int k_cap) { return (top_k <= 0 || top_k > k_cap) ? k_cap : top_k; }

/* Penalties from a history of token ids (plus `n_extra` ids counted as already chosen: the draft prefix
 * of a verification column, src/kernels.cu:738-741).  c = occurrences of id i; for c > 0, in fp32 with
 * each operation rounded separately:
 *     x = x > 0 ? x / repetition : x * repetition;   x = x - frequency * (float) c;   x = x - presence;
 * With repetition 1 and frequency 0 this is the reference's x - presence * seen (src/kernels.cu:726).
 * Ids outside [0, n) are ignored (as the -1 token at src/kernels.cu:730).  counts: scratch of n ints, zero on
 * entry and zero again on return. */
static void penalize(float * x, int n, const int32_t * hist, int n_hist, const int32_t * extra, int n_extra,
                     float repetition, float presence, float frequency, int32_t * counts) {
    for (int j = 0; j < n_hist + n_extra; ++j) {
        const int32_t id = j < n_hist ? hist[j] : extra[j - n_hist];
        if (id >= 0 && id < n) ++counts[id];
    }
    for (int j = 0; j < n_hist + n_extra; ++j) {
        const int32_t id = j < n_hist ? hist[j] : extra[j - n_hist];
        if (id < 0 || id >= n || counts[id] == 0) continue;
        const float c = (float) counts[id];
        counts[id] = 0; /* each id once */
        volatile float v = x[id];
        v = v > 0.0f ? v / repetition : v * repetition;
        volatile float fc = frequency * c;
        v = v - fc;
        v = v - presence;
        x[id] = v;
    }
}

void fns_oracle_penalize(float * x, int n, const int32_t * hist, int n_hist, const int32_t * extra, int n_extra,
                         float repetition, float presence, float frequency) {
    int32_t * counts = (int32_t *) calloc((size_t) n, sizeof(int32_t));
    penalize(x, n, hist, n_hist, extra, n_extra, repetition, presence, frequency, counts);
    free(counts);
}

/* (v, i) precedes (w, j) in the reference's total order: value descending, then index ascending
 * (src/kernels.cu:637-638).  Float compares, so -0.0 and +0.0 tie. */
static int before(float v, int32_t i, float w, int32_t j) { return v > w || (v == w && i < j); }

/* First k allowed, eligible elements of x in the total order.  Eligible = finite: NaN fails every compare,
 * +inf fails `xi < prev_v` against FLT_MAX and `xi == FLT_MAX`, -inf fails `xi > -FLT_MAX` and
 * `xi == -FLT_MAX` (src/kernels.cu:629-639).  -FLT_MAX and FLT_MAX themselves are eligible.
 * id_base is added to the reported ids (vocabulary shards).  Returns the number found (<= k); the rest of
 * cand_v / cand_i is filled with the reference's empty slot (-FLT_MAX, 0x7fffffff) (src/kernels.cu:632-633). */
int fns_oracle_topk(const float * x, int n, const uint32_t * mask, int k, int32_t id_base, float * cand_v,
                    int32_t * cand_i) {
    int nk = 0;
    for (int i = 0; i < n; ++i) {
        if (mask && !((mask[i >> 5] >> (i & 31)) & 1u)) continue;
        const float xi = x[i];
        if (!(xi >= -FLT_MAX && xi <= FLT_MAX)) continue;
        if (nk == k && !before(xi, i, cand_v[k - 1], cand_i[k - 1] - id_base)) continue;
        /* binary search for the insertion point (list is sorted in the total order) */
        int lo = 0, hi = nk;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (before(xi, i, cand_v[mid], cand_i[mid] - id_base)) hi = mid;
            else lo = mid + 1;
        }
        const int last = nk < k ? nk : k - 1;
        memmove(cand_v + lo + 1, cand_v + lo, (size_t) (last - lo) * sizeof(float));
        memmove(cand_i + lo + 1, cand_i + lo, (size_t) (last - lo) * sizeof(int32_t));
        cand_v[lo] = xi;
        cand_i[lo] = i + id_base;
        if (nk < k) ++nk;
    }
    for (int j = nk; j < k; ++j) {
        cand_v[j] = -FLT_MAX;
        cand_i[j] = FNS_EMPTY_ID;
    }
    return nk;
}

/* Merge `lists` candidate lists of `len` entries each (empty slots have id 0x7fffffff) into the first k of
 * their union in the total order: what k_sample's selection rounds do over the 128 slices
 * (src/kernels.cu:680-695).  Ids must be distinct across lists. */
int fns_oracle_merge(const float * v, const int32_t * id, int lists, int len, int k, float * cand_v,
                     int32_t * cand_i) {
    int nk = 0;
    for (int j = 0; j < lists * len; ++j) {
        if (id[j] == FNS_EMPTY_ID) continue;
        if (nk == k && !before(v[j], id[j], cand_v[k - 1], cand_i[k - 1])) continue;
        int lo = 0, hi = nk;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (before(v[j], id[j], cand_v[mid], cand_i[mid])) hi = mid;
            else lo = mid + 1;
        }
        const int last = nk < k ? nk : k - 1;
        memmove(cand_v + lo + 1, cand_v + lo, (size_t) (last - lo) * sizeof(float));
        memmove(cand_i + lo + 1, cand_i + lo, (size_t) (last - lo) * sizeof(int32_t));
        cand_v[lo] = v[j];
        cand_i[lo] = id[j];
        if (nk < k) ++nk;
    }
    for (int j = nk; j < k; ++j) {
        cand_v[j] = -FLT_MAX;
        cand_i[j] = FNS_EMPTY_ID;
    }
    return nk;
}

/* The tail of k_sample (src/kernels.cu:698-720) over nk sorted candidates, plus min-p.
 *   nk == 0 -> -1;  T <= 0 or nk == 1 -> first candidate.
 *   p_j = exp((double) v_j - (double) v_0), sum accumulated in order;
 *   keep = first j + 1 with cum += p_j / sum reaching top_p (float promoted), else nk;
 *   min-p (extension, applied after the top-p cut on the same T=1 weights): keep the longest prefix with
 *   p_j >= (double) min_p, at least one;
 *   w_j = exp(((double) v_j - (double) v_0) / T), wsum in order; u = uniform * wsum; first j with u < acc,
 *   default keep - 1.
 * Optional outputs: q[j] = w_j / wsum for j < keep (0 beyond), *keep_out, *u_out (the uniform in [0,1)),
 * cdf[j] = running acc / wsum (for the CDF-boundary tolerance rule). */
int32_t fns_oracle_draw(const float * cand_v, const int32_t * cand_i, int nk, const fns_oracle_params * p, double * q,
                        int32_t * keep_out, double * u_out, double * cdf) {
    if (keep_out) *keep_out = nk > 0 ? 1 : 0;
    if (u_out) *u_out = 0.0;
    if (nk == 0) return -1;
    if (p->temperature <= 0.0f || nk == 1) {
        if (q) q[0] = 1.0;
        if (cdf) cdf[0] = 1.0;
        return cand_i[0];
    }
    double * pj = (double *) malloc(sizeof(double) * 2 * (size_t) nk), *w = pj + nk;
    double sum = 0.0;
    for (int j = 0; j < nk; ++j) sum += pj[j] = exp((double) cand_v[j] - (double) cand_v[0]);
    int keep = nk;
    double cum = 0.0;
    for (int j = 0; j < nk; ++j) {
        cum += pj[j] / sum;
        if (cum >= p->top_p) { keep = j + 1; break; }
    }
    if (p->min_p > 0.0f) {
        int m = 1;
        while (m < keep && pj[m] >= (double) p->min_p) ++m;
        keep = m;
    }
    double wsum = 0.0;
    for (int j = 0; j < keep; ++j) wsum += w[j] = exp(((double) cand_v[j] - (double) cand_v[0]) / p->temperature);
    const float uf = fns_oracle_philox_uniform(p->seed, p->counter);
    const double u = uf * wsum;
    double acc = 0.0;
    int pick = keep - 1, found = 0;
    for (int j = 0; j < keep; ++j) {
        acc += w[j];
        if (cdf) cdf[j] = acc / wsum;
        if (!found && u < acc) {
            pick = j;
            found = 1;
            if (!cdf) break;
        }
    }
    if (q) for (int j = 0; j < nk; ++j) q[j] = j < keep ? w[j] / wsum : 0.0;
    if (keep_out) *keep_out = keep;
    if (u_out) *u_out = (double) uf;
    const int32_t tok = cand_i[pick];
    free(pj);
    return tok;
}

/* One row end to end: penalties on a private copy of the logits (the reference mutates them in place,
 * src/kernels.cu:726; the copy keeps the caller's row intact), selection, draw.
 * Optional outputs cand_v / cand_i (k_cap entries, penalised values) and *nk_out. */
int32_t fns_oracle_sample_row(const float * x, int n, const uint32_t * mask, const int32_t * hist, int n_hist,
                              const int32_t * extra, int n_extra, const fns_oracle_params * p, int k_cap,
                              float * cand_v, int32_t * cand_i, int32_t * nk_out) {
    const int k = p->temperature <= 0.0f ? 1 : fns_oracle_clamp_k(p->top_k, k_cap);
    const float * src = x;
    float * copy = NULL;
    if ((n_hist + n_extra) > 0 && (p->repetition != 1.0f || p->presence != 0.0f || p->frequency != 0.0f)) {
        copy = (float *) malloc(sizeof(float) * (size_t) n);
        memcpy(copy, x, sizeof(float) * (size_t) n);
        fns_oracle_penalize(copy, n, hist, n_hist, extra, n_extra, p->repetition, p->presence, p->frequency);
        src = copy;
    }
    float * cv = cand_v ? cand_v : (float *) malloc(sizeof(float) * (size_t) k);
    int32_t * ci = cand_i ? cand_i : (int32_t *) malloc(sizeof(int32_t) * (size_t) k);
    const int nk = fns_oracle_topk(src, n, mask, k, 0, cv, ci);
    if (cand_v) for (int j = k; j < k_cap; ++j) { cand_v[j] = -FLT_MAX; cand_i[j] = FNS_EMPTY_ID; }
    const int32_t tok = fns_oracle_draw(cv, ci, nk, p, NULL, NULL, NULL, NULL);
    if (nk_out) *nk_out = nk;
    if (!cand_v) free(cv);
    if (!cand_i) free(ci);
    free(copy);
    return tok;
}

/* Rows in parallel over host threads (the reference's own host check is single-threaded,
 * tests/sample_check.cu:43; threads = 0 uses every core).  hist: [rows][hist_stride], hist_len[rows];
 * masks: [rows][mask_stride] or NULL; returns the number of threads used. */
int fns_oracle_sample_rows(const float * x, int64_t row_stride, int n, int rows, const uint32_t * masks,
                           int64_t mask_stride, const int32_t * hist, int64_t hist_stride,
                           const int32_t * hist_len, const fns_oracle_params * params, int k_cap, int32_t * out,
                           int threads) {
    int used = 1;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
    used = threads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
#endif
    for (int r = 0; r < rows; ++r) {
        out[r] = fns_oracle_sample_row(x + r * row_stride, n, masks ? masks + r * mask_stride : NULL,
                                       hist ? hist + r * hist_stride : NULL, hist ? hist_len[r] : 0, NULL, 0,
                                       params + r, k_cap, NULL, NULL, NULL);
    }
    return used;
}

/* bf16 -> fp32 widening is exact (the bits become the high half of the float). */
void fns_oracle_widen_bf16(const uint16_t * src, float * dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const uint32_t b = (uint32_t) src[i] << 16;
        memcpy(dst + i, &b, 4);
    }
}

/* Accept rule of a verification window (tools/fns_serve/fns_serve.cpp:492-508): column 0 is always
 * committed; column c + 1 is valid only while tokens[c] == draft[c] and c < n_draft.  Returns a = number of
 * leading matches; the emitted tokens are tokens[0 .. a], tokens[a] being the bonus / correction. */
int32_t fns_oracle_accept_len(const int32_t * tokens, const int32_t * draft, int n_draft) {
    int a = 0;
    while (a < n_draft && tokens[a] == draft[a]) ++a;
    return a;
}

/* A whole window: W = n_draft + 1 rows of logits; column c is penalised with the history plus draft[0 .. c)
 * (src/kernels.cu:735-742) and drawn with Philox counter `counter + c` (src/engine.cu:750-757).
 * masks: [W][mask_stride] or NULL.  Writes tokens[W] and returns the accept length. */
int32_t fns_oracle_verify_window(const float * x, int64_t row_stride, int n, int n_draft, const int32_t * draft,
                                 const uint32_t * masks, int64_t mask_stride, const int32_t * hist, int n_hist,
                                 const fns_oracle_params * p, int k_cap, int32_t * tokens) {
    for (int c = 0; c <= n_draft; ++c) {
        fns_oracle_params pc = *p;
        pc.counter = p->counter + (uint64_t) c;
        tokens[c] = fns_oracle_sample_row(x + c * row_stride, n, masks ? masks + c * mask_stride : NULL, hist, n_hist,
                                          draft, c, &pc, k_cap, NULL, NULL, NULL);
    }
    return fns_oracle_accept_len(tokens, draft, n_draft);
}

/* Prompt-lookup draft (include/fns/lookup.h:12-27): the continuation of the latest earlier occurrence of the
 * final n-gram of the history, n = 4 down to 2. */
int fns_oracle_lookup_draft(const int32_t * h, int n_h, int want, int32_t * out) {
    for (int n = 4; n >= 2; --n) {
        if (n_h < n + 1) continue;
        for (int s = n_h - n - 1; s >= 0; --s) {
            if (memcmp(h + s, h + n_h - n, sizeof(int32_t) * (size_t) n) != 0) continue;
            int k = 0;
            while (k < want && s + n + k < n_h) { out[k] = h[s + n + k]; ++k; }
            if (k > 0) return k;
        }
    }
    return 0;
}

/* Dense presence helpers of the reference (src/kernels.cu:724-752), for the compat entry points. */
void fns_oracle_presence_apply(float * x, const float * seen, int n, float penalty) {
    for (int i = 0; i < n; ++i) {
        volatile float t = penalty * seen[i];
        x[i] = x[i] - t;
    }
}

void fns_oracle_presence_apply_col(float * x, const float * seen, const int32_t * draft, int c, int n, float penalty) {
    for (int i = 0; i < n; ++i) {
        float s = seen[i];
        for (int k = 0; k < c; ++k)
            if (draft[k] == i) s = 1.0f;
        volatile float t = penalty * s;
        x[i] = x[i] - t;
    }
}

void fns_oracle_io_advance(int32_t * io, int pos) {
    io[0] = io[2] < 0 ? 0 : io[2];
    io[1] = pos;
}
