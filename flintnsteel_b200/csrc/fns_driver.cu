// fns_driver.cu - the callers either side of the sampler, as far as they belong to the sampler's path:
//   * the speculation driver pieces of fns-serve (NomenAK/FlintNSteel tools/fns_serve/fns_serve.cpp:340-354, 383-521):
//     window-mask protocol over a grammar matcher, adaptive width policy, the accept / commit loop, and the whole
//     decode loop around fns_b200_engine (sequential and speculative) with the model behind a callback;
//   * the prompt-lookup draft (include/fns/lookup.h:12-27) for batched rows on the device;
//   * the request surface of fns-serve (fns_serve.cpp:291-303): the sampling fields of one JSON line.
// Host C++ behind the C ABI; the only kernel here is the batched lookup.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "fns_internal.h"

// ---- prompt-lookup draft for a batch of rows, on the device -----------------------------------------------------
namespace {

// One block per row.  The rule of include/fns/lookup.h:12-27: for n = 4, 3, 2 take the LATEST earlier start s
// (s <= len - n - 1) whose n ids equal the final n ids; the draft is what followed it, at most `want` ids.  The
// threads test the starts in parallel; the latest match is a maximum.
__global__ void k_lookup_draft(const int32_t * history, int64_t stride, const int32_t * history_len, int want, int32_t * out,
                               int64_t out_stride, int32_t * out_n) {
    __shared__ int best;
    const int row = blockIdx.x;
    const int32_t * h = history + (size_t) row * stride;
    int len = history_len[row];
    if (len < 0) len = 0;
    if (len > stride) len = (int) stride;
    int got = 0;
    for (int n = 4; n >= 2 && got == 0; --n) {
        if (threadIdx.x == 0) best = -1;
        __syncthreads();
        if (len >= n + 1) {
            const int32_t * tail = h + len - n;
            for (int s = len - n - 1 - (int) threadIdx.x; s >= 0; s -= (int) blockDim.x) {
                bool same = true;
                for (int j = 0; j < n && same; ++j) same = h[s + j] == tail[j];
                if (same) {
                    atomicMax(&best, s);
                    break;  // this thread's later starts are smaller
                }
            }
        }
        __syncthreads();
        const int s = best;
        if (s >= 0) {
            int k = len - (s + n);
            k = k < want ? k : want;
            for (int j = threadIdx.x; j < k; j += blockDim.x) out[(size_t) row * out_stride + j] = h[s + n + j];
            got = k;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out_n[row] = got;
}

}  // namespace

extern "C" {

int fns_b200_lookup_draft_rows(const int32_t * history, int64_t history_stride, const int32_t * history_len, int rows,
                               int want, int32_t * out, int64_t out_stride, int32_t * out_n, void * stream) {
    if (!history || !history_len || !out || !out_n || rows <= 0 || want <= 0 || history_stride <= 0 || out_stride < want)
        return FNS_B200_ERR_ARG;
    k_lookup_draft<<<(unsigned) rows, 128, 0, (cudaStream_t) stream>>>(history, history_stride, history_len, want, out,
                                                                       out_stride, out_n);
    return cudaGetLastError() == cudaSuccess ? FNS_B200_OK : FNS_B200_ERR_CUDA;
}

// ---- adaptive window width (fns_serve.cpp:430-459) and its cost record (:470-476, :511-516) ---------------------
void fns_b200_spec_policy_init(fns_b200_spec_policy * p, int spec) {
    if (!p) return;
    std::memset(p, 0, sizeof *p);
    p->spec = spec < 0 ? 0 : (spec > FNS_B200_MAX_WINDOW ? FNS_B200_MAX_WINDOW : spec);
}

void fns_b200_spec_policy_new_request(fns_b200_spec_policy * p) {  // acceptance is request-local, costs persist
    if (!p) return;
    p->accepted = p->offered = 0;
    p->skipped_proposals = 0;
}

int fns_b200_spec_choose_width(fns_b200_spec_policy * p, int nd_max) {
    if (!p || nd_max <= 0) return 0;
    const double a = (double) (p->accepted + 1) / (double) (p->offered + 2);
    double t1_cost = p->cost[1];
    if (t1_cost == 0.0) {  // no sequential cost observed: infer its scale from a measured width
        for (int w = 2; w <= p->spec; ++w) {
            if (p->cost[w] > 0.0) {
                t1_cost = p->cost[w] / (1.0 + 0.25 * (w - 1));
                break;
            }
        }
        if (t1_cost == 0.0) t1_cost = 1.0;
    }
    int best = 0;
    double best_score = 1.0, expected = 1.0, power = 1.0;
    for (int n = 1; n <= nd_max && n + 1 <= FNS_B200_MAX_WINDOW; ++n) {
        power *= a;
        expected += power;
        const double cost = p->cost[n + 1] > 0.0 ? p->cost[n + 1] / t1_cost : 1.0 + 0.25 * n;
        const double score = expected / cost;
        if (score > best_score) {
            best_score = score;
            best = n;
        }
    }
    if (best == 0 && p->skipped_proposals >= 16) best = 1;
    if (best == 0) ++p->skipped_proposals;
    else p->skipped_proposals = 0;
    return best;
}

void fns_b200_spec_observe(fns_b200_spec_policy * p, int width, double elapsed_s, int window_accepted, int window_offered) {
    if (!p || width < 1 || width > FNS_B200_MAX_WINDOW) return;
    p->accepted += (uint64_t) (window_accepted > 0 ? window_accepted : 0);
    p->offered += (uint64_t) (window_offered > 0 ? window_offered : 0);
    if (elapsed_s > 0.0) p->cost[width] = p->cost[width] > 0.0 ? p->cost[width] * 0.875 + elapsed_s * 0.125 : elapsed_s;
}

// ---- masks of a window (fns_serve.cpp:340-354) ---------------------------------------------------------------------
int fns_b200_spec_window_masks(const fns_b200_grammar * g, const int32_t * draft, int nd, int words, uint32_t * wmask) {
    if (!g) return nd + 1;
    if (!g->fill || !g->accept || !g->rollback || !wmask || nd < 0 || words <= 0 || (nd > 0 && !draft)) return -1;
    int c = 0, accepted = 0;
    for (;; ++c) {
        g->fill(g->user, reinterpret_cast<int32_t *>(wmask + (size_t) c * words));  // column c follows the prefix + d[0 .. c)
        if (c == nd || !g->accept(g->user, draft[c])) break;
        ++accepted;
        if (g->terminated && g->terminated(g->user)) break;  // d[c] terminates: nothing to predict after it
    }
    if (accepted) g->rollback(g->user, accepted);
    return (c < nd ? c : nd) + 1;
}

// ---- the accept / commit loop over one verified window (fns_serve.cpp:486-508) -------------------------------------
int fns_b200_spec_commit(const int32_t * out, int W, const int32_t * draft, int nd, const int32_t * stop, int n_stop,
                         int max_tokens, const fns_b200_grammar * g, fns_b200_spec_counters * c, int32_t * committed,
                         int * engaged, int * window_accepted, int * window_offered) {
    if (!out || !c || !committed || !engaged || W < 1 || nd < 0 || nd > W - 1 || (nd > 0 && !draft)) return -1;
    int done = 0, eng = 0, acc = 0, off = 0;
    for (int col = 0; col < W && !done; ++col) {
        const int32_t t = out[col];
        if (g && g->accept && (t < 0 || !g->accept(g->user, t))) return -2;  // token rejected by the grammar
        committed[eng++] = t;
        ++c->emitted;
        if (col < nd) {
            ++off;
            if (t == draft[col]) {
                ++c->accepted;
                ++acc;
            }
        }
        ++c->generated;
        for (int j = 0; j < n_stop && !done; ++j)
            if (stop[j] == t) done = 1;  // a stop token ends the generation ...
        if (!done && c->generated >= max_tokens) done = 2;  // ... and so does the output budget
        if (col == nd || t != draft[col]) break;  // the next column was computed on another token
    }
    *engaged = eng;
    if (window_accepted) *window_accepted = acc;
    if (window_offered) *window_offered = off;
    return done;
}

// ---- the decode loop of fns-serve around the engine glue (fns_serve.cpp:383-521) -----------------------------------
int fns_b200_spec_decode(fns_b200_engine * e, const fns_b200_model * m, const fns_b200_grammar * g, const int32_t * prompt,
                         int n_prompt, int max_tokens, const int32_t * stop, int n_stop, const fns_b200_params * sp, int dtype,
                         int spec, fns_b200_spec_policy * policy, int32_t * out_tokens, fns_b200_spec_counters * counters,
                         void * stream) {
    if (!e || !m || !m->forward || !prompt || n_prompt <= 0 || max_tokens <= 0 || !sp || !out_tokens || !counters)
        return FNS_B200_ERR_ARG;
    if (spec < 0 || spec > FNS_B200_MAX_WINDOW) return FNS_B200_ERR_ARG;
    std::memset(counters, 0, sizeof *counters);
    const int words = fns_b200_engine_words(e);
    std::vector<int32_t> ctx(prompt, prompt + n_prompt), d(spec > 0 ? spec : 1), out(spec > 0 ? spec : 1), ids(spec > 0 ? spec : 1);
    std::vector<uint32_t> wmask(g ? (size_t) (spec > 0 ? spec : 1) * words : 0);
    const bool penal = sp->presence != 0.0f || sp->repetition != 1.0f || sp->frequency != 0.0f;
    int rc = FNS_B200_OK;
    if (penal && (rc = fns_b200_engine_reset(e, stream)) != FNS_B200_OK) return rc;  // Engine::reset_presence
    uint64_t draw = 0;
    fns_b200_params p = *sp;
    // one choice from one row of logits, masked by the grammar if any (begin_choice / end_choice, :326-338)
    auto choose = [&](const void * logits, int64_t row_stride, int32_t * tok) -> int {
        p.counter = sp->counter + draw++;
        if (g) g->fill(g->user, reinterpret_cast<int32_t *>(wmask.data()));
        int r = fns_b200_engine_pick_async(e, logits, 0, dtype, row_stride, 1, g ? wmask.data() : nullptr, nullptr, 0, nullptr,
                                           &p, stream);
        if (r != FNS_B200_OK) return r;
        if (penal) {  // k::presence_mark: the chosen token joins the session's history (src/engine.cu:843)
            r = fns_b200_engine_append(e, fns_b200_engine_device_tokens(e), 1, 1, nullptr, stream);
            if (r != FNS_B200_OK) return r;
        }
        r = fns_b200_engine_pick_wait(e, tok);
        if (r != FNS_B200_OK) return r;
        if (g && (*tok < 0 || !g->accept(g->user, *tok))) return FNS_B200_ERR_ARG;  // token rejected by the grammar
        return FNS_B200_OK;
    };
    auto stops = [&](int32_t t) {
        for (int j = 0; j < n_stop; ++j)
            if (stop[j] == t) return true;
        return false;
    };
    const void * logits = nullptr;
    int64_t row_stride = 0;
    // the first choice comes from the logits of the last prompt token (prefill; counter 0)
    int32_t last = ctx.back();
    if ((rc = m->forward(m->user, &last, 1, n_prompt - 1, &logits, &row_stride)) != FNS_B200_OK) return rc;
    int32_t tok = -1;
    if ((rc = choose(logits, row_stride, &tok)) != FNS_B200_OK) return rc;
    const bool speculate = spec > 1;
    if (!speculate) {  // sequential decode (:390-409)
        while (counters->generated < max_tokens) {
            out_tokens[counters->generated++] = tok;
            if (stops(tok) || counters->generated == max_tokens) break;
            ctx.push_back(tok);
            ++counters->iterations;
            if ((rc = m->forward(m->user, &tok, 1, (int) ctx.size() - 1, &logits, &row_stride)) != FNS_B200_OK) return rc;
            if ((rc = choose(logits, row_stride, &tok)) != FNS_B200_OK) return rc;
        }
        return FNS_B200_OK;
    }
    // speculation (:410-519).  `last`: the last committed token, not yet consumed by a forward pass.
    last = tok;
    auto commit_one = [&](int32_t t) -> bool {  // emits t; true if generation stops
        out_tokens[counters->generated++] = t;
        ctx.push_back(t);
        return stops(t) || counters->generated == max_tokens;
    };
    bool done = commit_one(last);
    if (policy) fns_b200_spec_policy_new_request(policy);
    while (!done) {
        const int room = std::min(spec - 1, max_tokens - counters->generated);
        int nd = room > 0 ? fns_b200_lookup_draft(ctx.data(), (int) ctx.size(), room, d.data()) : 0;
        if (policy && nd > 0) {
            nd = fns_b200_spec_choose_width(policy, nd);
            if (nd == 0) ++counters->skipped;
        }
        const auto t_start = std::chrono::steady_clock::now();
        const int W = nd > 0 ? fns_b200_spec_window_masks(g, d.data(), nd, words, wmask.data()) : 1;
        if (W < 1) return FNS_B200_ERR_ARG;
        nd = W - 1;
        const int p0 = (int) ctx.size() - 1;
        ++counters->iterations;
        if (nd == 0) {  // no draft: one ordinary step
            if ((rc = m->forward(m->user, &last, 1, p0, &logits, &row_stride)) != FNS_B200_OK) return rc;
            if ((rc = choose(logits, row_stride, &last)) != FNS_B200_OK) return rc;
            if (policy)
                fns_b200_spec_observe(policy, 1, std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count(), 0, 0);
            done = commit_one(last);
            continue;
        }
        ids[0] = last;
        for (int k = 0; k < nd; ++k) ids[1 + k] = d[k];
        if ((rc = m->forward(m->user, ids.data(), W, p0, &logits, &row_stride)) != FNS_B200_OK) return rc;
        // column c: the choice for generated token number draw + c (Engine::verify, src/engine.cu:745-757)
        p.counter = sp->counter + draw;
        int32_t accept_len = 0;
        if ((rc = fns_b200_engine_verify(e, logits, dtype, row_stride, 1, nd, d.data(), g ? wmask.data() : nullptr, &p, out.data(),
                                         &accept_len, stream)) != FNS_B200_OK)
            return rc;
        ++counters->windows;
        counters->drafted += nd;
        std::vector<int32_t> committed(W);
        int engaged = 0, w_acc = 0, w_off = 0;
        const int before = counters->generated;
        const int fin = fns_b200_spec_commit(out.data(), W, d.data(), nd, stop, n_stop, max_tokens, g, counters, committed.data(),
                                             &engaged, &w_acc, &w_off);
        if (fin < 0) return FNS_B200_ERR_ARG;
        counters->generated = before;  // (commit_one counts and stores them)
        for (int c = 0; c < engaged; ++c) {
            last = committed[c];
            ++draw;
            done = commit_one(last);
        }
        done = done || fin != 0;
        if (policy)
            fns_b200_spec_observe(policy, W, std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count(), w_acc,
                                  w_off);
        if (penal) {  // Engine::presence_commit: only the committed choices are remembered (src/engine.cu:862-866)
            const int32_t n = engaged;
            if ((rc = fns_b200_engine_append(e, fns_b200_engine_device_tokens(e), W, 1, &n, stream)) != FNS_B200_OK) return rc;
        }
    }
    return FNS_B200_OK;
}

// ---- the sampling fields of a request line (fns_serve.cpp:291-303) -------------------------------------------------
// `"key": number` pairs of one JSON object, by name.  The reference reads "temperature", "top_p", "top_k", "seed",
// "presence_penalty" (defaults: greedy, no cut, 64 candidates, seed 0, no penalty); "min_p", "repetition_penalty" and
// "frequency_penalty" are this library's additions.  A field that is absent or not a number keeps its default.
static bool json_number(const char * line, const char * key, double * out) {
    const size_t klen = std::strlen(key);
    for (const char * at = line; (at = std::strchr(at, '"')) != nullptr; ++at) {
        if (std::strncmp(at + 1, key, klen) != 0 || at[1 + klen] != '"') continue;
        const char * q = at + klen + 2;
        while (*q == ' ' || *q == '\t') ++q;
        if (*q != ':') continue;
        ++q;
        while (*q == ' ' || *q == '\t') ++q;
        char * end = nullptr;
        const double v = std::strtod(q, &end);
        if (end == q) return false;  // not a number: the default stands
        *out = v;
        return true;
    }
    return false;
}

int fns_b200_params_from_json(const char * line, fns_b200_params * out) {
    if (!line || !out) return FNS_B200_ERR_ARG;
    auto num = [&](const char * k, double def) {
        double v = def;
        json_number(line, k, &v);
        return v;
    };
    std::memset(out, 0, sizeof *out);
    out->temperature = (float) num("temperature", 0.0);
    out->top_p = (float) num("top_p", 1.0);
    out->top_k = (int32_t) num("top_k", 0.0);
    out->seed = (uint64_t) num("seed", 0.0);
    out->presence = (float) num("presence_penalty", 0.0);
    out->min_p = (float) num("min_p", 0.0);
    out->repetition = (float) num("repetition_penalty", 1.0);
    out->frequency = (float) num("frequency_penalty", 0.0);
    out->counter = 0;  // the draw for generated token n uses Philox counter n: the caller counts
    return FNS_B200_OK;
}

}  // extern "C"
