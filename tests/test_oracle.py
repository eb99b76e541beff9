"""Pins the CPU oracle (oracle/fns_oracle.c) without a GPU:

* against the known answers and the statistical criterion of the reference's own sampler test
  (tests/sample_check.cu in the reference tree), on that test's own inputs;
* against independent numpy restatements of each stage (stable sort, bincount penalties, big-integer Philox);
* against the fixtures in tests/golden/, which hold outputs of the reference's CUDA kernels run on a B200.
"""
import json
import os

import numpy as np
import pytest

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.sampler import make_params

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
N_REF = 150_144  # vocabulary of the reference's test (tests/sample_check.cu:79)


@pytest.fixture(scope="module")
def lcg():
    return wl.lcg_logits(N_REF)


# ---- known answers of tests/sample_check.cu ---------------------------------------------------------------
def test_lcg_inputs_have_the_documented_shape(lcg):
    x, mask, spikes = lcg
    assert x[0] == 8.0 and x[spikes[1]] == 7.75 and x[spikes[29]] == 0.75  # :86, 8 - 0.25 j
    assert np.all(np.abs(np.delete(x, spikes)) <= 3.0)                       # :85
    assert sum(bin(int(w)).count("1") for w in mask) == 15                   # :87-88, every other spike


def test_masked_greedy_is_id_0(oracle, lcg):  # :102-105
    x, mask, _ = lcg
    assert oracle.sample_row(x, make_params(1, temperature=0.0, top_k=20, top_p=0.95), mask=mask) == 0


def test_ties_across_slices_pick_the_smallest_index(oracle):  # :109-114
    flat = np.ones(N_REF, np.float32)
    flat[[149000, 70000, 1201, 1200]] = 5.0
    assert oracle.sample_row(flat, make_params(1)) == 1200


def test_masked_tie(oracle):  # :115-121
    flat = np.ones(N_REF, np.float32)
    flat[[149000, 70000, 1201, 1200]] = 5.0
    m = np.zeros((N_REF + 31) // 32, np.uint32)
    for i in (70000, 149000):
        m[i >> 5] |= np.uint32(1 << (i & 31))
    assert oracle.sample_row(flat, make_params(1), mask=m) == 70000


def test_all_equal_is_id_0_and_empty_mask_is_minus_1(oracle):  # :122-131
    flat = np.full(N_REF, 2.0, np.float32)
    assert oracle.sample_row(flat, make_params(1)) == 0
    m = np.zeros((N_REF + 31) // 32, np.uint32)
    assert oracle.sample_row(flat, make_params(1, temperature=1.0, top_k=20), mask=m) == -1


@pytest.mark.parametrize("case", [
    dict(top_k=20, top_p=0.95, temperature=1.0, masked=False),   # :90
    dict(top_k=0, top_p=1.0, temperature=0.7, masked=False),     # :91
    dict(top_k=20, top_p=1.0, temperature=1.0, masked=True),     # :92
])
def test_draw_frequencies_within_five_sigma(oracle, lcg, case):
    """The reference's criterion (tests/sample_check.cu:63-75): 200 000 draws with seed 1234 and counters
    0 .. N-1; every kept candidate within 5 binomial standard deviations, nothing outside the kept set.  The
    expected distribution is rebuilt here with numpy (stable sort = index ascending on ties, :43)."""
    x, mask, _ = lcg
    m = mask if case["masked"] else None
    n_draws = 200_000
    allowed = np.arange(N_REF) if m is None else np.nonzero(wl.mask_allows(m, np.arange(N_REF)))[0]
    order = allowed[np.argsort(-x[allowed].astype(np.float64), kind="stable")]
    k = min(order.size, 64 if case["top_k"] <= 0 or case["top_k"] > 64 else case["top_k"])
    idx = order[:k]
    p = np.exp(x[idx].astype(np.float64) - float(x[idx[0]]))
    cum = np.cumsum(p / p.sum())
    hit = np.nonzero(cum >= np.float32(case["top_p"]))[0]
    keep = int(hit[0]) + 1 if hit.size else k
    w = np.exp((x[idx[:keep]].astype(np.float64) - float(x[idx[0]])) / np.float32(case["temperature"]))
    q = w / w.sum()

    cv, ci, nk = oracle.topk(x, m, k)
    assert nk == k and np.array_equal(ci, idx.astype(np.int32))
    counts = {}
    base = make_params(1, temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"], seed=1234)
    for c in range(n_draws):
        base["counter"] = c
        t = oracle.draw(cv, ci, nk, base)
        counts[t] = counts.get(t, 0) + 1
    outside = n_draws - sum(counts.get(int(i), 0) for i in idx[:keep])
    assert outside == 0
    f = np.array([counts.get(int(i), 0) for i in idx[:keep]]) / n_draws
    sd = np.sqrt(q * (1 - q) / n_draws) + 1e-12
    assert np.max(np.abs(f - q) / sd) < 5.0


# ---- stage by stage against numpy -------------------------------------------------------------------------
def philox_reference(seed: int, counter: int) -> int:
    """src/kernels.cu:652-665 with Python integers."""
    c0, c1, c2, c3 = counter & 0xFFFFFFFF, counter >> 32, seed & 0xFFFFFFFF, seed >> 32
    for i in range(10):
        m0, m1 = 0x9E3779B9 * c0, 0xBB67AE85 * c2
        c0, c1, c2, c3 = (m1 >> 32) ^ c1 ^ i, m1 & 0xFFFFFFFF, (m0 >> 32) ^ c3, m0 & 0xFFFFFFFF
    return c0


def test_philox_matches_big_integer_restatement(oracle):
    g = np.random.default_rng(5)
    cases = [(0, 0), (1234, 0), (0, 1), (2**64 - 1, 2**64 - 1), (1 << 32, 1 << 32)]
    cases += [(int(a), int(b)) for a, b in g.integers(0, 2**63, size=(200, 2))]
    for seed, counter in cases:
        w = philox_reference(seed, counter)
        assert oracle.philox_word(seed, counter) == w
        u = oracle.philox_uniform(seed, counter)
        assert u == np.float32(w >> 8) * np.float32(2.0 ** -24) and 0.0 <= u < 1.0


def test_philox_uniform_is_uniform(oracle):
    u = np.array([oracle.philox_uniform(7, c) for c in range(50_000)])
    hist, _ = np.histogram(u, bins=20, range=(0, 1))
    assert np.all(np.abs(hist - 2500) < 5 * np.sqrt(2500))


def test_clamp_k_follows_the_reference(oracle):  # src/kernels.cu:778
    assert [oracle.clamp_k(k, 64) for k in (-1, 0, 1, 40, 64, 65, 1000)] == [64, 64, 1, 40, 64, 64, 64]
    assert oracle.clamp_k(100, 128) == 100


def topk_numpy(x, mask, k):
    ids = np.arange(x.size)
    ok = np.isfinite(x)
    if mask is not None:
        ok &= wl.mask_allows(mask, ids)
    ids = ids[ok]
    xs = x[ids].astype(np.float64) + 0.0  # -0.0 + 0.0 = +0.0: the float compare ties them
    order = ids[np.argsort(-xs, kind="stable")][:k]
    return order.astype(np.int32)


@pytest.mark.parametrize("n", [1, 31, 32, 33, 1187, 1188, 5000])
@pytest.mark.parametrize("k", [1, 7, 64])
def test_topk_matches_stable_sort(oracle, n, k):
    g = np.random.default_rng(n * 131 + k)
    x = g.standard_normal(n).astype(np.float32)
    x[g.integers(0, n, size=max(1, n // 8))] = np.float32(0.5)   # ties
    x[g.integers(0, n, size=max(1, n // 16))] = np.float32(-0.0)
    x[g.integers(0, n, size=max(1, n // 16))] = np.float32(0.0)
    for v in (np.nan, np.inf, -np.inf):
        x[g.integers(0, n)] = v
    mask = wl.random_mask(g, n, 0.6)
    for m in (None, mask):
        cv, ci, nk = oracle.topk(x, m, k)
        exp = topk_numpy(x, m, k)
        assert nk == exp.size
        assert np.array_equal(ci[:nk], exp)
        assert np.array_equal(cv[:nk].view(np.uint32), x[exp].view(np.uint32))
        assert np.all(ci[nk:] == 0x7FFFFFFF) and np.all(cv[nk:] == -np.finfo(np.float32).max)


def test_flt_max_values_are_eligible_infinities_are_not(oracle):  # src/kernels.cu:629-639
    fmax = np.finfo(np.float32).max
    x = np.array([-np.inf, -fmax, np.nan, np.inf], np.float32)
    cv, ci, nk = oracle.topk(x, None, 4)
    assert nk == 1 and ci[0] == 1
    x = np.array([np.inf, fmax, 3.0], np.float32)
    cv, ci, nk = oracle.topk(x, None, 4)
    assert nk == 2 and list(ci[:2]) == [1, 2]


def test_penalties_match_numpy_and_reduce_to_presence(oracle):
    g = np.random.default_rng(11)
    n = 4096
    x = g.standard_normal(n).astype(np.float32) * 3
    hist = g.integers(-5, n + 5, size=900).astype(np.int32)  # some ids outside the vocabulary: ignored
    rep, pres, freq = np.float32(1.1), np.float32(0.5), np.float32(0.3)
    got = oracle.penalize(x, hist, None, rep, pres, freq)
    inside = hist[(hist >= 0) & (hist < n)]
    c = np.bincount(inside, minlength=n).astype(np.float32)
    exp = x.copy()
    seen = c > 0
    exp[seen] = np.where(x[seen] > 0, x[seen] / rep, x[seen] * rep)
    exp[seen] = exp[seen] - freq * c[seen]
    exp[seen] = exp[seen] - pres
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))
    # repetition 1, frequency 0: the reference's x - penalty * seen (src/kernels.cu:726)
    got = oracle.penalize(x, hist, None, 1.0, 0.25, 0.0)
    ref = oracle.presence_apply(x, seen.astype(np.float32), 0.25)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    # a verification column counts draft[0 .. c) as seen (src/kernels.cu:738-741)
    draft = np.array([5, 7, 5], np.int32)
    got = oracle.penalize(x, inside, draft[:2], 1.0, 0.25, 0.0)
    ref = oracle.presence_apply_col(x, seen.astype(np.float32), draft, 2, 0.25)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_draw_short_cuts_and_default_pick(oracle):  # src/kernels.cu:700-701, :715
    cv = np.array([2.0, 1.0, 0.0], np.float32)
    ci = np.array([10, 20, 30], np.int32)
    assert oracle.draw(cv, ci, 0, make_params(1, temperature=1.0)) == -1
    assert oracle.draw(cv, ci, 1, make_params(1, temperature=1.0)) == 10
    assert oracle.draw(cv, ci, 3, make_params(1, temperature=0.0)) == 10
    assert oracle.draw(cv, ci, 3, make_params(1, temperature=-1.0)) == 10
    tok, q, keep, u, cdf = oracle.draw(cv, ci, 3, make_params(1, temperature=1.0, top_p=1.0, seed=3, counter=9), True)
    assert keep == 3 and abs(q.sum() - 1) < 1e-12 and abs(cdf[2] - 1) < 1e-12
    assert tok == ci[np.searchsorted(cdf, u, side="right")]
    # top_p cut: p = (0.665, 0.245, 0.090); 0.6 keeps one candidate, 0.9 keeps two
    assert oracle.draw(cv, ci, 3, make_params(1, temperature=1.0, top_p=0.6), True)[2] == 1
    assert oracle.draw(cv, ci, 3, make_params(1, temperature=1.0, top_p=0.9), True)[2] == 2
    # min_p (extension): exp(v_j - v_0) = 1, 0.368, 0.135
    assert oracle.draw(cv, ci, 3, make_params(1, temperature=1.0, min_p=0.2), True)[2] == 2
    assert oracle.draw(cv, ci, 3, make_params(1, temperature=1.0, min_p=0.5), True)[2] == 1
    assert oracle.draw(cv, ci, 3, make_params(1, temperature=1.0, min_p=0.1), True)[2] == 3


def test_merge_of_slice_lists_equals_global_topk(oracle):  # src/kernels.cu:594-597
    g = np.random.default_rng(3)
    n, k, parts = 6000, 16, 6
    x = np.round(g.standard_normal(n) * 4).astype(np.float32) / 4  # many ties
    vals, ids = [], []
    step = n // parts
    for s in range(parts):
        cv, ci, _ = oracle.topk(x[s * step:(s + 1) * step], None, k, id_base=s * step)
        vals.append(cv)
        ids.append(ci)
    mv, mi, nk = oracle.merge(np.stack(vals), np.stack(ids), k)
    gv, gi, gk = oracle.topk(x, None, k)
    assert nk == gk and np.array_equal(mi, gi) and np.array_equal(mv, gv)


def test_accept_rule(oracle):  # tools/fns_serve/fns_serve.cpp:492-508
    assert oracle.accept_len([5, 6, 7, 8], [5, 6, 7]) == 3
    assert oracle.accept_len([5, 6, 9, 8], [5, 6, 7]) == 2
    assert oracle.accept_len([4, 6, 7, 8], [5, 6, 7]) == 0
    assert oracle.accept_len([4], []) == 0


def test_verify_window_equals_sequential_sampling(oracle):
    """Column c must equal what the sequential path draws at generation index counter + c once draft[0 .. c)
    is in the history (src/engine.cu:745-748)."""
    w = wl.spec_windows(seed=4, windows=1, n_draft=3, vocab=5000, temperature=0.8)
    hist = np.array([1, 2, 3, 2], np.int32)
    p = w.params.copy()
    p["presence"] = 0.7
    tokens, a = oracle.verify_window(w.logits, w.draft[0], p, hist=hist)
    for c in range(4):
        pc = p.copy()
        pc["counter"] += c
        seq = oracle.sample_row(w.logits[c], pc, hist=np.concatenate([hist, w.draft[0][:c]]))
        assert tokens[c] == seq
    assert a == oracle.accept_len(tokens, w.draft[0])


def test_lookup_draft(oracle):  # include/fns/lookup.h:12-27
    h = [1, 2, 3, 4, 9, 9, 1, 2, 3, 4]
    assert list(oracle.lookup_draft(h, 3)) == [9, 9, 1]   # 4-gram (1,2,3,4) seen at 0: continuation
    assert list(oracle.lookup_draft([7, 8, 5, 7, 8], 4)) == [5, 7, 8]  # 2-gram
    assert list(oracle.lookup_draft([1, 2, 3], 2)) == []
    assert list(oracle.lookup_draft([1, 1, 1, 1, 1, 1], 2)) == [1]  # latest earlier occurrence: s = 1, one id left


def test_bf16_widening_is_exact(oracle):
    bits = np.arange(0, 65536, dtype=np.uint16)
    assert np.array_equal(oracle.widen_bf16(bits).view(np.uint32), bits.astype(np.uint32) << 16)


def test_workloads_are_deterministic():
    a, b = wl.session_batch(seed=2, rows=3, vocab=4096, history=64), wl.session_batch(seed=2, rows=3, vocab=4096, history=64)
    assert np.array_equal(a.logits, b.logits) and np.array_equal(a.masks, b.masks) and np.array_equal(a.params, b.params)
    w = wl.grammar_row()
    allowed = sum(bin(int(x)).count("1") for x in w.masks[0])
    assert 0.010 * w.vocab < allowed <= 0.0155 * w.vocab and w.row_bytes() == 643_124
    assert wl.single_row().row_bytes() == 609_796 and wl.session_batch(rows=1).row_bytes() == 634_932
    assert wl.large_vocab(rows=1).row_bytes() == 557_060


# ---- fixtures made by the reference's own kernels on a B200 -----------------------------------------------
def golden_files():
    return sorted(f for f in os.listdir(GOLDEN) if f.endswith(".json")) if os.path.isdir(GOLDEN) else []


@pytest.mark.parametrize("name", golden_files())
def test_oracle_reproduces_reference_outputs(oracle, name):
    from tests.golden.make_golden import replay_case

    with open(os.path.join(GOLDEN, name)) as f:
        doc = json.load(f)
    for case in doc["cases"]:
        replay_case(oracle, case)
