"""Parity of the CUDA sampler (through the C ABI) with the CPU oracle and with the reference's own kernels.

Bit-exact: greedy tokens, candidate lists (values and ids), accept lengths, presence arithmetic.
Stochastic picks: the same token as the checker for the same (seed, counter); a difference is accepted only
when the uniform lies within 1e-6 of a CDF boundary of the oracle's distribution (against the CPU oracle, whose
libm exp may differ from CUDA's in the last bit).  Against the reference's kernels the tokens must be identical.
"""
import ctypes

import numpy as np
import pytest

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.sampler import (BF16, F32, Sampler, SamplerError, cands_tensor, cands_to_numpy, make_params,
                                      params_to_device)

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
CDF_TOL = 1e-6
FMAX = np.finfo(np.float32).max


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ref():
    from oracle.binding import RefGpu

    return RefGpu()


def upload(w, dev):
    if w.bf16:
        lg = torch.from_numpy(w.logits.view(np.int16)).to(dev).view(torch.bfloat16)
    else:
        lg = torch.from_numpy(w.logits).to(dev)
    masks = None if w.masks is None else torch.from_numpy(w.masks.view(np.int32)).to(dev)
    hist = None if w.history is None else torch.from_numpy(w.history).to(dev)
    hl = None if w.history is None else torch.from_numpy(w.history_len).to(dev)
    return lg, masks, hist, hl


def run_rows(w, dev, k_cap=None, slices=0, max_history=4096, cluster_rows=None):
    """cluster_rows: None = the library's own choice of kernel for the row count; 0 = never the cluster kernel; n = the
    cluster kernel for calls of up to n rows."""
    k_cap = k_cap or w.k_cap
    s = Sampler(0, max_rows=w.rows, max_vocab=w.vocab, k_cap=k_cap, max_history=max_history)
    if slices:
        s.set_slices(slices)
    if cluster_rows is not None:
        s.set_cluster_rows(cluster_rows)
    lg, masks, hist, hl = upload(w, dev)
    pd = params_to_device(w.params, dev)
    out = torch.full((w.rows,), -7, dtype=torch.int32, device=dev)
    s.sample_rows(lg, pd, out, masks=masks, history=hist, history_len=hl)
    cd = cands_tensor(w.rows, k_cap, dev)
    s.select_rows(lg, pd, cd, masks=masks, history=hist, history_len=hl)
    torch.cuda.synchronize()
    s.device_status()
    s.close()
    return out.cpu().numpy(), cands_to_numpy(cd)


def check_against_oracle(oracle, w, tokens, cands, k_cap=None):
    """Candidates bit-exact; tokens equal, or the draw sits on a CDF boundary."""
    k_cap = k_cap or w.k_cap
    x = w.logits_f32()
    boundary = 0
    for r in range(w.rows):
        p = w.params[r:r + 1]
        m = None if w.masks is None else w.masks[r]
        h = None if w.history is None else w.history[r][: w.history_len[r]]
        tok, cv, ci, nk = oracle.sample_row(x[r], p, k_cap, m, h, want_cands=True)
        assert np.array_equal(cands["id"][r], ci), f"row {r}: candidate ids differ"
        # values bit for bit, except that the library reports a zero candidate as +0.0 (the reference's order
        # ties -0.0 and +0.0, and the key that carries the order has one pattern for both)
        assert np.array_equal(cands["value"][r].view(np.uint32), (cv + np.float32(0.0)).view(np.uint32)), \
            f"row {r}: candidate values differ"
        if tokens[r] != tok:
            k = 1 if p["temperature"][0] <= 0 else oracle.clamp_k(int(p["top_k"][0]), k_cap)
            _, q, keep, u, cdf = oracle.draw(cv[:k], ci[:k], nk, p, detail=True)
            assert p["temperature"][0] > 0 and np.min(np.abs(cdf[:keep] - u)) < CDF_TOL, \
                f"row {r}: token {tokens[r]} vs oracle {tok}, u={u}"
            boundary += 1
    assert boundary <= max(1, w.rows // 100)


# ---- the reference test's known answers (tests/sample_check.cu:102-131) -----------------------------------
def test_known_answers_of_the_reference_test(dev):
    n = 150_144
    x, mask, _ = wl.lcg_logits(n)
    s = Sampler(0, max_rows=1, max_vocab=n, k_cap=64)
    out = torch.zeros(1, dtype=torch.int32, device=dev)
    dx, dm = torch.from_numpy(x).to(dev), torch.from_numpy(mask.view(np.int32)).to(dev)
    s.sample_one(dx, make_params(1, temperature=0.0, top_k=20, top_p=0.95), out, mask=dm)
    assert out.item() == 0
    flat = np.ones(n, np.float32)
    flat[[149000, 70000, 1201, 1200]] = 5.0
    dflat = torch.from_numpy(flat).to(dev)
    s.sample_one(dflat, make_params(1), out)
    assert out.item() == 1200
    m2 = np.zeros((n + 31) // 32, np.uint32)
    for i in (70000, 149000):
        m2[i >> 5] |= np.uint32(1 << (i & 31))
    dm2 = torch.from_numpy(m2.view(np.int32)).to(dev)
    s.sample_one(dflat, make_params(1), out, mask=dm2)
    assert out.item() == 70000
    dflat.fill_(2.0)
    s.sample_one(dflat, make_params(1), out)
    assert out.item() == 0
    dm2.zero_()
    s.sample_one(dflat, make_params(1, temperature=1.0, top_k=20), out, mask=dm2)
    assert out.item() == -1
    s.device_status()


@pytest.mark.parametrize("case", [
    dict(top_k=20, top_p=0.95, temperature=1.0, masked=False),
    dict(top_k=0, top_p=1.0, temperature=0.7, masked=False),
    dict(top_k=20, top_p=1.0, temperature=1.0, masked=True),
])
def test_frequency_criterion_of_the_reference_test(dev, oracle, ref, case):
    """tests/sample_check.cu:63-75 on the CUDA path: 200 000 draws, seed 1234, counters 0 .. N-1, every kept
    candidate within 5 sigma, no draw outside the kept set; and the first 20 000 draws identical to the
    reference's kernels."""
    n, draws = 150_144, 200_000
    x, mask, _ = wl.lcg_logits(n)
    m = mask if case["masked"] else None
    dx = torch.from_numpy(x).to(dev)
    dm = None if m is None else torch.from_numpy(m.view(np.int32)).to(dev)
    p = make_params(draws, temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"], seed=1234)
    p["counter"] = np.arange(draws, dtype=np.uint64)
    s = Sampler(0, max_rows=draws, max_vocab=n, k_cap=64)
    s.set_slices(8)
    # one row of logits for every draw: candidates once, then the draw per counter
    cd = cands_tensor(1, 64, dev)
    s.select_rows(dx[None, :], params_to_device(p[:1], dev), cd, masks=None if dm is None else dm[None, :])
    out = torch.empty(draws, dtype=torch.int32, device=dev)
    s.finalize_rows(cd, 1, 64, draws, params_to_device(p, dev), out_tokens=out, row_stride=0)
    torch.cuda.synchronize()
    tokens = out.cpu().numpy()
    k = oracle.clamp_k(case["top_k"], 64)
    cv, ci, nk = oracle.topk(x, m, k)
    _, q, keep, _, _ = oracle.draw(cv, ci, nk, p[:1], detail=True)
    counts = np.bincount(tokens, minlength=n)
    assert counts[ci[:keep]].sum() == draws
    f = counts[ci[:keep]] / draws
    sd = np.sqrt(q[:keep] * (1 - q[:keep]) / draws) + 1e-12
    assert np.max(np.abs(f - q[:keep]) / sd) < 5.0
    rout = torch.empty(20_000, dtype=torch.int32, device=dev)
    ref.sample_counters(dx, dm, case["top_k"], case["top_p"], case["temperature"], 1234, 0, 20_000, rout)
    torch.cuda.synchronize()
    assert np.array_equal(rout.cpu().numpy(), tokens[:20_000])


# ---- the benchmark configurations against the oracle ------------------------------------------------------
def test_config1_single_row(dev, oracle):
    for seed in range(4):
        for greedy in (False, True):
            w = wl.single_row(seed=seed, greedy=greedy)
            check_against_oracle(oracle, w, *run_rows(w, dev))


def test_config2_grammar_row(dev, oracle):
    for seed in range(4):
        w = wl.grammar_row(seed=seed)
        check_against_oracle(oracle, w, *run_rows(w, dev))


@pytest.mark.parametrize("k_cap", [64, 128])
def test_config4_session_batch(dev, oracle, k_cap):
    w = wl.session_batch(seed=1, rows=256)
    check_against_oracle(oracle, w, *run_rows(w, dev, k_cap=k_cap), k_cap=k_cap)


def test_config5_large_vocab_bf16(dev, oracle):
    w = wl.large_vocab(seed=0, rows=64)
    check_against_oracle(oracle, w, *run_rows(w, dev))


def test_many_counters_on_one_row_against_the_oracle(dev, oracle):
    w = wl.grammar_row(seed=5)
    rows = 2000
    p = np.repeat(w.params, rows)
    p["counter"] = np.arange(rows, dtype=np.uint64) + np.uint64(1 << 40)
    p["seed"] = 99
    lg, masks, hist, hl = upload(w, dev)
    s = Sampler(0, max_rows=rows, max_vocab=w.vocab, k_cap=64, max_history=4096)
    s.set_slices(4)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    s.sample_rows(lg.expand(rows, -1), params_to_device(p, dev), out, masks=masks.expand(rows, -1),
                  history=hist.expand(rows, -1).contiguous(), history_len=hl.expand(rows).contiguous())
    torch.cuda.synchronize()
    tokens = out.cpu().numpy()
    _, cv, ci, nk = oracle.sample_row(w.logits[0], p[:1], 64, w.masks[0], w.history[0], want_cands=True)
    diff = 0
    for r in range(rows):
        tok, q, keep, u, cdf = oracle.draw(cv[:20], ci[:20], nk, p[r:r + 1], detail=True)
        if tok != tokens[r]:
            assert np.min(np.abs(cdf[:keep] - u)) < CDF_TOL
            diff += 1
    assert diff <= 2


# ---- against the reference's own kernels on the same GPU --------------------------------------------------
def test_tokens_identical_to_reference_kernels(dev, oracle, ref):
    """Compat mode (k_cap 64): identical tokens for greedy and sampled rows.  Rows are penalised on the host by
    the oracle's rule first, because the reference has a presence term only."""
    w = wl.session_batch(seed=3, rows=48)
    x = w.logits.copy()
    for r in range(w.rows):
        x[r] = oracle.penalize(x[r], w.history[r], None, 1.1, 0.5, 0.3)
    p = w.params.copy()
    p["temperature"][::5] = 0.0  # some greedy rows
    lg, masks, hist, hl = upload(w, dev)
    s = Sampler(0, max_rows=w.rows, max_vocab=w.vocab, k_cap=64)
    out = torch.empty(w.rows, dtype=torch.int32, device=dev)
    s.sample_rows(lg, params_to_device(p, dev), out, masks=masks, history=hist, history_len=hl)
    rout = torch.empty(w.rows, dtype=torch.int32, device=dev)
    ref.sample_rows(torch.from_numpy(x).to(dev), masks, p, rout)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), rout.cpu().numpy())


def test_candidate_lists_identical_to_reference_by_peeling(dev, ref):
    """The reference keeps its candidates in file-scope device arrays that cannot be read from outside; its
    ordered top-k is recovered with its own argmax: take the best, clear its mask bit, repeat."""
    w = wl.session_batch(seed=4, rows=3, history=16)
    w.params["repetition"], w.params["presence"], w.params["frequency"] = 1.0, 0.0, 0.0
    w.params["temperature"], w.params["top_k"] = 1.0, 24
    _, cands = run_rows(w, dev)
    lg, masks, _, _ = upload(w, dev)
    out = torch.empty(1, dtype=torch.int32, device=dev)
    for r in range(w.rows):
        m = w.masks[r].copy()
        ids = []
        for _ in range(24):
            ref.argmax(lg[r], out, torch.from_numpy(m.view(np.int32)).to(dev))
            t = int(out.item())
            if t < 0:
                break
            ids.append(t)
            m[t >> 5] &= np.uint32(~np.uint32(1 << (t & 31)))
        assert list(cands["id"][r][: len(ids)]) == ids
        assert np.all(cands["id"][r][len(ids):] == 0x7FFFFFFF)


def test_compat_entry_points_match_reference_kernels(dev, ref, library_path):
    """fns::k::sample / argmax exported by this library (mangled names, same signatures as src/kernels.cuh:67-75)
    against the reference's, on identical device buffers."""
    lib = ctypes.CDLL(library_path)
    vp, i32, u64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_float
    sample = lib._ZN3fns1k6sampleEPKfiPKjiffmmPiP11CUstream_st
    sample.argtypes, sample.restype = [vp, i32, vp, i32, f32, f32, u64, u64, vp, vp], None
    argmax = lib._ZN3fns1k6argmaxEPKfiPiP11CUstream_stPKj
    argmax.argtypes, argmax.restype = [vp, i32, vp, vp, vp], None
    w = wl.grammar_row(seed=9)
    lg, masks, _, _ = upload(w, dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    mine = torch.empty(64, dtype=torch.int32, device=dev)
    theirs = torch.empty(64, dtype=torch.int32, device=dev)
    for c in range(62):
        for tgt, fn in ((mine, sample), (theirs, ref.lib.fns_ref_sample)):
            fn(lg.data_ptr(), w.vocab, masks.data_ptr(), 0 if c % 2 else 33, 0.92, 0.85, 4321, c,
               tgt[c:c + 1].data_ptr(), st)
    argmax(lg.data_ptr(), w.vocab, mine[62:63].data_ptr(), st, None)
    ref.lib.fns_ref_argmax(lg.data_ptr(), w.vocab, theirs[62:63].data_ptr(), st, None)
    argmax(lg.data_ptr(), w.vocab, mine[63:64].data_ptr(), st, masks.data_ptr())
    ref.lib.fns_ref_argmax(lg.data_ptr(), w.vocab, theirs[63:64].data_ptr(), st, masks.data_ptr())
    torch.cuda.synchronize()
    assert np.array_equal(mine.cpu().numpy(), theirs.cpu().numpy())


def test_presence_entry_points_match_reference_kernels(dev, ref):
    lib = Sampler(0, 1, 1024).lib
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = np.random.default_rng(8)
    n = 151_936
    x = torch.from_numpy(g.standard_normal(n).astype(np.float32) * 3).to(dev)
    seen = torch.zeros(n, device=dev)
    tokens = torch.from_numpy(g.integers(0, n, size=32).astype(np.int32)).to(dev)
    tokens[3] = -1  # ignored (src/kernels.cu:730)
    a, b = x.clone(), x.clone()
    sa, sb = seen.clone(), seen.clone()
    assert lib.fns_b200_presence_mark_n(sa.data_ptr(), tokens.data_ptr(), 32, st) == 0
    ref.presence_mark_n(sb, tokens, 32)
    assert lib.fns_b200_presence_mark(sa.data_ptr(), tokens[:1].data_ptr(), st) == 0
    ref.presence_mark(sb, tokens[:1])
    assert lib.fns_b200_presence_apply(a.data_ptr(), sa.data_ptr(), n, 0.7, st) == 0
    ref.presence_apply(b, sb, 0.7)
    draft = tokens[10:17].contiguous()
    assert lib.fns_b200_presence_apply_col(a.data_ptr(), sa.data_ptr(), draft.data_ptr(), 5, n, 1.3, st) == 0
    ref.presence_apply_col(b, sb, draft, 5, 1.3)
    io_a = torch.tensor([9, 9, -1, 0], dtype=torch.int32, device=dev)
    io_b = io_a.clone()
    assert lib.fns_b200_io_advance(io_a.data_ptr(), 41, st) == 0
    ref.io_advance(io_b, 41)
    torch.cuda.synchronize()
    assert torch.equal(sa, sb) and torch.equal(a.view(torch.int32), b.view(torch.int32)) and torch.equal(io_a, io_b)
    assert io_a.tolist() == [0, 41, -1, 0]


# ---- speculative verification ------------------------------------------------------------------------------
def test_config3_greedy_accept_10000_trials(dev, oracle, ref):
    """10 000 seeded trials: windows of 4 rows (3 draft positions + bonus) cut from a pool of rows; drafts equal
    the row's argmax with probability 0.7.  Accept length and every token bit-exact against the oracle, and a
    sample of windows against the reference's per-row argmax + the host accept rule."""
    pool = wl.spec_windows(seed=11, windows=50, n_draft=3)  # 200 rows
    lg = torch.from_numpy(pool.logits).to(dev)
    arg = pool.logits.argmax(axis=1).astype(np.int32)
    g = wl.rng(12)
    s = Sampler(0, max_rows=200, max_vocab=pool.vocab, k_cap=64)
    trials = 0
    rtok = torch.empty(4, dtype=torch.int32, device=dev)
    for batch in range(200):
        # 50 windows per call, each at its own 4-row block; drafts re-drawn per batch
        match = g.random((50, 3)) < 0.7
        draft = np.where(match, arg.reshape(50, 4)[:, :3], g.integers(0, pool.vocab, size=(50, 3))).astype(np.int32)
        p = make_params(50, temperature=0.0)
        toks = torch.empty(200, dtype=torch.int32, device=dev)
        acc = torch.empty(50, dtype=torch.int32, device=dev)
        s.verify_accept(lg, torch.from_numpy(draft).to(dev), params_to_device(p, dev), toks, acc)
        torch.cuda.synchronize()
        toks_h, acc_h = toks.cpu().numpy().reshape(50, 4), acc.cpu().numpy()
        assert np.array_equal(toks_h, arg.reshape(50, 4))  # greedy: first index of the maximum
        for wdw in range(50):
            assert acc_h[wdw] == oracle.accept_len(toks_h[wdw], draft[wdw])
        if batch < 3:
            for wdw in range(0, 50, 7):
                for c in range(4):
                    ref.argmax(lg[wdw * 4 + c], rtok[c:c + 1])
                torch.cuda.synchronize()
                rt = rtok.cpu().numpy()
                assert np.array_equal(rt, toks_h[wdw]) and acc_h[wdw] == oracle.accept_len(rt, draft[wdw])
        trials += 50
    assert trials == 10_000
    s.device_status()


def test_sampled_verification_with_presence_matches_sequential_path(dev, oracle, ref):
    """Column c of a window must draw what the sequential path draws at counter + c with draft[0 .. c) counted as
    seen (src/engine.cu:745-757): checked against the oracle and against the reference's presence_apply_col +
    sample on a copy of the logits."""
    w = wl.spec_windows(seed=21, windows=6, n_draft=3, temperature=0.9)
    w.params["presence"] = 0.8
    w.params["top_k"] = 30
    hist = wl.rng(5).integers(0, w.vocab, size=(6, 300), dtype=np.int32)
    hl = np.array([300, 0, 17, 300, 1, 255], np.int32)
    w.draft[2, 1] = w.draft[2, 0]  # a repeated draft id
    lg = torch.from_numpy(w.logits).to(dev)
    s = Sampler(0, max_rows=24, max_vocab=w.vocab, k_cap=64, max_history=512)
    toks = torch.empty(24, dtype=torch.int32, device=dev)
    acc = torch.empty(6, dtype=torch.int32, device=dev)
    s.verify_accept(lg, torch.from_numpy(w.draft).to(dev), params_to_device(w.params, dev), toks, acc,
                    history=torch.from_numpy(hist).to(dev), history_len=torch.from_numpy(hl).to(dev))
    torch.cuda.synchronize()
    s.device_status()
    toks_h, acc_h = toks.cpu().numpy().reshape(6, 4), acc.cpu().numpy()
    rout = torch.empty(1, dtype=torch.int32, device=dev)
    for wdw in range(6):
        exp, a = oracle.verify_window(w.logits[wdw * 4:(wdw + 1) * 4], w.draft[wdw], w.params[wdw:wdw + 1],
                                      hist=hist[wdw][: hl[wdw]])
        assert np.array_equal(toks_h[wdw], exp) and acc_h[wdw] == a
        seen = np.zeros(w.vocab, np.float32)
        seen[hist[wdw][: hl[wdw]]] = 1.0
        dseen, ddraft = torch.from_numpy(seen).to(dev), torch.from_numpy(w.draft[wdw]).to(dev)
        for c in range(4):
            row = lg[wdw * 4 + c].clone()
            ref.presence_apply_col(row, dseen, ddraft, c, 0.8)
            ref.sample(row, None, 30, float(w.params["top_p"][wdw]), 0.9, int(w.params["seed"][wdw]),
                       int(w.params["counter"][wdw]) + c, rout)
            assert rout.item() == toks_h[wdw, c]


# ---- geometry independence, edge cases ----------------------------------------------------------------------
def test_results_do_not_depend_on_the_launch_geometry(dev):
    w = wl.session_batch(seed=6, rows=12)
    base_t, base_c = run_rows(w, dev)
    for slices in (1, 3, 7, 16, 64, 128):
        t, c = run_rows(w, dev, slices=slices)
        assert np.array_equal(t, base_t) and np.array_equal(c, base_c), slices


@pytest.mark.parametrize("n", [1, 2, 31, 32, 33, 127, 1187, 1188, 4000, 4097, 20_000, 65_537])
def test_small_and_ragged_vocabularies(dev, oracle, n):
    g = wl.rng(n)
    rows = 5
    x = g.standard_normal((rows, n), dtype=np.float32)
    masks = np.stack([wl.random_mask(g, n, 0.7) for _ in range(rows)])
    masks[0] = 0                                             # nothing allowed
    masks[1] = 0
    masks[1][(n - 1) >> 5] = np.uint32(1 << ((n - 1) & 31))  # only the last id
    hist = g.integers(-3, n + 3, size=(rows, 40), dtype=np.int32)
    p = make_params(rows, temperature=0.8, top_k=0, top_p=0.9, repetition=1.3, presence=0.2, frequency=0.1, seed=n)
    p["temperature"][2] = 0.0
    w = wl.Workload("small", x, p, masks, hist, np.array([40, 40, 0, 7, 40], np.int32))
    tokens, cands = run_rows(w, dev, max_history=64)
    assert tokens[0] == -1 and tokens[1] == n - 1
    check_against_oracle(oracle, w, tokens, cands)


def test_special_values(dev, oracle):
    """NaN and infinities are never candidates; +-FLT_MAX are; -0.0 ties +0.0 by index (src/kernels.cu:629-639)."""
    n = 5000
    x = np.full((6, n), -3.0, np.float32)
    x[0, 10], x[0, 20], x[0, 30] = np.inf, np.nan, 2.0
    x[1, :] = -np.inf
    x[1, 77] = -FMAX
    x[2, 5], x[2, 3] = FMAX, np.inf
    x[3, :] = np.float32(-0.0)
    x[3, 40] = np.float32(0.0)
    x[4, :] = np.nan
    x[5, ::2] = np.float32(-0.0)
    x[5, 1::2] = np.float32(0.0)
    p = make_params(6, temperature=1.0, top_k=8)
    p["temperature"][:5] = 0.0
    w = wl.Workload("special", x, p)
    tokens, cands = run_rows(w, dev)
    assert list(tokens[:5]) == [30, 77, 5, 0, -1]
    assert list(cands["id"][5][:8]) == list(range(8))
    check_against_oracle(oracle, w, tokens, cands)


def test_unaligned_rows_take_the_scalar_path(dev, oracle):
    """A row stride that is not a multiple of 16 bytes cannot use 128-bit loads."""
    w = wl.session_batch(seed=7, rows=6, vocab=10_001, history=32)
    buf = torch.zeros((6, 10_003), dtype=torch.float32, device=dev)
    buf[:, :10_001] = torch.from_numpy(w.logits).to(dev)
    _, masks, hist, hl = upload(w, dev)
    s = Sampler(0, max_rows=6, max_vocab=10_001, k_cap=64)
    out = torch.empty(6, dtype=torch.int32, device=dev)
    s.sample_rows(buf, params_to_device(w.params, dev), out, masks=masks, history=hist, history_len=hl, vocab=10_001)
    cd = cands_tensor(6, 64, dev)
    s.select_rows(buf, params_to_device(w.params, dev), cd, masks=masks, history=hist, history_len=hl, vocab=10_001)
    torch.cuda.synchronize()
    check_against_oracle(oracle, w, out.cpu().numpy(), cands_to_numpy(cd))
    # bf16 on an odd stride
    wb = wl.large_vocab(seed=2, rows=3, vocab=9_999)
    bb = torch.zeros((3, 10_001), dtype=torch.bfloat16, device=dev)
    bb[:, :9_999] = torch.from_numpy(wb.logits.view(np.int16)).to(dev).view(torch.bfloat16)
    s2 = Sampler(0, max_rows=3, max_vocab=9_999, k_cap=1024)
    out2 = torch.empty(3, dtype=torch.int32, device=dev)
    dm = torch.from_numpy(wb.masks.view(np.int32)).to(dev)
    s2.sample_rows(bb, params_to_device(wb.params, dev), out2, masks=dm, vocab=9_999)
    cd2 = cands_tensor(3, 1024, dev)
    s2.select_rows(bb, params_to_device(wb.params, dev), cd2, masks=dm, vocab=9_999)
    torch.cuda.synchronize()
    check_against_oracle(oracle, wb, out2.cpu().numpy(), cands_to_numpy(cd2))


def test_adversarial_orders_force_repeated_compaction(dev, oracle):
    """Ascending logits make every element beat the running threshold; all-equal logits make every key differ
    only in the id bits; a history that covers a whole slice fills the penalty table."""
    n = 151_936
    x = np.empty((4, n), np.float32)
    x[0] = np.linspace(-8, 8, n, dtype=np.float32)
    x[1] = np.linspace(8, -8, n, dtype=np.float32)
    x[2] = 1.25
    x[3] = np.repeat(np.arange(n // 64, dtype=np.float32), 64)[:n]
    hist = np.tile(np.arange(4096, dtype=np.int32) + 60_000, (4, 1))
    hist[3] = 7  # one id 4096 times
    p = make_params(4, temperature=0.7, top_k=64, top_p=0.99, repetition=1.2, presence=0.4, frequency=0.01)
    w = wl.Workload("adversarial", x, p, None, hist, np.full(4, 4096, np.int32))
    for slices in (0, 3, 40):
        tokens, cands = run_rows(w, dev, slices=slices)
        check_against_oracle(oracle, w, tokens, cands)


def test_history_of_the_largest_logits_with_repeats_and_every_penalty_sign(dev, oracle):
    """The history holds exactly the ids a sampler would pick: the largest logits of the row, many of them several
    times.  Unmasked rows stream these ids at their raw value (they must not count as witnesses for the bound);
    the occurrence counts decide which of them stay candidates; a negative frequency penalty raises a value with
    every occurrence; a history longer than one round of the scatter takes the slow publishing path."""
    g = wl.rng(123)
    rows, n = 6, 151_936
    x = wl.gaussian_logits(g, rows, n, 2.5)
    top = np.argsort(-x, axis=1)[:, :400].astype(np.int32)
    hist = np.zeros((rows, 6000), np.int32)
    hlen = np.zeros(rows, np.int32)
    for r in range(rows):
        reps = g.integers(1, 9, size=400)
        ids = np.repeat(top[r], reps)
        g.shuffle(ids)
        ids = ids[: min(ids.size, 6000 if r % 2 else 1500)]
        hist[r, : ids.size] = ids
        hlen[r] = ids.size
    p = make_params(rows, temperature=0.8, top_k=64, top_p=0.97, repetition=1.15, presence=0.6, frequency=0.25)
    p["frequency"][2] = -0.2   # more occurrences raise the value
    p["presence"][3] = -1.5    # penalised above raw
    p["repetition"][4] = 0.8
    p["frequency"][5] = 0.0    # no counts needed
    p["top_k"][1] = 7
    p["seed"] = np.arange(rows, dtype=np.uint64) + 5
    w = wl.Workload("hot_history", x, p, None, hist, hlen)
    for slices in (0, 1, 5):
        tokens, cands = run_rows(w, dev, slices=slices, max_history=6000)
        check_against_oracle(oracle, w, tokens, cands)
    # the same under a mask that cuts the row into allowed and excluded runs
    w.masks = np.stack([wl.run_mask(g, n, 0.6, 20) for _ in range(rows)])
    tokens, cands = run_rows(w, dev, max_history=6000)
    check_against_oracle(oracle, w, tokens, cands)


def test_history_too_long_for_a_whole_row_falls_back_to_slices(dev, oracle):
    """60,000 history ids per row do not fit the shared memory of a whole-row block: the plan cuts the rows."""
    g = wl.rng(5)
    rows, n, h = 6, 151_936, 60_000
    x = wl.gaussian_logits(g, rows, n, 2.5)
    hist = g.integers(0, n, size=(rows, h), dtype=np.int32)
    hlen = np.full(rows, h, np.int32)
    hlen[1] = 12_345
    p = make_params(rows, temperature=0.8, top_k=50, top_p=0.95, repetition=1.1, presence=0.4, frequency=0.2, seed=3)
    w = wl.Workload("long_history", x, p, None, hist, hlen)
    s = Sampler(0, max_rows=rows, max_vocab=n, k_cap=64, max_history=h)
    assert s.plan(0, n, rows, h)["slices"] > 1
    s.close()
    tokens, cands = run_rows(w, dev, max_history=h)
    check_against_oracle(oracle, w, tokens, cands)


def test_whole_row_blocks_at_batch_sizes_around_the_sm_count(dev, oracle):
    """At 148 rows and more a row is one 512-thread block; just below, rows are cut into slices."""
    for rows in (147, 149, 300):
        w = wl.session_batch(seed=40 + rows, rows=rows, vocab=50_000, history=300)
        tokens, cands = run_rows(w, dev)
        check_against_oracle(oracle, w, tokens, cands)


# ---- vocabulary shards on one GPU (the exchange itself is tested with gloo on CPU and nccl on >1 GPU) -------
@pytest.mark.parametrize("shards", [2, 4, 8])
def test_vocab_shards_merge_to_the_unsharded_answer(dev, oracle, shards):
    w = wl.large_vocab(seed=3, rows=8)
    lg, masks, _, _ = upload(w, dev)
    pd = params_to_device(w.params, dev)
    s = Sampler(0, max_rows=8, max_vocab=w.vocab, k_cap=1024)
    full = cands_tensor(8, 1024, dev)
    s.select_rows(lg, pd, full, masks=masks)
    step = w.vocab // shards
    parts = []
    for g in range(shards):
        part = cands_tensor(8, 1024, dev)
        s.select_rows(lg[:, g * step:(g + 1) * step], pd, part, id_base=g * step,
                      masks=masks[:, g * step // 32:(g + 1) * step // 32], vocab=step)
        parts.append(part)
    gathered = torch.stack(parts, dim=1).contiguous()  # [rows][shards][k_cap]
    out = torch.empty(8, dtype=torch.int32, device=dev)
    merged = cands_tensor(8, 1024, dev)
    s.finalize_rows(gathered, shards, 1024, 8, pd, out_tokens=out, out_cands=merged)
    direct = torch.empty(8, dtype=torch.int32, device=dev)
    s.sample_rows(lg, pd, direct, masks=masks)
    torch.cuda.synchronize()
    s.device_status()
    assert torch.equal(merged, full) and torch.equal(out, direct)
    check_against_oracle(oracle, w, out.cpu().numpy(), cands_to_numpy(merged))


@pytest.mark.parametrize("shards", [2, 8])
def test_vocab_shards_that_are_nothing_alike(dev, oracle, shards):
    """The merge prunes the lists by the smallest of their (k / lists)-th keys before it merges them.  Rows whose
    best keys all sit in one shard, whose other shards hold a handful of allowed ids or none, small k and greedy
    rows must come out as the unsharded call gives them."""
    w = wl.large_vocab(seed=4, rows=6)
    step = w.vocab // shards
    x = wl.bf16_bits_to_f32(w.logits)
    x[0, :step] += np.float32(20.0)                      # every candidate of row 0 comes from shard 0
    masks = w.masks.copy()
    words = step // 32
    masks[1, words:2 * words] = 0
    masks[1, words] = np.uint32(0x0000ffff)              # shard 1 of row 1: sixteen allowed ids
    masks[2, words:] = 0                                 # row 2: only shard 0 has allowed ids
    masks[5, :] = 0
    masks[5, ::27] = np.uint32(0x00010000)               # row 5: about 300 allowed ids in all
    p = w.params.copy()
    p["top_k"][3] = 5
    p["temperature"][4] = 0.0
    w2 = wl.Workload("skewed_shards", wl.f32_to_bf16_bits(x), p, masks, None, None, bf16=True, k_cap=1024)
    lg, mk, _, _ = upload(w2, dev)
    pd = params_to_device(p, dev)
    s = Sampler(0, max_rows=6, max_vocab=w.vocab, k_cap=1024)
    full = cands_tensor(6, 1024, dev)
    s.select_rows(lg, pd, full, masks=mk)
    parts = []
    for g in range(shards):
        part = cands_tensor(6, 1024, dev)
        s.select_rows(lg[:, g * step:(g + 1) * step], pd, part, id_base=g * step, masks=mk[:, g * words:(g + 1) * words], vocab=step)
        parts.append(part)
    gathered = torch.stack(parts, dim=1).contiguous()
    out = torch.empty(6, dtype=torch.int32, device=dev)
    merged = cands_tensor(6, 1024, dev)
    s.finalize_rows(gathered, shards, 1024, 6, pd, out_tokens=out, out_cands=merged)
    direct = torch.empty(6, dtype=torch.int32, device=dev)
    s.sample_rows(lg, pd, direct, masks=mk)
    torch.cuda.synchronize()
    s.device_status()
    assert torch.equal(merged, full) and torch.equal(out, direct)
    check_against_oracle(oracle, w2, out.cpu().numpy(), cands_to_numpy(merged))


# ---- error behaviour ---------------------------------------------------------------------------------------
def test_capacity_and_argument_errors(dev):
    s = Sampler(0, max_rows=2, max_vocab=1000, k_cap=64, max_history=16)
    lg = torch.zeros((2, 1000), device=dev)
    pd = params_to_device(make_params(2), dev)
    out = torch.empty(2, dtype=torch.int32, device=dev)
    with pytest.raises(SamplerError) as e:
        s.sample_rows(torch.zeros((3, 1000), device=dev), params_to_device(make_params(3), dev), out)
    assert e.value.code == 3
    with pytest.raises(SamplerError) as e:
        s.sample_rows(torch.zeros((2, 2000), device=dev), pd, out)
    assert e.value.code == 3
    hist = torch.zeros((2, 32), dtype=torch.int32, device=dev)
    with pytest.raises(SamplerError) as e:
        s.sample_rows(lg, pd, out, history=hist, history_len=torch.zeros(2, dtype=torch.int32, device=dev))
    assert e.value.code == 3
    with pytest.raises(SamplerError) as e:
        s.sample_rows(lg, pd, out, history=hist[:, :8].contiguous(), history_len=None)
    assert e.value.code == 1
    s.sample_rows(lg, pd, out)  # the handle still works
    torch.cuda.synchronize()
    assert out.tolist() == [0, 0]
