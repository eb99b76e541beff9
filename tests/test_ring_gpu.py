"""The bulk-copy kernel (k_ring) and the cluster kernel (k_cluster) against the oracle on the inputs that stress them.

Calls of many rows take k_ring when they have no mask, and always when k_cap exceeds 512 (then also under a mask);
small batches with k_cap up to 128 take k_cluster.  The cases below pick k_cap and masks accordingly and say which
kernel a small batch is meant for (run_rows' cluster_rows).  Everything goes through the C ABI; candidates must be
bit-exact and tokens equal (or on a CDF boundary within 1e-6), as in test_parity_gpu.py.
"""
import numpy as np
import pytest

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.sampler import make_params

from .test_parity_gpu import check_against_oracle, dev, run_rows  # noqa: F401  (dev is a fixture)

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 15, 16, 17, 33, 1187, 4097, 8192, 8193, 20_000, 65_537])
@pytest.mark.parametrize("bf16", [False, True])
def test_ragged_vocabularies_masked_and_unmasked(dev, oracle, n, bf16):
    """Rows that end inside a 16-byte vector, inside a cell, exactly on a stage, one element into the next stage."""
    g = wl.rng(1000 + n)
    rows = 6
    x = g.standard_normal((rows, n), dtype=np.float32) * np.float32(2.0)
    masks = np.stack([wl.random_mask(g, n, 0.6) for _ in range(rows)])
    masks[0] = 0                                             # nothing allowed
    masks[1] = 0
    masks[1][(n - 1) >> 5] = np.uint32(1 << ((n - 1) & 31))  # only the last id
    hist = g.integers(-3, n + 3, size=(rows, 48), dtype=np.int32)
    hist[4, :8] = n - 1                                      # the last id, several times
    p = make_params(rows, temperature=0.8, top_k=0, top_p=0.9, repetition=1.3, presence=0.2, frequency=0.1, seed=n)
    p["temperature"][2] = 0.0
    logits = wl.f32_to_bf16_bits(x) if bf16 else x
    hl = np.array([48, 48, 0, 7, 48, 48], np.int32)
    w = wl.Workload("ragged", logits, p, masks, hist, hl, bf16=bf16, k_cap=1024)
    tokens, cands = run_rows(w, dev, max_history=64)         # k_cap 1024: k_ring also under a mask
    assert tokens[0] == -1 and tokens[1] == n - 1
    check_against_oracle(oracle, w, tokens, cands)
    w2 = wl.Workload("ragged_unmasked", logits, p, None, hist, hl, bf16=bf16, k_cap=64)
    check_against_oracle(oracle, w2, *run_rows(w2, dev, max_history=64, cluster_rows=0))   # k_ring
    check_against_oracle(oracle, w2, *run_rows(w2, dev, max_history=64, cluster_rows=6))   # six clusters
    w3 = wl.Workload("ragged_masked_k64", logits, p, masks, hist, hl, bf16=bf16, k_cap=64)
    check_against_oracle(oracle, w3, *run_rows(w3, dev, max_history=64, cluster_rows=6))   # six clusters, under the masks
    check_against_oracle(oracle, w3, *run_rows(w3, dev, max_history=64, cluster_rows=0))   # k_select


def test_equal_values_take_the_careful_walk(dev, oracle):
    """Rows of one value (and of long runs of one value) flag every cell: the work list and the candidate buffer
    overflow and every cell is offered again with compaction.  Greedy rows must still return the smallest id."""
    n = 151_936
    x = np.empty((6, n), np.float32)
    x[0] = 1.25
    x[1] = 0.0
    x[2] = np.repeat(np.arange(n // 64, dtype=np.float32), 64)[:n]
    x[3] = np.linspace(-8, 8, n, dtype=np.float32)
    x[4] = np.linspace(8, -8, n, dtype=np.float32)
    x[5] = -3.0
    x[5, 77_777] = -3.0 + 1e-3
    hist = np.tile(np.arange(3000, dtype=np.int32) * 50, (6, 1))
    hl = np.array([3000, 0, 3000, 3000, 0, 3000], np.int32)
    for temperature in (0.0, 0.7):
        p = make_params(6, temperature=temperature, top_k=64, top_p=0.99, repetition=1.2, presence=0.4, frequency=0.01,
                        seed=11)
        w = wl.Workload("equal", x, p, None, hist, hl)
        for cluster_rows in (0, 6):  # k_ring, and six clusters
            tokens, cands = run_rows(w, dev, cluster_rows=cluster_rows)
            check_against_oracle(oracle, w, tokens, cands)
            if temperature == 0.0:
                assert tokens[1] == 0  # no history: the first of all the equal values
    # the same rows under masks go through k_select: a greedy row whose work list overflows takes its careful walk
    masks = np.stack([wl.run_mask(wl.rng(3 + r), n, 0.7, 20) for r in range(6)])
    p = make_params(6, temperature=0.0, repetition=1.2, presence=0.4, frequency=0.01)
    w = wl.Workload("equal_masked", x, p, masks, hist, hl)
    check_against_oracle(oracle, w, *run_rows(w, dev, cluster_rows=0))
    check_against_oracle(oracle, w, *run_rows(w, dev, cluster_rows=6))


def test_more_owned_history_ids_than_the_registers_hold(dev, oracle):
    """5,000 distinct history ids per row: the first 2,048 owned ids ride in registers and take their logits from the
    ring, the rest are fetched from global memory."""
    g = wl.rng(77)
    rows, n, h = 6, 151_936, 5000
    x = wl.gaussian_logits(g, rows, n, 2.5)
    top = np.argsort(-x, axis=1)[:, :h].astype(np.int32)   # the largest logits: every one of them matters
    hist = top.copy()
    for r in range(rows):
        g.shuffle(hist[r])
    hist[:, ::7] = hist[:, 1::7][:, : hist[:, ::7].shape[1]]  # repeats
    p = make_params(rows, temperature=0.9, top_k=64, top_p=0.98, repetition=1.1, presence=0.3, frequency=0.2, seed=5)
    p["temperature"][0] = 0.0
    p["frequency"][3] = -0.1
    w = wl.Workload("many_owned", x, p, None, hist, np.full(rows, h, np.int32))
    check_against_oracle(oracle, w, *run_rows(w, dev, max_history=h, cluster_rows=0))
    check_against_oracle(oracle, w, *run_rows(w, dev, max_history=h, cluster_rows=6))


@pytest.mark.parametrize("k", [513, 700, 1024])
def test_k_beyond_the_thread_count(dev, oracle, k):
    """k > 512: the bound comes from the cell maxima; fp32 rows with and without a mask, with history."""
    g = wl.rng(k)
    rows, n = 7, 100_003
    x = wl.gaussian_logits(g, rows, n, 3.0)
    masks = np.stack([wl.random_mask(g, n, d) for d in (1.0, 0.5, 0.02, 0.9, 0.004, 0.3, 0.7)])
    hist = g.integers(0, n, size=(rows, 1500), dtype=np.int32)
    p = make_params(rows, temperature=1.0, top_k=k, top_p=0.95, min_p=0.001, repetition=1.05, presence=0.1, frequency=0.05,
                    seed=k)
    for m in (masks, None):
        w = wl.Workload("big_k", x, p, m, hist, np.full(rows, 1500, np.int32), k_cap=1024)
        check_against_oracle(oracle, w, *run_rows(w, dev, max_history=1500))


def test_special_values_in_whole_rows(dev, oracle):
    """NaN and infinities never win, +-FLT_MAX can, -0.0 ties +0.0 by index (src/kernels.cu:629-639), at the full
    vocabulary where the values are spread over many stages."""
    n = 151_936
    fmax = np.finfo(np.float32).max
    x = np.full((6, n), -3.0, np.float32)
    x[0, 10], x[0, 20], x[0, 100_000] = np.inf, np.nan, 2.0
    x[1, :] = -np.inf
    x[1, 150_077] = -fmax
    x[2, 90_005], x[2, 3] = fmax, np.inf
    x[3, :] = np.float32(-0.0)
    x[3, 40_000] = np.float32(0.0)
    x[4, :] = np.nan
    x[5, ::2] = np.inf
    x[5, 1::2] = np.float32(1.0)
    p = make_params(6, temperature=1.0, top_k=8)
    p["temperature"][:5] = 0.0
    w = wl.Workload("special", x, p)
    for cluster_rows in (0, 6):  # k_ring, and six clusters
        tokens, cands = run_rows(w, dev, cluster_rows=cluster_rows)
        assert list(tokens[:5]) == [100_000, 150_077, 90_005, 0, -1]
        check_against_oracle(oracle, w, tokens, cands)


# ---- one to four rows: the cluster kernel (16 CTAs per row, candidates meet in distributed shared memory) -----------
@pytest.mark.parametrize("n", [1, 33, 127, 2048, 2049, 20_000, 151_936, 262_144, 524_288])
@pytest.mark.parametrize("bf16", [False, True])
def test_few_rows_of_any_length(dev, oracle, n, bf16):
    """Slices that are empty, partly filled, ragged at the end; masks, histories with repeats; k_cap 64 and 128."""
    g = wl.rng(7000 + n)
    for rows, k_cap in ((1, 64), (3, 128), (4, 64)):
        x = g.standard_normal((rows, n), dtype=np.float32) * np.float32(2.5)
        masks = np.stack([wl.random_mask(g, n, d) for d in (0.6, 1.0, 0.02, 0.3)[:rows]])
        hist = g.integers(-2, n + 2, size=(rows, 300), dtype=np.int32)
        hist[0, :50] = hist[0, 0]
        p = make_params(rows, temperature=0.9, top_k=0, top_p=0.95, min_p=0.01, repetition=1.2, presence=0.3, frequency=0.2, seed=n)
        p["temperature"][rows - 1] = 0.0
        logits = wl.f32_to_bf16_bits(x) if bf16 else x
        w = wl.Workload("few", logits, p, masks, hist, np.array([300, 0, 7, 300][:rows], np.int32), bf16=bf16, k_cap=k_cap)
        check_against_oracle(oracle, w, *run_rows(w, dev, max_history=300))


def test_few_rows_with_equal_values_and_hot_histories(dev, oracle):
    """Rows of one value overflow every CTA's region, so every CTA reduces its slice to its own best k and the lists are
    merged; a history that holds the row's largest logits many times exercises the occurrence count."""
    n = 151_936
    g = wl.rng(99)
    x = np.empty((4, n), np.float32)
    x[0] = 1.25
    x[1] = np.repeat(np.arange(n // 512 + 1, dtype=np.float32), 512)[:n]
    x[2:] = wl.gaussian_logits(g, 2, n, 2.5)
    top = np.argsort(-x[2])[:200].astype(np.int32)
    hist = np.zeros((4, 6000), np.int32)
    hist[:] = np.tile(np.arange(6000, dtype=np.int32) * 37 % n, (4, 1))
    hist[2, :2000] = np.repeat(top, 10)
    hist[3, :3000] = np.tile(top[:30], 100)
    hl = np.array([6000, 0, 2500, 5100], np.int32)  # (lengths that end inside a batch of sixteen ids per thread, and of four)
    for temperature in (0.0, 0.8):
        p = make_params(4, temperature=temperature, top_k=64, top_p=0.98, repetition=1.15, presence=0.5, frequency=0.25, seed=4)
        p["frequency"][3] = -0.05  # more occurrences raise the value: every owned id needs its count
        w = wl.Workload("few_equal", x, p, None, hist, hl)
        check_against_oracle(oracle, w, *run_rows(w, dev, max_history=6000))


def test_few_rows_under_masks_that_leave_no_bound(dev, oracle):
    """A mask that allows a few dozen to a few thousand ids, all in one or two slices: too few witnesses for a bound.
    With fewer than k allowed ids every one is a candidate and the CTA that holds them sends only its own best k; with
    more, the CTA's own thread maxima give the row its bound."""
    n = 151_936
    g = wl.rng(123)
    rows = 12
    x = wl.gaussian_logits(g, rows, n, 2.5)
    masks = np.zeros((rows, (n + 31) // 32), np.uint32)
    for r in range(rows):
        start = int(g.integers(0, n - 4000))
        if r >= 9:  # one contiguous block: few threads see an allowed id at all (150 ids: 38 threads, fewer than k)
            ids = start + np.arange((150, 200, 400)[r - 9])
        else:
            ids = start + np.sort(g.choice(3000, size=(30, 130, 200, 600, 1500, 2600)[r % 6], replace=False))
        np.bitwise_or.at(masks[r], ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
    hist = g.integers(0, n, size=(rows, 256), dtype=np.int32)
    p = make_params(rows, temperature=0.8, top_k=64, top_p=0.97, repetition=1.1, presence=0.2, frequency=0.1, seed=9)
    p["temperature"][::3] = 0.0
    w = wl.Workload("no_bound", x, p, masks, hist, np.full(rows, 256, np.int32))
    check_against_oracle(oracle, w, *run_rows(w, dev, max_history=256, cluster_rows=12))
    check_against_oracle(oracle, w, *run_rows(w, dev, max_history=256, cluster_rows=0))


def test_one_verification_window_of_four_columns(dev, oracle):
    """Engine::verify's shape (src/engine.cu:745-757): one window, three draft ids, masks per column, history."""
    sw = wl.spec_windows(seed=31, windows=1, n_draft=3, temperature=0.85)
    sw.params["presence"], sw.params["top_k"] = 0.9, 30
    g = wl.rng(32)
    masks = np.stack([wl.random_mask(g, sw.vocab, 0.5) for _ in range(4)])
    hist = g.integers(0, sw.vocab, size=(1, 64), dtype=np.int32)
    from flintnsteel_b200.sampler import Sampler, params_to_device

    s = Sampler(0, max_rows=4, max_vocab=sw.vocab, k_cap=64, max_history=64)
    toks = torch.empty(4, dtype=torch.int32, device=dev)
    acc = torch.empty(1, dtype=torch.int32, device=dev)
    s.verify_accept(torch.from_numpy(sw.logits).to(dev), torch.from_numpy(sw.draft).to(dev), params_to_device(sw.params, dev),
                    toks, acc, masks=torch.from_numpy(masks.view(np.int32)).to(dev), history=torch.from_numpy(hist).to(dev),
                    history_len=torch.tensor([64], dtype=torch.int32, device=dev))
    torch.cuda.synchronize()
    s.device_status()
    et, ea = oracle.verify_window(sw.logits, sw.draft[0], sw.params, masks=masks, hist=hist[0])
    assert np.array_equal(toks.cpu().numpy(), et) and acc.item() == ea
    s.close()
