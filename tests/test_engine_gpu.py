"""The engine glue (fns_b200_engine_*) on a GPU against the CPU oracle.

The glue replaces the sampler part of the reference's Engine (src/engine.cu:715-866): pick_async / pick_wait with
host-side masks and parameters, device-side session histories (reset / append = reset_presence / presence_mark),
and verify for a speculative window.  Every way the inputs can reach the device must give the same tokens:
staged pageable buffers, page-locked buffers read in place, logits on the device or on the host.
"""
import numpy as np
import pytest

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.sampler import Engine, make_params

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def expected(oracle, w, k_cap=64):
    tok, _ = oracle.sample_rows(w.logits, w.params, k_cap, w.masks, w.history, w.history_len)
    return tok


def test_pick_gives_the_oracle_tokens_however_the_inputs_arrive(dev, oracle):
    w = wl.session_batch(seed=21, rows=24, vocab=40_000, history=256)
    w.params["temperature"][::3] = 0.0  # a third of the rows greedy: no boundary cases there
    want = expected(oracle, w)
    eng = Engine(0, max_rows=24, vocab=w.vocab, k_cap=64, max_history=256)
    lg_dev = torch.from_numpy(w.logits).to(dev)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    lg_pin, masks_pin = pin(w.logits), pin(w.masks.view(np.int32))
    hist_pin, hl_pin, par_pin = pin(w.history), pin(w.history_len), pin(w.params.view(np.uint8))
    got = {
        "device logits, pageable side buffers": eng.pick(
            lg_dev, w.params, masks_host=w.masks, history_host=w.history, history_len_host=w.history_len),
        "pageable host logits (staged)": eng.pick(
            torch.from_numpy(w.logits), w.params, masks_host=w.masks, history_host=w.history,
            history_len_host=w.history_len, logits_on_host=True),
        "pinned host logits, copied": eng.pick(
            lg_pin, par_pin, masks_host=masks_pin, history_host=hist_pin, history_len_host=hl_pin, logits_on_host=True),
        "pinned host logits read in place": eng.pick(
            lg_pin, par_pin, masks_host=masks_pin, history_host=hist_pin, history_len_host=hl_pin, logits_on_host=True,
            host_stable=True),
        "device logits, pinned side buffers read in place": eng.pick(
            lg_dev, par_pin, masks_host=masks_pin, history_host=hist_pin, history_len_host=hl_pin, host_stable=True),
        "stable promised but buffers pageable": eng.pick(
            torch.from_numpy(w.logits), w.params, masks_host=w.masks, history_host=w.history,
            history_len_host=w.history_len, logits_on_host=True, host_stable=True),
    }
    eng.close()
    first = got["device logits, pageable side buffers"]
    greedy = w.params["temperature"] <= 0
    assert np.array_equal(first[greedy], want[greedy])
    assert (first != want).sum() <= 1  # a draw on a CDF boundary may differ from the CPU's libm
    for name, tokens in got.items():
        assert np.array_equal(tokens, first), name


def test_two_picks_in_flight_come_back_in_order(dev, oracle):
    a = wl.session_batch(seed=31, rows=5, vocab=8192, history=16)
    b = wl.session_batch(seed=32, rows=5, vocab=8192, history=16)
    for w in (a, b):
        w.params["temperature"][:] = 0.0
    eng = Engine(0, max_rows=5, vocab=8192, k_cap=64, max_history=16)
    la, lb = torch.from_numpy(a.logits).to(dev), torch.from_numpy(b.logits).to(dev)
    eng.pick_async(la, a.params, masks_host=a.masks, history_host=a.history, history_len_host=a.history_len)
    eng.pick_async(lb, b.params, masks_host=b.masks, history_host=b.history, history_len_host=b.history_len)
    with pytest.raises(Exception):
        eng.pick_async(la, a.params)  # a third one is refused, nothing is queued
    ta, tb = eng.pick_wait(5), eng.pick_wait(5)
    eng.close()
    assert np.array_equal(ta, expected(oracle, a)) and np.array_equal(tb, expected(oracle, b))


def test_session_histories_on_the_device_follow_the_presence_rule(dev, oracle):
    """Greedy decoding of 3 sessions for 12 steps with a presence penalty: the engine remembers every chosen token
    (reset_presence / presence_mark of the reference, src/engine.cu:715-731), the oracle gets the list."""
    rows, vocab, steps = 3, 5000, 12
    g = wl.rng(77)
    logits = (g.standard_normal((rows, vocab)) * 0.5).astype(np.float32)
    params = make_params(rows, temperature=0.0, top_k=1, top_p=1.0, presence=0.9, seed=1)
    eng = Engine(0, max_rows=rows, vocab=vocab, k_cap=64, max_history=steps)
    eng.reset()
    lg = torch.from_numpy(logits).to(dev)
    hist = np.zeros((rows, steps), np.int32)
    hl = np.zeros(rows, np.int32)
    for t in range(steps):
        got = eng.pick(lg, params)
        eng.append(eng.device_tokens_ptr(), 1, rows)
        want, _ = oracle.sample_rows(logits, params, 64, None, hist, hl)
        assert np.array_equal(got, want), f"step {t}"
        hist[np.arange(rows), hl] = want
        hl += 1
    assert len(set(hist[0].tolist())) == steps  # the penalty is large enough that no token repeats
    eng.reset()
    again = eng.pick(lg, params)
    eng.close()
    assert np.array_equal(again, hist[:, 0])


def test_verify_window_matches_the_oracle(dev, oracle):
    sw = wl.spec_windows(seed=4, windows=16, vocab=32_000)
    n_draft = sw.draft.shape[1]
    eng = Engine(0, max_rows=16 * (n_draft + 1), vocab=sw.vocab, k_cap=64, max_history=0)
    tokens, accept = eng.verify(torch.from_numpy(sw.logits).to(dev), sw.draft, sw.params)
    eng.close()
    for i in range(16):
        et, ea = oracle.verify_window(sw.logits[i * (n_draft + 1):(i + 1) * (n_draft + 1)], sw.draft[i], sw.params[i:i + 1])
        assert accept[i] == ea and np.array_equal(tokens[i], et), f"window {i}"


def test_verify_with_masks_and_device_side_history(dev, oracle):
    """Engine::verify with per-column masks (src/engine.cu:734-744) after the sessions' histories were filled by
    engine_append: column c is penalised with the session history plus draft[0 .. c) (src/kernels.cu:738-741)."""
    windows, n_draft, vocab, steps = 5, 3, 20_000, 9
    W = n_draft + 1
    sw = wl.spec_windows(seed=14, windows=windows, n_draft=n_draft, vocab=vocab, temperature=0.8)
    sw.params["presence"] = 0.9
    sw.params["top_k"] = 24
    g = wl.rng(15)
    masks = np.stack([wl.random_mask(g, vocab, 0.4) for _ in range(windows * W)])
    eng = Engine(0, max_rows=windows * W, vocab=vocab, k_cap=64, max_history=steps + 4)
    eng.reset()
    # nine committed tokens per session (presence_commit): device-side histories, one column at a time
    committed = g.integers(0, vocab, size=(windows, steps), dtype=np.int32)
    committed[2, 3] = -1  # "no token" is skipped (src/kernels.cu:730)
    for t in range(steps):
        col = torch.from_numpy(np.ascontiguousarray(committed[:, t])).to(dev)
        eng.append(col.data_ptr(), 1, windows)
    torch.cuda.synchronize()
    tokens, accept = eng.verify(torch.from_numpy(sw.logits).to(dev), sw.draft, sw.params, masks_host=masks)
    eng.close()
    for i in range(windows):
        hist = committed[i][committed[i] >= 0]
        et, ea = oracle.verify_window(sw.logits[i * W:(i + 1) * W], sw.draft[i], sw.params[i:i + 1],
                                      masks=masks[i * W:(i + 1) * W], hist=hist)
        assert accept[i] == ea and np.array_equal(tokens[i], et), f"window {i}"


def test_compat_shim_grows_its_workspace(dev, library_path):
    """fns::k::argmax on a vocabulary larger than the shim's default workspace (262,144): the per-device handle is
    replaced by a larger one and the next, smaller call still works."""
    import ctypes

    lib = ctypes.CDLL(library_path)
    argmax = lib._ZN3fns1k6argmaxEPKfiPiP11CUstream_stPKj
    argmax.argtypes, argmax.restype = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p], None
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = torch.zeros(3, dtype=torch.int32, device=dev)
    small = torch.zeros(1000, device=dev)
    small[123] = 1.0
    big = torch.zeros(300_001, device=dev)
    big[299_999] = 2.0
    argmax(small.data_ptr(), 1000, out[0:1].data_ptr(), st, None)
    argmax(big.data_ptr(), 300_001, out[1:2].data_ptr(), st, None)
    argmax(small.data_ptr(), 1000, out[2:3].data_ptr(), st, None)
    torch.cuda.synchronize()
    assert out.tolist() == [123, 299_999, 123]


def test_calls_can_be_captured_in_a_cuda_graph(dev, oracle):
    """The sampler is stream-ordered with no host synchronisation and no set-up left in the call path after
    fns_b200_create, so a call can be captured and replayed: one row (sliced plan, tickets in the workspace), a
    whole-row masked batch (k_select) and an unmasked batch (k_ring, bulk copies), each against its eager run."""
    from flintnsteel_b200.sampler import Sampler, params_to_device

    cases = [wl.grammar_row(seed=3), wl.session_batch(seed=5, rows=9, vocab=40_000, history=128),
             wl.session_batch(seed=6, rows=9, vocab=40_000, history=128)]
    cases[2].masks = None
    for w in cases:
        s = Sampler(0, max_rows=w.rows, max_vocab=w.vocab, k_cap=64, max_history=4096)
        lg = torch.from_numpy(w.logits).to(dev)
        masks = None if w.masks is None else torch.from_numpy(w.masks.view(np.int32)).to(dev)
        hist, hl = torch.from_numpy(w.history).to(dev), torch.from_numpy(w.history_len).to(dev)
        pd = params_to_device(w.params, dev)
        eager = torch.empty(w.rows, dtype=torch.int32, device=dev)
        s.sample_rows(lg, pd, eager, masks=masks, history=hist, history_len=hl)
        torch.cuda.synchronize()
        out = torch.full((w.rows,), -5, dtype=torch.int32, device=dev)
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(3):  # back-to-back launches inside one graph (programmatic dependent launch edges)
                    s.sample_rows(lg, pd, out, masks=masks, history=hist, history_len=hl)
        for _ in range(2):
            out.fill_(-5)
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, eager)
        s.device_status()
        s.close()
