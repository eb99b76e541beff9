"""The callers either side of the sampler on a GPU: the bitmask tensor with the device-side cache of grammar states,
the batched prompt-lookup draft, and the decode loop of fns-serve (sequential against speculative, token for token,
as the reference checks at tests/speed_native_smoke.py:305-319: greedy seed 0, sampled seeds 0 and 7)."""
import ctypes

import numpy as np
import pytest

from flintnsteel_b200 import sampler as S
from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.sampler import Engine, make_params
from oracle import spec_counters as sc

from .test_driver_cpu import ToyGrammar

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def test_lookup_draft_rows_match_the_host_function(dev):
    g = np.random.default_rng(5)
    rows, stride, want = 200, 96, 6
    hist = np.zeros((rows, stride), np.int32)
    lens = g.integers(0, stride + 1, size=rows).astype(np.int32)
    for r in range(rows):
        hist[r, : lens[r]] = g.integers(0, int(g.integers(2, 6)), size=lens[r])
    lens[0], lens[1] = 0, 2
    out = torch.full((rows, want), -1, dtype=torch.int32, device=dev)
    n = torch.zeros(rows, dtype=torch.int32, device=dev)
    rc = S.load_library().fns_b200_lookup_draft_rows(
        torch.from_numpy(hist).to(dev).data_ptr(), stride, torch.from_numpy(lens).to(dev).data_ptr(), rows, want,
        out.data_ptr(), want, n.data_ptr(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    out, n = out.cpu().numpy(), n.cpu().numpy()
    for r in range(rows):
        exp = S.lookup_draft(hist[r, : lens[r]], want)
        assert n[r] == len(exp) and list(out[r, : n[r]]) == list(exp), r


def test_bitmask_tensor_and_state_cache(dev, oracle):
    """The producer's int32 tensor goes in as it is; with grammar-state ids a repeated state uploads nothing and the
    tokens stay the same."""
    w = wl.session_batch(seed=61, rows=12, vocab=50_000, history=64)
    w.params["temperature"][::2] = 0.0
    w.params["repetition"], w.params["presence"], w.params["frequency"] = 1.0, 0.0, 0.0  # (no session history here)
    want, _ = oracle.sample_rows(w.logits, w.params, 64, w.masks, None, None)
    eng = Engine(0, max_rows=12, vocab=w.vocab, k_cap=64, max_history=0)
    lg = torch.from_numpy(w.logits).to(dev)
    bm = torch.from_numpy(w.masks.view(np.int32).copy())  # what xgrammar.allocate_token_bitmask returns: CPU int32
    eng.pick_async_dl(lg, w.params, masks=bm)
    plain = eng.pick_wait(12)
    greedy = w.params["temperature"] <= 0
    assert np.array_equal(plain[greedy], want[greedy]) and (plain != want).sum() <= 1
    # a strided view of a wider tensor gives the same tokens
    wide = torch.zeros(12, bm.shape[1] + 40, dtype=torch.int32)
    wide[:, : bm.shape[1]] = bm
    eng.pick_async_dl(lg, w.params, masks=wide[:, : bm.shape[1]])
    assert np.array_equal(eng.pick_wait(12), plain)
    # the cache: 12 rows in 4 grammar states (rows of one state share its mask) + unmasked rows
    states = np.array([10, 11, 12, 13] * 3, np.uint64)
    shared = bm[:4].repeat(3, 1).contiguous()
    shared_np = shared.numpy().view(np.uint32)
    want_shared, _ = oracle.sample_rows(w.logits, w.params, 64, shared_np, None, None)
    eng.mask_cache(6)
    eng.pick_async_dl(lg, w.params, masks=shared, mask_states=states)
    first = eng.pick_wait(12)
    assert np.array_equal(first[greedy], want_shared[greedy]) and (first != want_shared).sum() <= 1
    hits, misses, nbytes = eng.mask_stats()
    assert (hits, misses, nbytes) == (8, 4, 4 * eng.words() * 4)
    shared.zero_()  # the producer's buffer is reused: a cached state must not be read from it again
    eng.pick_async_dl(lg, w.params, masks=shared, mask_states=states)
    assert np.array_equal(eng.pick_wait(12), first)
    assert eng.mask_stats() == (20, 4, nbytes)
    # new states push out the ones not asked for longest; an unmasked row needs no slot
    states2 = np.array([20, 21, 22, 10, 11, S.EMPTY_ID] * 2, np.uint64)
    states2[5] = states2[11] = 0xFFFFFFFFFFFFFFFF
    masks2 = bm[[4, 5, 6, 0, 1, 7] * 2].contiguous()
    m2 = masks2.numpy().view(np.uint32).copy()
    m2[5] = m2[11] = 0xFFFFFFFF
    want2, _ = oracle.sample_rows(w.logits, w.params, 64, m2, None, None)
    eng.pick_async_dl(lg, w.params, masks=masks2, mask_states=states2)
    got2 = eng.pick_wait(12)
    assert np.array_equal(got2[greedy], want2[greedy]) and (got2 != want2).sum() <= 1
    assert eng.mask_stats()[1] == 7  # three new states
    with pytest.raises(Exception):  # more distinct states in one call than slots
        eng.pick_async_dl(lg, w.params, masks=bm, mask_states=np.arange(100, 112, dtype=np.uint64))
    eng.close()


def test_one_session_with_cached_grammar_states(dev, oracle):
    """The decode loop's own shape: one row per call, the mask named by its grammar state, the history kept on the
    device.  A state that the cache holds uploads nothing; the tokens are the oracle's with the history so far."""
    w = wl.session_batch(seed=62, rows=4, vocab=50_000, history=8)
    eng = Engine(0, max_rows=1, vocab=w.vocab, k_cap=64, max_history=64)
    eng.mask_cache(3)
    lg = torch.from_numpy(w.logits).to(dev)
    p = w.params[:1].copy()
    p["temperature"], p["repetition"], p["presence"], p["frequency"] = 0.7, 1.2, 0.3, 0.2
    hist: list[int] = []
    states = [5, 6, 5, 5, 0xFFFFFFFFFFFFFFFF, 6, 7, 8, 5, 6]   # (three slots: 8 pushes 5 out, the last 5 pushes 6 out)
    for step, st in enumerate(states):
        r = step % 4
        masked = st != 0xFFFFFFFFFFFFFFFF
        m = w.masks[(st - 5) % 4][None, :] if masked else None
        p["counter"] = step
        eng.pick_async_dl(lg[r:r + 1], p, masks=None if m is None else torch.from_numpy(m.view(np.int32).copy()),
                          mask_states=np.array([st], np.uint64))
        eng.append(eng.device_tokens_ptr(), 1, 1)
        tok = int(eng.pick_wait(1)[0])
        h = np.array(hist + [0] * (64 - len(hist)), np.int32)[None, :]
        want, _ = oracle.sample_rows(w.logits[r:r + 1], p, 64, m, h, np.array([len(hist)], np.int32))
        assert tok == want[0], (step, tok, want)
        if tok >= 0:
            hist.append(tok)
    hits, misses, _ = eng.mask_stats()
    assert misses == 6 and hits == 3   # 5, 6, 7, 8 and then 5 and 6 again are uploaded; three calls find theirs
    eng.close()


class ToyModel:
    """Logits that depend on the last token only (a table of rows on the device): greedy decoding soon cycles, so the
    prompt-lookup draft finds continuations; sampling leaves the cycle now and then."""

    def __init__(self, dev, vocab=4096, rows=37, seed=1):
        g = wl.rng(seed)
        t = g.standard_normal((rows, vocab), dtype=np.float32) * np.float32(2.0)
        for r in range(rows):
            t[r, (r * 7 + 3) % rows] += np.float32(9.0)  # a likely successor inside the small alphabet
        self.table = torch.from_numpy(t).to(dev)
        self.rows, self.vocab, self.calls = rows, vocab, []
        self.out = torch.empty((S.MAX_WINDOW, vocab), dtype=torch.float32, device=dev)
        self.c = S.Model(None, S.MODEL_FORWARD(self.forward))

    def forward(self, user, ids, W, p0, logits, row_stride):
        idx = torch.tensor([ids[c] % self.rows for c in range(W)], device=self.table.device)
        torch.index_select(self.table, 0, idx, out=self.out[:W])
        self.calls.append((W, p0))
        logits[0] = self.out.data_ptr()
        row_stride[0] = self.vocab
        return 0


def decode(dev, model, prompt, max_tokens, params, spec, grammar=None, stop=(), adapt=False):
    eng = Engine(0, max_rows=max(spec, 1), vocab=model.vocab, k_cap=64, max_history=max_tokens + 8)
    out = np.zeros(max_tokens, np.int32)
    c = S.SpecCounters()
    pol = S.SpecPolicy()
    S.load_library().fns_b200_spec_policy_init(ctypes.byref(pol), spec)
    pr = np.array(prompt, np.int32)
    st = np.array(list(stop) or [0], np.int32)
    rc = S.load_library().fns_b200_spec_decode(
        eng.handle, ctypes.byref(model.c), None if grammar is None else ctypes.byref(grammar.c), pr.ctypes.data, len(prompt),
        max_tokens, st.ctypes.data, len(stop), params.ctypes.data, 0, spec, ctypes.byref(pol) if adapt else None,
        out.ctypes.data, ctypes.byref(c), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, eng.lib.fns_b200_engine_last_error(eng.handle)
    eng.close()
    return out[: c.generated].tolist(), c


@pytest.mark.parametrize("mode,seed", [("greedy", 0), ("sample", 0), ("sample", 7)])
def test_speculative_decoding_emits_the_sequential_tokens(dev, mode, seed):
    model = ToyModel(dev)
    prompt = [3, 24, 23, 16, 4, 31, 35, 26, 3, 24]
    p = make_params(1, temperature=0.0 if mode == "greedy" else 0.9, top_k=20, top_p=0.95, seed=seed, presence=0.3)
    seq, c0 = decode(dev, model, prompt, 48, p, spec=0)
    assert len(seq) == 48 and c0.windows == 0 and c0.iterations == 47
    for width in (3, 4):
        spec, c = decode(dev, model, prompt, 48, p, spec=width)
        assert spec == seq, (mode, seed, width)
        want, _ = sc.expected_counters(prompt, spec, width)
        got = {"decode_iterations": c.iterations, "spec_windows": c.windows, "spec_drafted": c.drafted,
               "spec_accepted": c.accepted, "spec_emitted": c.emitted}
        assert got == want and c.windows > 0 and (mode != "greedy" or c.accepted > 0)
    adaptive, ca = decode(dev, model, prompt, 48, p, spec=4, adapt=True)
    assert adaptive == seq  # the width policy changes the cost, never the tokens
    stopped, cs = decode(dev, model, prompt, 48, p, spec=3, stop=(seq[20],))
    cut = seq.index(seq[20]) + 1
    assert stopped == seq[:cut]


def test_speculative_decoding_under_a_grammar(dev):
    """With a matcher, every window column gets the mask of its own prefix (Fill / AcceptToken / Rollback) and the
    speculative path still emits exactly the sequential tokens; every emitted id is one the matcher allowed."""
    model = ToyModel(dev, vocab=96, rows=31, seed=4)
    prompt = [5, 9, 5, 9, 5]
    p = make_params(1, temperature=0.8, top_k=12, top_p=0.9, seed=3)
    runs = []
    for width in (0, 3):
        g = ToyGrammar(96)
        g.terminated = lambda user: 0
        g.c = S.Grammar(None, S.GRAMMAR_FILL(g.fill), S.GRAMMAR_ACCEPT(g.accept), S.GRAMMAR_TERMINATED(g.terminated),
                        S.GRAMMAR_ROLLBACK(g.rollback))
        tokens, c = decode(dev, model, prompt, 30, p, spec=width, grammar=g)
        assert g.state == tokens  # the matcher ends on the committed tokens, nothing more
        check, ok = ToyGrammar(96), True
        for t in tokens:
            ok = ok and check.allowed(t)
            check.state.append(t)
        assert ok
        runs.append(tokens)
    assert runs[0] == runs[1] and len(runs[0]) == 30


def test_json_lines_service_answers_like_the_oracle(dev, oracle, tmp_path):
    """The request surface (tools/fns_serve/fns_serve.cpp:291-303) end to end: defaults = greedy, the five fields reach
    the sampler, `draw` is the Philox counter, a bad line gives an error line and the service goes on."""
    import io
    import json

    from flintnsteel_b200.serve import serve

    w = wl.session_batch(seed=71, rows=2, vocab=3000, history=8)
    np.save(tmp_path / "rows.npy", w.logits)
    allowed = [int(i) for i in np.nonzero(np.unpackbits(w.masks[0].view(np.uint8), bitorder="little")[:3000])[0]]
    lines = [
        json.dumps({"id": 1, "logits": w.logits[0].tolist()}),
        json.dumps({"id": 2, "logits_npy": str(tmp_path / "rows.npy"), "temperature": 0.9, "top_p": 0.9, "top_k": 30,
                    "seed": 11, "presence_penalty": 0.7, "history": [5, 9, 5], "allowed": allowed, "draw": 4}),
        "this is not json",
        json.dumps({"id": 3, "logits": [0.0, 1.0], "allowed": [7]}),
        json.dumps({"id": 4, "logits": [0.0, 3.0, 1.0]}),
    ]
    out = io.StringIO()
    serve(io.StringIO("\n".join(lines) + "\n"), out)
    replies = [json.loads(x) for x in out.getvalue().splitlines()]
    assert len(replies) == 5
    assert replies[0] == {"id": 1, "tokens": [int(w.logits[0].argmax())]}
    p = make_params(2, temperature=0.9, top_p=0.9, top_k=30, seed=11, presence=0.7)
    p["counter"] = [4, 5]
    masks = np.repeat(w.masks[:1], 2, axis=0)
    hist = np.array([[5, 9, 5], [5, 9, 5]], np.int32)
    want, _ = oracle.sample_rows(w.logits, p, 64, masks, hist, np.array([3, 3], np.int32))
    assert replies[1] == {"id": 2, "tokens": want.tolist()}
    assert "error" in replies[2] and "error" in replies[3] and "vocabulary" in replies[3]["error"]
    assert replies[4] == {"id": 4, "tokens": [1]}
