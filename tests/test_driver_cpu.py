"""Host pieces around the sampler, without a GPU: the request line, the adaptive window width, the window-mask
protocol, the accept / commit loop, and the bitmask tensor as xgrammar hands it over.

The checkers are restatements of the reference's own protocol oracle (oracle/spec_counters.py, after
tests/speed_native_smoke.py:41-98) and the installed xgrammar wheel's CPU bitmask helpers; the functions under test
are the library's (through the C ABI).
"""
import ctypes

import numpy as np
import pytest

from flintnsteel_b200 import sampler as S
from oracle import spec_counters as sc


@pytest.fixture(scope="module")
def lib(library_path):
    return S.load_library()


def test_request_fields_and_defaults_map_to_the_parameter_struct(lib):
    """tools/fns_serve/fns_serve.cpp:291-303: temperature, top_p, top_k, seed, presence_penalty; defaults greedy / 1 /
    k_cap / 0 / 0.  What the front end sends (serve/fns_server.py:387-395): T 1.0, top_p 0.95, top_k 20, seed 0."""
    p = S.params_from_json('{"prompt": [1, 2, 3], "max_tokens": 16}')[0]
    assert (p["temperature"], p["top_p"], p["top_k"], p["seed"], p["presence"]) == (0.0, 1.0, 0, 0, 0.0)
    assert (p["min_p"], p["repetition"], p["frequency"], p["counter"]) == (0.0, 1.0, 0.0, 0)
    p = S.params_from_json('{"id": 4, "temperature": 1.0, "top_p": 0.95, "top_k": 20, "seed": 0, "presence_penalty": 0.0}')[0]
    assert (p["temperature"], p["top_p"], p["top_k"], p["seed"]) == (1.0, np.float32(0.95), 20, 0)
    p = S.params_from_json('{"presence_penalty":1.5,"seed" : 1234567890123, "top_k":\t64 , "temperature":7e-1,'
                           ' "min_p": 0.05, "repetition_penalty": 1.1, "frequency_penalty": 0.3}')[0]
    assert p["presence"] == np.float32(1.5) and p["seed"] == 1234567890123 and p["top_k"] == 64
    assert p["temperature"] == np.float32(0.7) and p["min_p"] == np.float32(0.05)
    assert p["repetition"] == np.float32(1.1) and p["frequency"] == np.float32(0.3)
    # a field that is not a number keeps its default; a key inside another key's name is not that key
    p = S.params_from_json('{"temperature": "hot", "my_top_k": 5, "top_p": null}')[0]
    assert (p["temperature"], p["top_k"], p["top_p"]) == (0.0, 0, 1.0)


def test_adaptive_width_follows_the_reference_policy(lib):
    g = np.random.default_rng(3)
    for _ in range(2000):
        spec = int(g.integers(2, 9))
        pol = S.SpecPolicy()
        lib.fns_b200_spec_policy_init(ctypes.byref(pol), spec)
        cost = [0.0] * (S.MAX_WINDOW + 1)
        for w in range(1, spec + 1):
            if g.random() < 0.6:
                cost[w] = float(g.uniform(0.5, 3.0) * (1 + 0.2 * w))
                pol.cost[w] = cost[w]
        pol.accepted, pol.offered = int(g.integers(0, 50)), 0
        pol.offered = pol.accepted + int(g.integers(0, 50))
        pol.skipped_proposals = int(g.integers(0, 20))
        nd_max = int(g.integers(1, spec))
        want, skipped = sc.choose_width(cost, spec, pol.accepted, pol.offered, pol.skipped_proposals, nd_max)
        assert lib.fns_b200_spec_choose_width(ctypes.byref(pol), nd_max) == want
        assert pol.skipped_proposals == skipped
    # the cost record: first observation as it is, then 7/8 old + 1/8 new (fns_serve.cpp:470-476, 511-516)
    pol = S.SpecPolicy()
    lib.fns_b200_spec_policy_init(ctypes.byref(pol), 4)
    lib.fns_b200_spec_observe(ctypes.byref(pol), 3, 2.0, 1, 2)
    lib.fns_b200_spec_observe(ctypes.byref(pol), 3, 4.0, 2, 2)
    assert pol.cost[3] == 2.0 * 0.875 + 4.0 * 0.125 and (pol.accepted, pol.offered) == (3, 4)
    lib.fns_b200_spec_policy_new_request(ctypes.byref(pol))
    assert (pol.accepted, pol.offered) == (0, 0) and pol.cost[3] > 0  # acceptance is request-local, costs persist


class ToyGrammar:
    """A matcher with the four calls fns-serve uses: after the accepted ids `state`, id t is allowed iff
    (t + sum(state)) % 3 != 0; ids >= 90 terminate."""

    def __init__(self, vocab):
        self.vocab, self.words, self.state, self.calls = vocab, (vocab + 31) // 32, [], []
        self.c = S.Grammar(None, S.GRAMMAR_FILL(self.fill), S.GRAMMAR_ACCEPT(self.accept),
                           S.GRAMMAR_TERMINATED(self.terminated), S.GRAMMAR_ROLLBACK(self.rollback))

    def allowed(self, t):
        return (t + sum(self.state)) % 3 != 0

    def mask(self):
        bits = np.zeros(self.words * 32, bool)
        bits[: self.vocab] = [self.allowed(t) for t in range(self.vocab)]
        return np.packbits(bits.reshape(-1, 32), axis=1, bitorder="little").view(np.uint32).reshape(-1)

    def fill(self, user, out):
        self.calls.append("fill")
        np.ctypeslib.as_array(out, shape=(self.words,)).view(np.uint32)[:] = self.mask()

    def accept(self, user, t):
        self.calls.append(("accept", t))
        if t < 0 or t >= self.vocab or not self.allowed(t):
            return 0
        self.state.append(t)
        return 1

    def terminated(self, user):
        return 1 if self.state and self.state[-1] >= 90 else 0

    def rollback(self, user, n):
        self.calls.append(("rollback", n))
        del self.state[len(self.state) - n:]


def test_window_masks_follow_the_matcher_protocol(lib):
    """tools/fns_serve/fns_serve.cpp:340-354: Fill, AcceptToken(d[c]), ..., Rollback; a rejected draft id cuts the
    window; a terminating draft id ends it; the matcher is left at the committed prefix."""
    vocab = 100
    g = ToyGrammar(vocab)
    g.state = [1]
    wmask = np.zeros((4, g.words), np.uint32)

    def run(draft):
        d = np.array(draft, np.int32)
        g.calls.clear()
        wmask[:] = 0
        return lib.fns_b200_spec_window_masks(ctypes.byref(g.c), d.ctypes.data, len(draft), g.words, wmask.ctypes.data)

    def expect(prefix, draft):
        """Usable draft ids and the masks of the columns, straight from the toy rule."""
        state, usable, masks = list(prefix), 0, []
        for t in list(draft) + [None]:
            ref = ToyGrammar(vocab)
            ref.state = list(state)
            masks.append(ref.mask())
            if t is None or not ref.allowed(t):
                break
            state.append(t)
            usable += 1
        return usable, masks

    for draft in ([1, 4, 7], [1, 5, 7], [2, 2, 2], [4, 4, 4]):
        g.state = [1]
        usable, masks = expect([1], draft)
        W = run(draft)
        assert W == usable + 1, draft
        for c in range(W):
            assert np.array_equal(wmask[c], masks[c]), (draft, c)
        assert g.state == [1]  # rolled back to the committed prefix
        assert g.calls.count("fill") == W and (usable == 0 or g.calls[-1] == ("rollback", usable))
    assert {expect([1], d)[0] for d in ([1, 4, 7], [1, 5, 7], [2, 2, 2], [4, 4, 4])} >= {0, 3}  # both ends are exercised
    # a terminating id: nothing to predict after it
    g.state = [0]
    assert run([91, 5]) == 1 and g.state == [0]  # (the break comes before the column counter moves: fns_serve.cpp:349-353)
    # no grammar: every column is usable and nothing is written
    assert lib.fns_b200_spec_window_masks(None, None, 3, g.words, None) == 4


def emulate(lib, prompt, output, width, max_tokens, stop=()):
    """The driver's loop over a known output: drafts from the library's lookup, commits through fns_b200_spec_commit."""
    c = S.SpecCounters()
    ctx = list(prompt) + [output[0]]
    emitted = [output[0]]
    pos, done = 1, (output[0] in stop or max_tokens == 1)
    stop_a = np.array(list(stop) or [0], np.int32)
    while not done and pos < len(output):
        c.iterations += 1
        room = min(width - 1, max_tokens - len(emitted))
        d = S.lookup_draft(np.array(ctx, np.int32), room) if room > 0 else np.zeros(0, np.int32)
        nd = len(d)
        if nd == 0:
            t = output[pos]
            pos += 1
            ctx.append(t)
            emitted.append(t)
            done = t in stop or len(emitted) == max_tokens
            continue
        W = nd + 1
        # column c's choice is the true continuation while the draft matched; later columns are garbage
        out = np.full(W, -7, np.int32)
        for col in range(W):
            if pos + col < len(output):
                out[col] = output[pos + col]
            if col < nd and out[col] != d[col]:
                break
        committed = np.zeros(W, np.int32)
        engaged, acc, off = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        c.windows += 1
        c.drafted += nd
        c.generated = len(emitted)
        fin = lib.fns_b200_spec_commit(out.ctypes.data, W, d.ctypes.data, nd, stop_a.ctypes.data, len(stop), max_tokens, None,
                                       ctypes.byref(c), committed.ctypes.data, ctypes.byref(engaged), ctypes.byref(acc),
                                       ctypes.byref(off))
        assert fin >= 0
        for t in committed[: engaged.value]:
            ctx.append(int(t))
            emitted.append(int(t))
        pos += engaged.value
        done = fin != 0
    return c, emitted


def test_commit_loop_reproduces_the_reference_counters(lib):
    g = np.random.default_rng(11)
    for trial in range(300):
        period = int(g.integers(2, 7))
        base = list(g.integers(0, 50, size=period))
        prompt = (base * 6)[: int(g.integers(5, 25))]
        # an output that mostly continues the pattern, with random departures
        output, i = [], len(prompt)
        for _ in range(int(g.integers(4, 60))):
            output.append(int(base[i % period]) if g.random() < 0.85 else int(g.integers(0, 50)))
            i += 1
        width = int(g.integers(2, 6))
        want, _ = sc.expected_counters(prompt, output, width)
        c, emitted = emulate(lib, prompt, output, width, max_tokens=len(output))
        assert emitted == output
        got = {"decode_iterations": c.iterations, "spec_windows": c.windows, "spec_drafted": c.drafted,
               "spec_accepted": c.accepted, "spec_emitted": c.emitted}
        assert got == want, (trial, prompt, output, width)
    # a stop token inside a window ends the generation there
    c, emitted = emulate(lib, [1, 2, 3, 1, 2, 3, 1, 2], [3, 1, 2, 3, 1, 2], 4, max_tokens=6, stop=(2,))
    assert emitted == [3, 1, 2]


def test_xgrammar_bitmask_tensor_is_what_the_kernel_reads(lib):
    """The layout the producer fills (xgrammar.allocate_token_bitmask / get_bitmask_shape of the installed wheel):
    int32 CPU [rows][ceil(vocab / 32)], token i <-> bit (i & 31) of word (i >> 5), 1 = allowed - pinned with the
    wheel's own CPU apply_token_bitmask_inplace (the reference pins the same at tests/xgrammar_smoke.cpp:87-102)."""
    xgr = pytest.importorskip("xgrammar")
    torch = pytest.importorskip("torch")
    vocab, rows = 151_936, 3
    bm = xgr.allocate_token_bitmask(rows, vocab)
    assert tuple(bm.shape) == tuple(xgr.get_bitmask_shape(rows, vocab)) == (rows, (vocab + 31) // 32)
    assert bm.dtype == torch.int32 and bm.device.type == "cpu"
    dl = S.DLTensor.of(bm)
    n, words, stride = ctypes.c_int(), ctypes.c_void_p(), ctypes.c_int64()
    assert lib.fns_b200_mask_view(ctypes.byref(dl), vocab, ctypes.byref(n), ctypes.byref(words), ctypes.byref(stride)) == 0
    assert (n.value, words.value, stride.value) == (rows, bm.data_ptr(), (vocab + 31) // 32)
    # bit order: allow exactly the ids our layout names, let xgrammar mask a row of zeros, see which ids survive
    ids = [0, 31, 32, 69, 4095, 151_935]
    bm.zero_()
    host = bm.numpy().view(np.uint32)
    for i in ids:
        host[1, i >> 5] |= np.uint32(1 << (i & 31))
    logits = torch.zeros(rows, vocab)
    xgr.apply_token_bitmask_inplace(logits, bm)
    assert (logits[1] == 0).nonzero().flatten().tolist() == ids and bool(torch.isinf(logits[0]).all())
    # one row, a strided view, and the refusals
    one = S.DLTensor.of(bm[2])
    assert lib.fns_b200_mask_view(ctypes.byref(one), vocab, ctypes.byref(n), ctypes.byref(words), ctypes.byref(stride)) == 0
    assert n.value == 1
    wide = torch.zeros(rows, 5000, dtype=torch.int32)[:, : (vocab + 31) // 32]
    dlw = S.DLTensor.of(wide)
    assert lib.fns_b200_mask_view(ctypes.byref(dlw), vocab, ctypes.byref(n), ctypes.byref(words), ctypes.byref(stride)) == 0
    assert stride.value == 5000
    for bad in (S.DLTensor.of(torch.zeros(rows, 10, dtype=torch.int32)), S.DLTensor.of(torch.zeros(rows, 4748)),
                S.DLTensor.of(torch.zeros(rows, 4748, dtype=torch.int64))):
        assert lib.fns_b200_mask_view(ctypes.byref(bad), vocab, ctypes.byref(n), ctypes.byref(words), ctypes.byref(stride)) == 1
