"""Generates the golden fixtures in this folder by running the REFERENCE's own sampler kernels
(oracle/_ref/libfns_ref.so: the reference's src/kernels.cu compiled unmodified for sm_100a) on a GPU.

    python -m tests.golden.make_golden OUT_DIR      # on a machine with a B200; writes OUT_DIR/*.json

Inputs are not stored: each case records the seeded generator call that rebuilds them (flintnsteel_b200.workloads)
and the reference's outputs.  ``replay_case`` is the other half: it rebuilds the inputs and checks the CPU oracle
against the recorded outputs (tests/test_oracle.py runs it without a GPU).

Case kinds
  greedy   k::argmax per row (masked or not)                         -> tokens, exact
  peel     ordered top-k by peeling: k::argmax, clear that id's mask bit, repeat -> ids, exact
  sample   k::sample for counters 0 .. n-1 at one (seed, top_k, top_p, T)       -> tokens; the oracle must give
           the same token unless the uniform lies within 1e-6 of a CDF boundary (CUDA's exp and libm's may
           differ in the last bit)
  presence k::presence_apply / presence_apply_col                     -> checksum of the output bits, exact
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.sampler import make_params

CDF_TOL = 1e-6


def build_inputs(spec: dict):
    """(logits float32 (rows, V), masks or None, history or None) for a generator spec."""
    gen = spec["gen"]
    if gen == "lcg":
        x, mask, _ = wl.lcg_logits(spec.get("n", 150_144))
        return x[None, :], (mask[None, :] if spec.get("masked") else None), None
    if gen == "single_row":
        w = wl.single_row(seed=spec["seed"], vocab=spec.get("vocab", wl.V_QWEN))
    elif gen == "grammar_row":
        w = wl.grammar_row(seed=spec["seed"], vocab=spec.get("vocab", wl.V_QWEN))
    elif gen == "session_batch":
        w = wl.session_batch(seed=spec["seed"], rows=spec["rows"], vocab=spec.get("vocab", wl.V_QWEN),
                             history=spec.get("history", 2048))
    elif gen == "spec_windows":
        w = wl.spec_windows(seed=spec["seed"], windows=spec["windows"], n_draft=spec.get("n_draft", 3),
                            vocab=spec.get("vocab", wl.V_QWEN))
    elif gen == "ties":
        g = wl.rng(spec["seed"])
        n = spec["n"]
        x = (np.round(g.standard_normal((spec["rows"], n)) * 2) / 2).astype(np.float32)  # heavy ties
        x[:, ::97] = np.float32(-0.0)
        x[:, 5::89] = np.float32(0.0)
        masks = np.stack([wl.random_mask(g, n, 0.5) for _ in range(spec["rows"])]) if spec.get("masked") else None
        return x, masks, None
    else:
        raise ValueError(gen)
    masks = w.masks if spec.get("masked", True) else None
    return w.logits, masks, w.history


def penalised(oracle, x, hist, spec):
    pen = spec.get("penalty")
    if not pen or hist is None:
        return x
    out = x.copy()
    for r in range(x.shape[0]):
        out[r] = oracle.penalize(x[r], hist[r], None, pen["repetition"], pen["presence"], pen["frequency"])
    return out


def checksum(a: np.ndarray) -> int:
    b = np.ascontiguousarray(a).view(np.uint32).astype(np.uint64)
    return int((b * (np.arange(b.size, dtype=np.uint64) % np.uint64(65521) + np.uint64(1))).sum() % np.uint64(2**61 - 1))


# ---- replay on the CPU oracle --------------------------------------------------------------------------------
def replay_case(oracle, case: dict):
    spec = case["spec"]
    x, masks, hist = build_inputs(spec)
    x = penalised(oracle, x, hist, spec)
    kind = case["kind"]
    if kind == "greedy":
        for r, tok in enumerate(case["tokens"]):
            got = oracle.sample_row(x[r], make_params(1), mask=None if masks is None else masks[r])
            assert got == tok, (spec, r, got, tok)
    elif kind == "peel":
        for r, ids in zip(case["rows"], case["ids"]):
            cv, ci, nk = oracle.topk(x[r], None if masks is None else masks[r], len(ids))
            assert list(ci) == ids, (spec, r)
    elif kind == "sample":
        r = case["row"]
        p = make_params(1, temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"], seed=case["seed"])
        k = oracle.clamp_k(case["top_k"], 64)
        cv, ci, nk = oracle.topk(x[r], None if masks is None else masks[r], k)
        exact = 0
        for c, tok in enumerate(case["tokens"]):
            p["counter"] = case["counter0"] + c
            got, q, keep, u, cdf = oracle.draw(cv, ci, nk, p, detail=True)
            if got == tok:
                exact += 1
                continue
            # allowed only when u sits on a CDF boundary between the two answers
            assert np.min(np.abs(cdf[:keep] - u)) < CDF_TOL, (spec, c, got, tok, u)
        assert exact >= len(case["tokens"]) - 2
    elif kind == "presence":
        seen = np.zeros(x.shape[1], np.float32)
        seen[np.asarray(case["seen_ids"], dtype=np.int64)] = 1.0
        if case["col"] is None:
            y = oracle.presence_apply(x[0], seen, case["penalty"])
        else:
            y = oracle.presence_apply_col(x[0], seen, np.asarray(case["draft"], np.int32), case["col"], case["penalty"])
        assert checksum(y) == case["checksum"], spec
    else:
        raise ValueError(kind)


# ---- generation on the GPU -----------------------------------------------------------------------------------
def main(out_dir: str):
    import torch

    from oracle.binding import Oracle, RefGpu

    oracle, ref = Oracle(), RefGpu()
    dev = torch.device("cuda:0")
    os.makedirs(out_dir, exist_ok=True)

    def to_dev(a, dtype=None):
        return None if a is None else torch.from_numpy(np.ascontiguousarray(a if dtype is None else a.view(dtype))).to(dev)

    def greedy_case(spec):
        x, masks, hist = build_inputs(spec)
        x = penalised(oracle, x, hist, spec)
        dx, dm = to_dev(x), to_dev(masks, np.int32)
        out = torch.empty(x.shape[0], dtype=torch.int32, device=dev)
        for r in range(x.shape[0]):
            ref.argmax(dx[r], out[r:r + 1], None if dm is None else dm[r])
        return {"kind": "greedy", "spec": spec, "tokens": out.cpu().tolist()}

    def peel_case(spec, rows, k):
        x, masks, hist = build_inputs(spec)
        x = penalised(oracle, x, hist, spec)
        dx = to_dev(x)
        words = (x.shape[1] + 31) // 32
        all_ids = []
        out = torch.empty(1, dtype=torch.int32, device=dev)
        for r in rows:
            m = np.full(words, 0xFFFFFFFF, np.uint32) if masks is None else masks[r].copy()
            ids = []
            for _ in range(k):
                ref.argmax(dx[r], out, to_dev(m, np.int32))
                t = int(out.item())
                if t < 0:
                    break
                ids.append(t)
                m[t >> 5] &= np.uint32(~np.uint32(1 << (t & 31)))
            ids += [0x7FFFFFFF] * (k - len(ids))
            all_ids.append(ids)
        return {"kind": "peel", "spec": spec, "rows": list(rows), "ids": all_ids}

    def sample_case(spec, row, top_k, top_p, temperature, seed, counter0, draws):
        x, masks, hist = build_inputs(spec)
        x = penalised(oracle, x, hist, spec)
        dx, dm = to_dev(x), to_dev(masks, np.int32)
        out = torch.empty(draws, dtype=torch.int32, device=dev)
        ref.sample_counters(dx[row], None if dm is None else dm[row], top_k, top_p, temperature, seed, counter0, draws, out)
        return {"kind": "sample", "spec": spec, "row": row, "top_k": top_k, "top_p": top_p, "temperature": temperature,
                "seed": seed, "counter0": counter0, "tokens": out.cpu().tolist()}

    def presence_case(spec, seen_ids, penalty, col=None, draft=None):
        x, _, _ = build_inputs(spec)
        dx = to_dev(x[0].copy())
        seen = np.zeros(x.shape[1], np.float32)
        seen[seen_ids] = 1.0
        ds = to_dev(seen)
        if col is None:
            ref.presence_apply(dx, ds, penalty)
        else:
            ref.presence_apply_col(dx, ds, to_dev(np.asarray(draft, np.int32)), col, penalty)
        return {"kind": "presence", "spec": spec, "seen_ids": list(map(int, seen_ids)), "penalty": penalty, "col": col,
                "draft": draft, "checksum": checksum(dx.cpu().numpy())}

    pen2 = {"repetition": 1.1, "presence": 0.5, "frequency": 0.3}
    pen1 = {"repetition": 1.1, "presence": 0.0, "frequency": 0.0}
    lcg, lcg_m = {"gen": "lcg"}, {"gen": "lcg", "masked": True}
    docs = {
        "sample_check_inputs": [   # the reference test's own three cases (tests/sample_check.cu:90-92) + argmax
            sample_case(lcg, 0, 20, 0.95, 1.0, 1234, 0, 3000),
            sample_case(lcg, 0, 0, 1.0, 0.7, 1234, 0, 3000),
            sample_case(lcg_m, 0, 20, 1.0, 1.0, 1234, 0, 3000),
            greedy_case(lcg), greedy_case(lcg_m),
            peel_case(lcg, [0], 64), peel_case(lcg_m, [0], 20),
        ],
        "config1_single_row": [
            greedy_case({"gen": "single_row", "seed": 0, "penalty": pen1, "masked": False}),
            peel_case({"gen": "single_row", "seed": 0, "penalty": pen1, "masked": False}, [0], 40),
            sample_case({"gen": "single_row", "seed": 0, "penalty": pen1, "masked": False}, 0, 40, 0.95, 0.7, 0, 0, 4000),
            sample_case({"gen": "single_row", "seed": 1, "penalty": pen1, "masked": False}, 0, 40, 0.95, 0.7, 0, 1 << 33, 500),
        ],
        "config2_grammar_row": [
            greedy_case({"gen": "grammar_row", "seed": 0, "penalty": pen2}),
            peel_case({"gen": "grammar_row", "seed": 0, "penalty": pen2}, [0], 20),
            sample_case({"gen": "grammar_row", "seed": 0, "penalty": pen2}, 0, 20, 0.9, 0.6, 0, 0, 4000),
        ],
        "config3_spec_rows": [
            greedy_case({"gen": "spec_windows", "seed": s, "windows": 8, "masked": False}) for s in range(3)
        ],
        "config4_sessions": [
            greedy_case({"gen": "session_batch", "seed": 0, "rows": 24, "penalty": pen2}),
            peel_case({"gen": "session_batch", "seed": 0, "rows": 24, "penalty": pen2}, [0, 5, 11, 17], 24),
        ] + [
            sample_case({"gen": "session_batch", "seed": 0, "rows": 24, "penalty": pen2}, r, tk, tp, t, 77 + r, 0, 400)
            for r, tk, tp, t in [(0, 0, 0.9, 0.3), (3, 20, 0.8, 1.2), (7, 40, 1.0, 0.75), (12, 100, 0.95, 1.0),
                                 (19, 64, 0.85, 0.5), (23, 1, 1.0, 1.0)]
        ],
        "ties_and_zeros": [
            greedy_case({"gen": "ties", "seed": 1, "rows": 6, "n": 70_001}),
            greedy_case({"gen": "ties", "seed": 2, "rows": 6, "n": 70_001, "masked": True}),
            peel_case({"gen": "ties", "seed": 3, "rows": 2, "n": 9_999, "masked": True}, [0, 1], 64),
            sample_case({"gen": "ties", "seed": 4, "rows": 1, "n": 33_333}, 0, 64, 1.0, 1.0, 5, 0, 1000),
        ],
        "presence": [
            presence_case({"gen": "single_row", "seed": 2, "masked": False}, [0, 17, 151_935, 4242], 0.8),
            presence_case({"gen": "single_row", "seed": 2, "masked": False}, [3, 9], 1.5, col=2, draft=[100, 3, 7]),
            presence_case({"gen": "single_row", "seed": 2, "masked": False}, [3, 9], -0.25, col=0, draft=[100, 3, 7]),
        ],
    }
    for name, cases in docs.items():
        with open(os.path.join(out_dir, name + ".json"), "w") as f:
            json.dump({"made_by": "tests/golden/make_golden.py on a B200 with the reference's kernels (sm_100a build)",
                       "cases": cases}, f, separators=(",", ":"))
        for case in cases:  # the oracle must already agree when the fixture is written
            replay_case(oracle, case)
        print("wrote", name, len(cases), "cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <output directory>   (on a machine with a B200)")
    main(sys.argv[1])
