"""ctypes bindings of the two checkers.  TEST INFRASTRUCTURE: imported by tests/, by ``__graft_entry__.smoke``
and by the CPU-baseline leg of ``bench.py`` only; the package ``flintnsteel_b200`` never imports this.

* ``Oracle``  - ``oracle/libfns_oracle.so``, the CPU restatement in ``fns_oracle.c`` (host numpy arrays).
* ``RefGpu``  - ``oracle/_ref/libfns_ref.so``, the reference's own CUDA sampler recompiled for sm_100a
                (device pointers; needs a GPU).
Both are built by ``oracle/Makefile``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libfns_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libfns_ref.so")

PARAMS_DTYPE = np.dtype(
    [("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("repetition", "<f4"), ("presence", "<f4"),
     ("frequency", "<f4"), ("top_k", "<i4"), ("reserved", "<i4"), ("seed", "<u8"), ("counter", "<u8")],
    align=True,
)
EMPTY_ID = 0x7FFFFFFF


def build(target: str = "all") -> None:
    env = dict(os.environ)
    env.pop("CC", None)
    subprocess.run(["make", "-C", HERE, target], check=True, capture_output=True, env=env)


def _p(a, t=ctypes.c_void_p):
    return None if a is None else a.ctypes.data_as(t)


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build("oracle")
        lib = ctypes.CDLL(ORACLE_SO)
        vp, i32, i64, u64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_float
        lib.fns_oracle_philox_word.argtypes = [u64, u64]
        lib.fns_oracle_philox_word.restype = ctypes.c_uint32
        lib.fns_oracle_philox_uniform.argtypes = [u64, u64]
        lib.fns_oracle_philox_uniform.restype = f32
        lib.fns_oracle_clamp_k.argtypes = [i32, i32]
        lib.fns_oracle_penalize.argtypes = [vp, i32, vp, i32, vp, i32, f32, f32, f32]
        lib.fns_oracle_penalize.restype = None
        lib.fns_oracle_topk.argtypes = [vp, i32, vp, i32, i32, vp, vp]
        lib.fns_oracle_merge.argtypes = [vp, vp, i32, i32, i32, vp, vp]
        lib.fns_oracle_draw.argtypes = [vp, vp, i32, vp, vp, vp, vp, vp]
        lib.fns_oracle_sample_row.argtypes = [vp, i32, vp, vp, i32, vp, i32, vp, i32, vp, vp, vp]
        lib.fns_oracle_sample_rows.argtypes = [vp, i64, i32, i32, vp, i64, vp, i64, vp, vp, i32, vp, i32]
        lib.fns_oracle_widen_bf16.argtypes = [vp, vp, i64]
        lib.fns_oracle_widen_bf16.restype = None
        lib.fns_oracle_accept_len.argtypes = [vp, vp, i32]
        lib.fns_oracle_verify_window.argtypes = [vp, i64, i32, i32, vp, vp, i64, vp, i32, vp, i32, vp]
        lib.fns_oracle_lookup_draft.argtypes = [vp, i32, i32, vp]
        lib.fns_oracle_presence_apply.argtypes = [vp, vp, i32, f32]
        lib.fns_oracle_presence_apply.restype = None
        lib.fns_oracle_presence_apply_col.argtypes = [vp, vp, vp, i32, i32, f32]
        lib.fns_oracle_presence_apply_col.restype = None
        lib.fns_oracle_io_advance.argtypes = [vp, i32]
        lib.fns_oracle_io_advance.restype = None
        self.lib = lib

    # -- scalar pieces
    def philox_word(self, seed: int, counter: int) -> int:
        return int(self.lib.fns_oracle_philox_word(seed, counter))

    def philox_uniform(self, seed: int, counter: int) -> float:
        return float(self.lib.fns_oracle_philox_uniform(seed, counter))

    def clamp_k(self, top_k: int, k_cap: int) -> int:
        return int(self.lib.fns_oracle_clamp_k(top_k, k_cap))

    # -- stages
    def penalize(self, x, hist, extra, repetition, presence, frequency):
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        hist = np.ascontiguousarray(hist if hist is not None else np.zeros(0), dtype=np.int32)
        extra = np.ascontiguousarray(extra if extra is not None else np.zeros(0), dtype=np.int32)
        self.lib.fns_oracle_penalize(_p(y), y.size, _p(hist), hist.size, _p(extra), extra.size,
                                     repetition, presence, frequency)
        return y

    def topk(self, x, mask, k, id_base=0):
        x = np.ascontiguousarray(x, dtype=np.float32)
        v = np.empty(k, np.float32)
        i = np.empty(k, np.int32)
        m = None if mask is None else np.ascontiguousarray(mask, dtype=np.uint32)
        nk = self.lib.fns_oracle_topk(_p(x), x.size, _p(m), k, id_base, _p(v), _p(i))
        return v, i, int(nk)

    def merge(self, values, ids, k):
        values = np.ascontiguousarray(values, dtype=np.float32)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        lists, length = values.shape
        v = np.empty(k, np.float32)
        i = np.empty(k, np.int32)
        nk = self.lib.fns_oracle_merge(_p(values), _p(ids), lists, length, k, _p(v), _p(i))
        return v, i, int(nk)

    def draw(self, cand_v, cand_i, nk, params, detail=False):
        """Token for one parameter struct; with detail also (q, keep, u, cdf)."""
        p = np.ascontiguousarray(params.reshape(-1)[:1], dtype=PARAMS_DTYPE)
        cand_v = np.ascontiguousarray(cand_v, dtype=np.float32)
        cand_i = np.ascontiguousarray(cand_i, dtype=np.int32)
        if not detail:
            return int(self.lib.fns_oracle_draw(_p(cand_v), _p(cand_i), nk, _p(p), None, None, None, None))
        n = max(nk, 1)
        q = np.zeros(n, np.float64)
        cdf = np.zeros(n, np.float64)
        keep = np.zeros(1, np.int32)
        u = np.zeros(1, np.float64)
        tok = int(self.lib.fns_oracle_draw(_p(cand_v), _p(cand_i), nk, _p(p), _p(q), _p(keep), _p(u), _p(cdf)))
        return tok, q, int(keep[0]), float(u[0]), cdf

    # -- whole rows
    def sample_row(self, x, params, k_cap=64, mask=None, hist=None, extra=None, want_cands=False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        p = np.ascontiguousarray(params.reshape(-1)[:1], dtype=PARAMS_DTYPE)
        m = None if mask is None else np.ascontiguousarray(mask, dtype=np.uint32)
        h = None if hist is None else np.ascontiguousarray(hist, dtype=np.int32)
        e = None if extra is None else np.ascontiguousarray(extra, dtype=np.int32)
        cv = np.empty(k_cap, np.float32) if want_cands else None
        ci = np.empty(k_cap, np.int32) if want_cands else None
        nk = np.zeros(1, np.int32)
        tok = int(self.lib.fns_oracle_sample_row(_p(x), x.size, _p(m), _p(h), 0 if h is None else h.size, _p(e),
                                                 0 if e is None else e.size, _p(p), k_cap, _p(cv), _p(ci), _p(nk)))
        if want_cands:
            return tok, cv, ci, int(nk[0])
        return tok

    def sample_rows(self, x, params, k_cap=64, masks=None, hist=None, hist_len=None, threads=0):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, n = x.shape
        p = np.ascontiguousarray(params, dtype=PARAMS_DTYPE)
        m = None if masks is None else np.ascontiguousarray(masks, dtype=np.uint32)
        h = None if hist is None else np.ascontiguousarray(hist, dtype=np.int32)
        hl = None if hist is None else np.ascontiguousarray(hist_len, dtype=np.int32)
        out = np.empty(rows, np.int32)
        used = self.lib.fns_oracle_sample_rows(_p(x), n, n, rows, _p(m), 0 if m is None else m.shape[1], _p(h),
                                               0 if h is None else h.shape[1], _p(hl), _p(p), k_cap, _p(out), threads)
        return out, int(used)

    def widen_bf16(self, bits):
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.shape, np.float32)
        self.lib.fns_oracle_widen_bf16(_p(bits), _p(out), bits.size)
        return out

    def accept_len(self, tokens, draft):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        draft = np.ascontiguousarray(draft, dtype=np.int32)
        return int(self.lib.fns_oracle_accept_len(_p(tokens), _p(draft), draft.size))

    def verify_window(self, x, draft, params, k_cap=64, masks=None, hist=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        draft = np.ascontiguousarray(draft, dtype=np.int32)
        p = np.ascontiguousarray(params.reshape(-1)[:1], dtype=PARAMS_DTYPE)
        m = None if masks is None else np.ascontiguousarray(masks, dtype=np.uint32)
        h = None if hist is None else np.ascontiguousarray(hist, dtype=np.int32)
        tokens = np.empty(draft.size + 1, np.int32)
        a = self.lib.fns_oracle_verify_window(_p(x), x.shape[1], x.shape[1], draft.size, _p(draft), _p(m),
                                              0 if m is None else m.shape[1], _p(h), 0 if h is None else h.size,
                                              _p(p), k_cap, _p(tokens))
        return tokens, int(a)

    def lookup_draft(self, history, want):
        h = np.ascontiguousarray(history, dtype=np.int32)
        out = np.zeros(max(want, 1), np.int32)
        n = self.lib.fns_oracle_lookup_draft(_p(h), h.size, want, _p(out))
        return out[:n].copy()

    def presence_apply(self, x, seen, penalty):
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        seen = np.ascontiguousarray(seen, dtype=np.float32)
        self.lib.fns_oracle_presence_apply(_p(y), _p(seen), y.size, penalty)
        return y

    def presence_apply_col(self, x, seen, draft, c, penalty):
        y = np.ascontiguousarray(x, dtype=np.float32).copy()
        seen = np.ascontiguousarray(seen, dtype=np.float32)
        draft = np.ascontiguousarray(draft, dtype=np.int32)
        self.lib.fns_oracle_presence_apply_col(_p(y), _p(seen), _p(draft), c, y.size, penalty)
        return y


class RefGpu:
    """The reference's own kernels on the current GPU.  Arguments are CUDA torch tensors."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise RuntimeError(f"{REF_SO} missing: run `make -C oracle ref` where the reference tree is mounted")
        lib = ctypes.CDLL(REF_SO)
        vp, i32, i64, u64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_float
        lib.fns_ref_sample.argtypes = [vp, i32, vp, i32, f32, f32, u64, u64, vp, vp]
        lib.fns_ref_argmax.argtypes = [vp, i32, vp, vp, vp]
        lib.fns_ref_presence_apply.argtypes = [vp, vp, i32, f32, vp]
        lib.fns_ref_presence_mark.argtypes = [vp, vp, vp]
        lib.fns_ref_presence_apply_col.argtypes = [vp, vp, vp, i32, i32, f32, vp]
        lib.fns_ref_presence_mark_n.argtypes = [vp, vp, i32, vp]
        lib.fns_ref_io_advance.argtypes = [vp, i32, vp]
        lib.fns_ref_sample_rows.argtypes = [vp, i64, i32, i32, vp, i64, vp, vp, vp, vp, vp, vp, vp]
        lib.fns_ref_sample_counters.argtypes = [vp, i32, vp, i32, f32, f32, u64, u64, i32, vp, vp]
        for name in ("fns_ref_sample", "fns_ref_argmax", "fns_ref_presence_apply", "fns_ref_presence_mark",
                     "fns_ref_presence_apply_col", "fns_ref_presence_mark_n", "fns_ref_io_advance",
                     "fns_ref_sample_rows", "fns_ref_sample_counters"):
            getattr(lib, name).restype = None
        self.lib = lib

    @staticmethod
    def _d(t):
        return None if t is None else ctypes.c_void_p(t.data_ptr())

    @staticmethod
    def _stream():
        import torch

        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def sample(self, x, mask, top_k, top_p, temperature, seed, counter, out):
        self.lib.fns_ref_sample(self._d(x), x.numel(), self._d(mask), top_k, top_p, temperature, seed, counter,
                                self._d(out), self._stream())

    def argmax(self, x, out, mask=None):
        self.lib.fns_ref_argmax(self._d(x), x.numel(), self._d(out), self._stream(), self._d(mask))

    def sample_counters(self, x, mask, top_k, top_p, temperature, seed, counter0, draws, out):
        self.lib.fns_ref_sample_counters(self._d(x), x.numel(), self._d(mask), top_k, top_p, temperature, seed,
                                         counter0, draws, self._d(out), self._stream())

    def sample_rows(self, x, masks, params: np.ndarray, out):
        """params: host PARAMS_DTYPE array; only the fields the reference has are used."""
        rows, n = x.shape
        tk = np.ascontiguousarray(params["top_k"], dtype=np.int32)
        tp = np.ascontiguousarray(params["top_p"], dtype=np.float32)
        tt = np.ascontiguousarray(params["temperature"], dtype=np.float32)
        sd = np.ascontiguousarray(params["seed"], dtype=np.uint64)
        ct = np.ascontiguousarray(params["counter"], dtype=np.uint64)
        self.lib.fns_ref_sample_rows(self._d(x), x.stride(0), n, rows, self._d(masks),
                                     0 if masks is None else masks.stride(0), _p(tk), _p(tp), _p(tt), _p(sd), _p(ct),
                                     self._d(out), self._stream())

    def presence_apply(self, x, seen, penalty):
        self.lib.fns_ref_presence_apply(self._d(x), self._d(seen), x.numel(), penalty, self._stream())

    def presence_apply_col(self, x, seen, draft, c, penalty):
        self.lib.fns_ref_presence_apply_col(self._d(x), self._d(seen), self._d(draft), c, x.numel(), penalty,
                                            self._stream())

    def presence_mark(self, seen, token):
        self.lib.fns_ref_presence_mark(self._d(seen), self._d(token), self._stream())

    def presence_mark_n(self, seen, tokens, n):
        self.lib.fns_ref_presence_mark_n(self._d(seen), self._d(tokens), n, self._stream())

    def io_advance(self, io, pos):
        self.lib.fns_ref_io_advance(self._d(io), pos, self._stream())
