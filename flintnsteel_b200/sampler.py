"""ctypes binding of the C ABI in ``include/fns_b200.h`` for tests, the benchmark and the multi-GPU dispatcher.

The CUDA library is the only implementation: if it is missing the import of this module's ``load_library``
fails loudly; there is no CPU path.  torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

OK, ERR_ARG, ERR_CUDA, ERR_CAPACITY, ERR_DEVICE = 0, 1, 2, 3, 4
F32, BF16 = 0, 1
EMPTY_ID = 0x7FFFFFFF
MAX_K = 1024

#: ``fns_b200_params`` (48 bytes); the reference's ``fns::SampleParams`` (include/fns/engine.h:75-84) plus the
#: Philox counter and the three extension terms.
PARAMS_DTYPE = np.dtype(
    [
        ("temperature", "<f4"),
        ("top_p", "<f4"),
        ("min_p", "<f4"),
        ("repetition", "<f4"),
        ("presence", "<f4"),
        ("frequency", "<f4"),
        ("top_k", "<i4"),
        ("reserved", "<i4"),
        ("seed", "<u8"),
        ("counter", "<u8"),
    ],
    align=True,
)
assert PARAMS_DTYPE.itemsize == 48

#: ``fns_b200_cand``: (value, id), the pair the reference keeps in g_cand_v / g_cand_i (src/kernels.cu:601-602).
CAND_DTYPE = np.dtype([("value", "<f4"), ("id", "<i4")])

#: every symbol that ``include/fns_b200.h`` declares
SYMBOLS = [
    "fns_b200_create",
    "fns_b200_destroy",
    "fns_b200_last_error",
    "fns_b200_device_status",
    "fns_b200_k_cap",
    "fns_b200_sample_rows",
    "fns_b200_sample_one",
    "fns_b200_sample_rows_noalloc",
    "fns_b200_select_rows",
    "fns_b200_finalize_rows",
    "fns_b200_verify_accept",
    "fns_b200_presence_apply",
    "fns_b200_presence_mark",
    "fns_b200_presence_apply_col",
    "fns_b200_presence_mark_n",
    "fns_b200_io_advance",
    "fns_b200_launch_count",
    "fns_b200_profile_begin",
    "fns_b200_profile_end",
    "fns_b200_engine_create",
    "fns_b200_engine_destroy",
    "fns_b200_engine_last_error",
    "fns_b200_engine_sampler",
    "fns_b200_engine_pick_async",
    "fns_b200_engine_pick_wait",
    "fns_b200_engine_device_tokens",
    "fns_b200_engine_reset",
    "fns_b200_engine_append",
    "fns_b200_engine_verify",
    "fns_b200_lookup_draft",
    "fns_b200_sample_rows_shared_masks",
    "fns_b200_mask_view",
    "fns_b200_engine_mask_cache",
    "fns_b200_engine_mask_stats",
    "fns_b200_engine_pick_async_dl",
    "fns_b200_engine_words",
    "fns_b200_lookup_draft_rows",
    "fns_b200_spec_window_masks",
    "fns_b200_spec_commit",
    "fns_b200_spec_policy_init",
    "fns_b200_spec_policy_new_request",
    "fns_b200_spec_choose_width",
    "fns_b200_spec_observe",
    "fns_b200_spec_decode",
    "fns_b200_params_from_json",
    "fns_b200_mg_unique_id",
    "fns_b200_mg_create",
    "fns_b200_mg_destroy",
    "fns_b200_mg_last_error",
    "fns_b200_mg_range",
    "fns_b200_mg_sample_rows",
    "fns_b200_mg_gather_tokens",
    "fns_b200_mg_profile_begin",
    "fns_b200_mg_profile_end",
]

#: exported for the tests, the benchmark and the engine glue only (csrc/fns_internal.h)
INTERNAL_SYMBOLS = ["fns_b200_plan", "fns_b200_set_slices", "fns_b200_set_threads", "fns_b200_set_cluster_rows", "fns_b200_hint_host_logits",
                    "fns_b200_mg_create_with_ops"]

_lib = None


class SamplerError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"fns_b200 status {code}: {text}")
        self.code = code


def make_params(rows: int, **fields) -> np.ndarray:
    """Host array of ``rows`` parameter structs with the reference's defaults (greedy, top_p 1, k_cap)."""
    p = np.zeros(rows, dtype=PARAMS_DTYPE)
    p["top_p"] = 1.0
    p["repetition"] = 1.0
    for name, value in fields.items():
        p[name] = value
    return p


def load_library() -> ctypes.CDLL:
    """Loads ``lib/libfns_b200.so``.  Raises if it has not been built: nothing stands in for it."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m flintnsteel_b200.build` (there is no CPU fallback)"
        )
    lib = ctypes.CDLL(path)
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    f64p = ctypes.POINTER(ctypes.c_double)
    lib.fns_b200_create.argtypes = [i32, i32, i32, i32, i32, ctypes.POINTER(vp)]
    lib.fns_b200_destroy.argtypes = [vp]
    lib.fns_b200_last_error.argtypes = [vp]
    lib.fns_b200_last_error.restype = ctypes.c_char_p
    lib.fns_b200_device_status.argtypes = [vp, vp]
    lib.fns_b200_k_cap.argtypes = [vp]
    lib.fns_b200_sample_rows.argtypes = [vp, vp, i32, i64, i32, i32, vp, i64, vp, i64, vp, vp, vp, vp]
    lib.fns_b200_sample_one.argtypes = [vp, vp, i32, i32, vp, vp, i32, vp, vp, vp]
    lib.fns_b200_sample_rows_noalloc.argtypes = [i32, vp, i32, i64, i32, i32, vp, i64, vp, i64, vp, vp, vp, vp,
                                                 ctypes.c_char_p, i32]
    lib.fns_b200_select_rows.argtypes = [vp, vp, i32, i64, i32, i32, i32, vp, i64, vp, i64, vp, vp, vp, vp]
    lib.fns_b200_finalize_rows.argtypes = [vp, vp, i32, i32, i64, i64, i32, vp, vp, vp, vp]
    lib.fns_b200_verify_accept.argtypes = [vp, vp, i32, i64, i32, i32, i32, vp, vp, i64, vp, i64, vp, vp, vp, vp, vp]
    lib.fns_b200_presence_apply.argtypes = [vp, vp, i32, f32, vp]
    lib.fns_b200_presence_mark.argtypes = [vp, vp, vp]
    lib.fns_b200_presence_apply_col.argtypes = [vp, vp, vp, i32, i32, f32, vp]
    lib.fns_b200_presence_mark_n.argtypes = [vp, vp, i32, vp]
    lib.fns_b200_io_advance.argtypes = [vp, i32, vp]
    lib.fns_b200_plan.argtypes = [vp, i32, i32, i32, i32, ctypes.POINTER(i32), ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.fns_b200_set_slices.argtypes = [vp, i32]
    lib.fns_b200_set_threads.argtypes = [vp, i32]
    lib.fns_b200_set_cluster_rows.argtypes = [vp, i32]
    lib.fns_b200_launch_count.argtypes = [vp]
    lib.fns_b200_profile_begin.argtypes = [vp, i32]
    lib.fns_b200_profile_end.argtypes = [vp, vp, f64p, f64p, ctypes.POINTER(i32)]
    lib.fns_b200_engine_create.argtypes = [i32, i32, i32, i32, i32, ctypes.POINTER(vp)]
    lib.fns_b200_engine_destroy.argtypes = [vp]
    lib.fns_b200_engine_last_error.argtypes = [vp]
    lib.fns_b200_engine_sampler.argtypes = [vp]
    lib.fns_b200_engine_pick_async.argtypes = [vp, vp, i32, i32, i64, i32, vp, vp, i64, vp, vp, vp]
    lib.fns_b200_engine_pick_wait.argtypes = [vp, vp]
    lib.fns_b200_engine_device_tokens.argtypes = [vp]
    lib.fns_b200_engine_reset.argtypes = [vp, vp]
    lib.fns_b200_engine_append.argtypes = [vp, vp, i64, i32, vp, vp]
    lib.fns_b200_engine_verify.argtypes = [vp, vp, i32, i64, i32, i32, vp, vp, vp, vp, vp, vp]
    lib.fns_b200_lookup_draft.argtypes = [vp, i32, i32, vp]
    lib.fns_b200_hint_host_logits.argtypes = [vp, i32]
    i32p, i64p = ctypes.POINTER(i32), ctypes.POINTER(i64)
    lib.fns_b200_sample_rows_shared_masks.argtypes = [vp, vp, i32, i64, i32, i32, vp, i64, vp, vp, i64, vp, vp, vp, vp]
    lib.fns_b200_mask_view.argtypes = [vp, i32, i32p, ctypes.POINTER(vp), i64p]
    lib.fns_b200_engine_mask_cache.argtypes = [vp, i32]
    lib.fns_b200_engine_mask_stats.argtypes = [vp, i64p, i64p, i64p]
    lib.fns_b200_engine_pick_async_dl.argtypes = [vp, vp, i32, i64, i32, vp, vp, vp, vp]
    lib.fns_b200_engine_words.argtypes = [vp]
    lib.fns_b200_lookup_draft_rows.argtypes = [vp, i64, vp, i32, i32, vp, i64, vp, vp]
    lib.fns_b200_spec_window_masks.argtypes = [vp, vp, i32, i32, vp]
    lib.fns_b200_spec_commit.argtypes = [vp, i32, vp, i32, vp, i32, i32, vp, vp, vp, i32p, i32p, i32p]
    lib.fns_b200_spec_policy_init.argtypes = [vp, i32]
    lib.fns_b200_spec_policy_new_request.argtypes = [vp]
    lib.fns_b200_spec_choose_width.argtypes = [vp, i32]
    lib.fns_b200_spec_observe.argtypes = [vp, i32, ctypes.c_double, i32, i32]
    lib.fns_b200_spec_decode.argtypes = [vp, vp, vp, vp, i32, i32, vp, i32, vp, i32, i32, vp, vp, vp, vp]
    lib.fns_b200_params_from_json.argtypes = [ctypes.c_char_p, vp]
    lib.fns_b200_mg_unique_id.argtypes = [vp]
    lib.fns_b200_mg_create.argtypes = [i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, ctypes.POINTER(vp)]
    lib.fns_b200_mg_create_with_ops.argtypes = [i32, i32, i32, i32, i32, i32, i32, vp, ctypes.POINTER(vp)]
    lib.fns_b200_mg_destroy.argtypes = [vp]
    lib.fns_b200_mg_last_error.argtypes = [vp]
    lib.fns_b200_mg_range.argtypes = [vp, i32, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.fns_b200_mg_sample_rows.argtypes = [vp, vp, i32, i64, i32, vp, i64, vp, i64, vp, vp, vp, vp]
    lib.fns_b200_mg_gather_tokens.argtypes = [vp, vp, i32, vp, vp]
    lib.fns_b200_mg_profile_begin.argtypes = [vp, i32]
    lib.fns_b200_mg_profile_end.argtypes = [vp, vp, f64p, f64p, f64p, ctypes.POINTER(i32)]
    for name in SYMBOLS + INTERNAL_SYMBOLS:
        getattr(lib, name).restype = i32
    lib.fns_b200_last_error.restype = ctypes.c_char_p
    lib.fns_b200_engine_last_error.restype = ctypes.c_char_p
    lib.fns_b200_mg_last_error.restype = ctypes.c_char_p
    lib.fns_b200_spec_policy_init.restype = None
    lib.fns_b200_spec_policy_new_request.restype = None
    lib.fns_b200_spec_observe.restype = None
    lib.fns_b200_launch_count.restype = ctypes.c_int64
    lib.fns_b200_engine_sampler.restype = vp
    lib.fns_b200_engine_device_tokens.restype = vp
    _lib = lib
    return lib


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _dtype_code(t) -> int:
    import torch

    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"logits must be float32 or bfloat16, got {t.dtype}")


def _stream():
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def params_to_device(params: np.ndarray, device):
    """Uploads a host parameter array as a uint8 tensor of the same bytes."""
    import torch

    assert params.dtype == PARAMS_DTYPE
    return torch.from_numpy(params.view(np.uint8).reshape(-1).copy()).to(device)


class Sampler:
    """One workspace (``fns_b200_sampler``) on one GPU.  Arguments are CUDA tensors; calls are asynchronous on
    torch's current stream, like the C calls they forward to."""

    def __init__(self, device: int = 0, max_rows: int = 256, max_vocab: int = 151936, k_cap: int = 64,
                 max_history: int = 4096):
        self.lib = load_library()
        self.device = int(device)
        self.k_cap = int(k_cap)
        h = ctypes.c_void_p()
        rc = self.lib.fns_b200_create(self.device, max_rows, max_vocab, k_cap, max_history, ctypes.byref(h))
        if rc != OK:
            raise SamplerError(rc, "fns_b200_create failed")
        self.handle = h

    def close(self):
        if getattr(self, "handle", None):
            self.lib.fns_b200_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != OK:
            raise SamplerError(rc, self.lib.fns_b200_last_error(self.handle).decode())

    def set_slices(self, slices: int):
        self._check(self.lib.fns_b200_set_slices(self.handle, slices))

    def set_cluster_rows(self, rows: int):
        self._check(self.lib.fns_b200_set_cluster_rows(self.handle, rows))

    def set_threads(self, threads: int):
        self._check(self.lib.fns_b200_set_threads(self.handle, threads))

    def plan(self, dtype: int, vocab: int, rows: int, history_bound: int = 0):
        s, l, b = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        self._check(self.lib.fns_b200_plan(self.handle, dtype, vocab, rows, history_bound, ctypes.byref(s),
                                           ctypes.byref(l), ctypes.byref(b)))
        return {"slices": s.value, "slice_len": l.value, "smem_bytes": b.value}

    def device_status(self):
        self._check(self.lib.fns_b200_device_status(self.handle, _stream()))

    def launch_count(self) -> int:
        return int(self.lib.fns_b200_launch_count(self.handle))

    def profile_begin(self, max_calls: int):
        self._check(self.lib.fns_b200_profile_begin(self.handle, max_calls))

    def profile_end(self):
        """(select_ms, finalize_ms, calls) summed over the calls recorded since profile_begin."""
        a, b, n = ctypes.c_double(), ctypes.c_double(), ctypes.c_int()
        self._check(self.lib.fns_b200_profile_end(self.handle, _stream(), ctypes.byref(a), ctypes.byref(b),
                                                  ctypes.byref(n)))
        return a.value, b.value, n.value

    def sample_rows(self, logits, params, out, masks=None, history=None, history_len=None, vocab=None):
        rows = logits.shape[0]
        vocab = int(vocab if vocab is not None else logits.shape[1])
        self._check(self.lib.fns_b200_sample_rows(
            self.handle, _ptr(logits), _dtype_code(logits), logits.stride(0), vocab, rows,
            _ptr(masks), masks.stride(0) if masks is not None else 0,
            _ptr(history), history.stride(0) if history is not None else 0, _ptr(history_len),
            _ptr(params), _ptr(out), _stream()))
        return out

    def sample_one(self, logits, params_host: np.ndarray, out, mask=None):
        p = np.ascontiguousarray(params_host.reshape(-1)[:1])
        self._check(self.lib.fns_b200_sample_one(
            self.handle, _ptr(logits), _dtype_code(logits), logits.numel(), _ptr(mask), None, 0,
            ctypes.c_void_p(p.ctypes.data), _ptr(out), _stream()))
        return out

    def select_rows(self, logits, params, out_cands, id_base=0, masks=None, history=None, history_len=None,
                    vocab=None):
        rows = logits.shape[0]
        vocab = int(vocab if vocab is not None else logits.shape[1])
        self._check(self.lib.fns_b200_select_rows(
            self.handle, _ptr(logits), _dtype_code(logits), logits.stride(0), vocab, rows, int(id_base),
            _ptr(masks), masks.stride(0) if masks is not None else 0,
            _ptr(history), history.stride(0) if history is not None else 0, _ptr(history_len),
            _ptr(params), _ptr(out_cands), _stream()))
        return out_cands

    def finalize_rows(self, cands, lists: int, list_len: int, rows: int, params, out_tokens=None, out_cands=None,
                      list_stride=None, row_stride=None):
        """Default layout [rows][lists][list_len]; pass strides (in entries) for anything else."""
        list_stride = list_len if list_stride is None else list_stride
        row_stride = lists * list_len if row_stride is None else row_stride
        self._check(self.lib.fns_b200_finalize_rows(
            self.handle, _ptr(cands), lists, list_len, list_stride, row_stride, rows, _ptr(params),
            _ptr(out_tokens), _ptr(out_cands), _stream()))

    def verify_accept(self, logits, draft, params, out_tokens, out_accept, masks=None, history=None,
                      history_len=None, vocab=None):
        n_draft = int(draft.shape[1])
        windows = int(draft.shape[0])
        assert logits.shape[0] == windows * (n_draft + 1)
        vocab = int(vocab if vocab is not None else logits.shape[1])
        self._check(self.lib.fns_b200_verify_accept(
            self.handle, _ptr(logits), _dtype_code(logits), logits.stride(0), vocab, windows, n_draft, _ptr(draft),
            _ptr(masks), masks.stride(0) if masks is not None else 0,
            _ptr(history), history.stride(0) if history is not None else 0, _ptr(history_len),
            _ptr(params), _ptr(out_tokens), _ptr(out_accept), _stream()))


def cands_tensor(rows: int, k_cap: int, device):
    """Device buffer for ``rows * k_cap`` ``fns_b200_cand`` entries (as int32 pairs: value bits, id)."""
    import torch

    return torch.empty((rows, k_cap, 2), dtype=torch.int32, device=device)


def cands_to_numpy(t) -> np.ndarray:
    """(rows, k_cap) structured array with fields value / id from a ``cands_tensor``."""
    a = t.detach().cpu().numpy()
    out = np.empty(a.shape[:2], dtype=CAND_DTYPE)
    out["value"] = a[..., 0].view(np.float32)
    out["id"] = a[..., 1]
    return out


def _host(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data if isinstance(a, np.ndarray) else a.data_ptr())


class Engine:
    """``fns_b200_engine``: the sampler part of the reference's ``fns::Engine`` (pick_async / pick_wait / verify /
    reset_presence / presence_commit, src/engine.cu:733-866) for a batch of sessions.  Host arguments are numpy
    arrays or pinned CPU tensors; logits are a CUDA tensor, or a (pinned) CPU tensor with ``logits_on_host``."""

    def __init__(self, device: int = 0, max_rows: int = 256, vocab: int = 151936, k_cap: int = 64,
                 max_history: int = 4096):
        self.lib = load_library()
        self.vocab = vocab
        h = ctypes.c_void_p()
        rc = self.lib.fns_b200_engine_create(device, max_rows, vocab, k_cap, max_history, ctypes.byref(h))
        if rc != OK:
            raise SamplerError(rc, "fns_b200_engine_create failed")
        self.handle = h

    def close(self):
        if getattr(self, "handle", None):
            self.lib.fns_b200_engine_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != OK:
            raise SamplerError(rc, self.lib.fns_b200_engine_last_error(self.handle).decode())

    def launch_count(self) -> int:
        return int(self.lib.fns_b200_launch_count(self.lib.fns_b200_engine_sampler(self.handle)))

    def pick_async(self, logits, params_host, masks_host=None, history_host=None, history_len_host=None,
                   logits_on_host=False, host_stable=False):
        """``host_stable``: the host buffers stay unchanged until ``pick_wait``; page-locked ones are then read by
        the GPU in place (FNS_B200_HOST_STABLE), and with a mask only the allowed logits cross PCIe."""
        rows = logits.shape[0]
        hs = 0 if history_host is None else history_host.shape[1]
        self._check(self.lib.fns_b200_engine_pick_async(
            self.handle, ctypes.c_void_p(logits.data_ptr()), (1 if logits_on_host else 0) | (2 if host_stable else 0),
            _dtype_code(logits),
            logits.stride(0), rows, _host(masks_host), _host(history_host), hs, _host(history_len_host),
            _host(params_host), _stream()))

    def mask_cache(self, slots: int):
        self._check(self.lib.fns_b200_engine_mask_cache(self.handle, slots))

    def mask_stats(self):
        """(hits, misses, bytes_uploaded) of the device-side mask cache."""
        a, b, c = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        self._check(self.lib.fns_b200_engine_mask_stats(self.handle, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
        return a.value, b.value, c.value

    def words(self) -> int:
        return int(self.lib.fns_b200_engine_words(self.handle))

    def pick_async_dl(self, logits, params_host, masks=None, mask_states=None):
        """``masks``: the producer's CPU int32 tensor ([words] or [rows][words]) or None; ``mask_states``: uint64
        [rows] grammar-state ids for the device-side cache, or None."""
        dl = None if masks is None else (masks if isinstance(masks, DLTensor) else DLTensor.of(masks))
        st = None if mask_states is None else np.ascontiguousarray(mask_states, dtype=np.uint64)
        self._check(self.lib.fns_b200_engine_pick_async_dl(
            self.handle, ctypes.c_void_p(logits.data_ptr()), _dtype_code(logits), logits.stride(0), logits.shape[0],
            None if dl is None else ctypes.addressof(dl), _host(st), _host(params_host), _stream()))

    def pick_wait(self, rows: int) -> np.ndarray:
        out = np.empty(rows, np.int32)
        self._check(self.lib.fns_b200_engine_pick_wait(self.handle, _host(out)))
        return out

    def pick(self, logits, params_host, **kw) -> np.ndarray:
        self.pick_async(logits, params_host, **kw)
        return self.pick_wait(logits.shape[0])

    def device_tokens_ptr(self) -> int:
        return int(self.lib.fns_b200_engine_device_tokens(self.handle) or 0)

    def reset(self):
        self._check(self.lib.fns_b200_engine_reset(self.handle, _stream()))

    def append(self, tokens_dev_ptr: int, tokens_stride: int, rows: int, counts_host=None):
        self._check(self.lib.fns_b200_engine_append(self.handle, ctypes.c_void_p(tokens_dev_ptr), tokens_stride, rows,
                                                    _host(counts_host), _stream()))

    def verify(self, logits, draft_host: np.ndarray, params_host, masks_host=None):
        windows, n_draft = draft_host.shape
        tokens = np.empty((windows, n_draft + 1), np.int32)
        accept = np.empty(windows, np.int32)
        self._check(self.lib.fns_b200_engine_verify(
            self.handle, ctypes.c_void_p(logits.data_ptr()), _dtype_code(logits), logits.stride(0), windows, n_draft,
            _host(np.ascontiguousarray(draft_host, dtype=np.int32)), _host(masks_host), _host(params_host),
            _host(tokens), _host(accept), _stream()))
        return tokens, accept


MAX_WINDOW = 32


class DLTensor(ctypes.Structure):
    """``fns_b200_dl_tensor`` = the layout of DLPack's DLTensor."""

    _fields_ = [("data", ctypes.c_void_p), ("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32),
                ("ndim", ctypes.c_int32), ("dtype_code", ctypes.c_uint8), ("dtype_bits", ctypes.c_uint8),
                ("dtype_lanes", ctypes.c_uint16), ("shape", ctypes.POINTER(ctypes.c_int64)),
                ("strides", ctypes.POINTER(ctypes.c_int64)), ("byte_offset", ctypes.c_uint64)]

    @classmethod
    def of(cls, t):
        """View of a CPU int32 / uint32 torch tensor or numpy array (kept alive by the returned object)."""
        import torch

        if isinstance(t, np.ndarray):
            t = torch.from_numpy(t.view(np.int32) if t.dtype == np.uint32 else t)
        d = cls()
        d._keep = (t, (ctypes.c_int64 * t.dim())(*t.shape), (ctypes.c_int64 * t.dim())(*t.stride()))
        d.data, d.device_type, d.device_id, d.ndim = t.data_ptr(), 3 if t.is_pinned() else 1, 0, t.dim()
        d.dtype_code, d.dtype_bits, d.dtype_lanes = (0 if t.dtype == torch.int32 else 2 if t.is_floating_point() else 1), \
            t.element_size() * 8, 1
        d.shape, d.strides, d.byte_offset = d._keep[1], d._keep[2], 0
        return d


class SpecCounters(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("generated", "windows", "drafted", "accepted", "emitted", "skipped", "iterations")]


class SpecPolicy(ctypes.Structure):
    _fields_ = [("spec", ctypes.c_int32), ("skipped_proposals", ctypes.c_int32), ("accepted", ctypes.c_uint64),
                ("offered", ctypes.c_uint64), ("cost", ctypes.c_double * (MAX_WINDOW + 1))]


GRAMMAR_FILL = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32))
GRAMMAR_ACCEPT = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_int32)
GRAMMAR_TERMINATED = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)
GRAMMAR_ROLLBACK = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int)
MODEL_FORWARD = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.c_int, ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int64))


class Grammar(ctypes.Structure):  # fns_b200_grammar
    _fields_ = [("user", ctypes.c_void_p), ("fill", GRAMMAR_FILL), ("accept", GRAMMAR_ACCEPT),
                ("terminated", GRAMMAR_TERMINATED), ("rollback", GRAMMAR_ROLLBACK)]


class Model(ctypes.Structure):  # fns_b200_model
    _fields_ = [("user", ctypes.c_void_p), ("forward", MODEL_FORWARD)]


def params_from_json(line: str) -> np.ndarray:
    """The sampling fields of one request line (tools/fns_serve/fns_serve.cpp:291-303) as one ``fns_b200_params``."""
    p = np.zeros(1, dtype=PARAMS_DTYPE)
    rc = load_library().fns_b200_params_from_json(line.encode(), ctypes.c_void_p(p.ctypes.data))
    if rc != OK:
        raise SamplerError(rc, "fns_b200_params_from_json failed")
    return p


def lookup_draft(history, want: int) -> np.ndarray:
    """Prompt-lookup draft of the reference (include/fns/lookup.h:12-27), through the library's host function."""
    h = np.ascontiguousarray(history, dtype=np.int32)
    out = np.zeros(max(want, 1), np.int32)
    n = load_library().fns_b200_lookup_draft(_host(h), h.size, want, _host(out))
    return out[:n].copy()
