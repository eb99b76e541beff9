"""The drop-in boundary without a GPU: the library builds for sm_100a, loads, and exports every symbol that
include/fns_b200.h declares; argument checks that run before any CUDA call return status codes."""
import ctypes
import os
import re
import subprocess

import numpy as np

from flintnsteel_b200 import sampler

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "fns_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fns_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert header_functions() == sorted(sampler.SYMBOLS)


def test_library_exports_every_declared_symbol(library_path):
    lib = ctypes.CDLL(library_path)
    for name in header_functions():
        assert hasattr(lib, name), name


def test_params_struct_layout_matches_header():
    # 6 floats, 2 int32, 2 uint64 = 48 bytes, the same bytes as the oracle's struct
    from oracle.binding import PARAMS_DTYPE as ORACLE_PARAMS

    assert sampler.PARAMS_DTYPE.itemsize == 48
    assert sampler.PARAMS_DTYPE == ORACLE_PARAMS
    assert [sampler.PARAMS_DTYPE.fields[n][1] for n in ("top_k", "seed", "counter")] == [24, 32, 40]
    assert sampler.CAND_DTYPE.itemsize == 8


def test_null_and_range_arguments_return_status_not_abort(library_path):
    lib = sampler.load_library()
    h = ctypes.c_void_p()
    assert lib.fns_b200_create(0, 0, 100, 64, 0, ctypes.byref(h)) == sampler.ERR_ARG       # rows = 0
    assert lib.fns_b200_create(0, 1, 100, 0, 0, ctypes.byref(h)) == sampler.ERR_ARG        # k_cap = 0
    assert lib.fns_b200_create(0, 1, 100, 2048, 0, ctypes.byref(h)) == sampler.ERR_ARG     # k_cap > 1024
    assert lib.fns_b200_create(0, 1, 100, 64, 10**6, ctypes.byref(h)) == sampler.ERR_ARG   # history too long
    assert lib.fns_b200_create(0, 1, 100, 64, 0, None) == sampler.ERR_ARG
    assert lib.fns_b200_sample_rows(None, None, 0, 0, 0, 0, None, 0, None, 0, None, None, None, None) == sampler.ERR_ARG
    assert lib.fns_b200_presence_apply(None, None, 0, 0.0, None) == sampler.ERR_ARG
    assert lib.fns_b200_io_advance(None, 0, None) == sampler.ERR_ARG
    assert lib.fns_b200_destroy(None) == sampler.OK
    assert lib.fns_b200_last_error(None) == b"null handle"


def test_compat_layer_exports_the_reference_signatures(library_path):
    """The fns::k entry points must mangle to the same names as the reference's (src/kernels.cuh:67-88): the
    mangled name encodes namespace, function name and every parameter type."""
    out = subprocess.run(["nm", "-D", "--defined-only", library_path], capture_output=True, text=True, check=True).stdout
    names = {line.split()[-1] for line in out.splitlines() if line.strip()}
    expected = [
        "_ZN3fns1k6argmaxEPKfiPiP11CUstream_stPKj",
        "_ZN3fns1k6sampleEPKfiPKjiffmmPiP11CUstream_st",
        "_ZN3fns1k14presence_applyEPfPKfifP11CUstream_st",
        "_ZN3fns1k13presence_markEPfPKiP11CUstream_st",
        "_ZN3fns1k18presence_apply_colEPfPKfPKiiifP11CUstream_st",
        "_ZN3fns1k15presence_mark_nEPfPKiiP11CUstream_st",
        "_ZN3fns1k10io_advanceEPiiP11CUstream_st",
    ]
    for name in expected:
        assert name in names, name
    ref = os.path.join(ROOT, "oracle", "_ref", "libfns_ref.so")
    if os.path.exists(ref):  # the reference's own object exports exactly these names
        rout = subprocess.run(["nm", "-D", "--defined-only", ref], capture_output=True, text=True, check=True).stdout
        rnames = {line.split()[-1] for line in rout.splitlines() if line.strip()}
        for name in expected:
            assert name in rnames, name


def test_make_params_defaults_are_the_references():
    p = sampler.make_params(3)
    assert np.all(p["temperature"] == 0) and np.all(p["top_p"] == 1) and np.all(p["top_k"] == 0)
    assert np.all(p["repetition"] == 1) and np.all(p["presence"] == 0) and np.all(p["min_p"] == 0)


def test_lookup_draft_of_the_library_matches_the_oracle(library_path, oracle):
    """fns_b200_lookup_draft (include/fns/lookup.h:12-27) is host code: the reference's cases and 1,000 random
    histories through the library's own entry point, against the oracle's restatement."""
    h = [1, 2, 3, 4, 9, 9, 1, 2, 3, 4]
    assert list(sampler.lookup_draft(h, 3)) == [9, 9, 1]
    assert list(sampler.lookup_draft([7, 8, 5, 7, 8], 4)) == [5, 7, 8]
    assert list(sampler.lookup_draft([1, 2, 3], 2)) == []
    assert list(sampler.lookup_draft([1, 1, 1, 1, 1, 1], 2)) == [1]
    assert list(sampler.lookup_draft([], 2)) == [] and list(sampler.lookup_draft([5, 5, 5], 0)) == []
    g = np.random.default_rng(12)
    for _ in range(1000):
        n = int(g.integers(0, 60))
        hist = g.integers(0, int(g.integers(2, 7)), size=n).astype(np.int32)  # a small alphabet: n-grams repeat
        want = int(g.integers(1, 9))
        assert list(sampler.lookup_draft(hist, want)) == list(oracle.lookup_draft(hist, want)), (hist.tolist(), want)
