"""The allocation-free entry point, fns_b200_sample_rows_noalloc (collected last on purpose).

Some hosts cannot allocate GPU memory when they sample: an engine that has given the whole device to its own arena,
or a call site where an allocation, which synchronises the device, is not allowed.  For them the library keeps the
sampler's scratch (candidate lists, tickets, error flag) in a static device array and offers one entry point that
needs no handle.  This test calls it through the C ABI several times in a row, with different inputs and shapes
(rows cut into slices, which use the static candidate lists and tickets, between whole-row calls), and requires the
tokens of the ordinary, handle-based entry point bit for bit: greedy rows are exact by construction, and the
sampled rows go through the same kernels with the same (seed, counter), so they are identical too.  Every call after
the first also shows that what the previous one left in the shared array does no harm.
"""
import ctypes

import numpy as np
import pytest

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.sampler import Sampler, load_library, params_to_device

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_noalloc_entry_point_matches_the_handle_based_one_call_after_call():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    dev = torch.device("cuda:0")
    lib = load_library()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ref = Sampler(0, max_rows=64, max_vocab=wl.V_QWEN, k_cap=64, max_history=2048)
    text = ctypes.create_string_buffer(256)
    # 48 and 7 rows are one block per row; 1, 3 and 4 rows are cut into slices, whose candidate lists and tickets
    # live in the static array: the calls alternate so that each kind finds what the other left behind
    for call, (seed, rows) in enumerate([(101, 48), (303, 1), (202, 7), (404, 3), (505, 4), (606, 48), (707, 1)]):
        w = wl.session_batch(seed=seed, rows=rows)
        w.params["temperature"][::3] = 0.0  # greedy rows among the sampled ones
        lg = torch.from_numpy(w.logits).to(dev)
        masks = torch.from_numpy(w.masks.view(np.int32)).to(dev)
        hist, hl = torch.from_numpy(w.history).to(dev), torch.from_numpy(w.history_len).to(dev)
        pd = params_to_device(w.params, dev)
        expect = torch.empty(rows, dtype=torch.int32, device=dev)
        ref.sample_rows(lg, pd, expect, masks=masks, history=hist, history_len=hl)
        got = torch.full((rows,), -9, dtype=torch.int32, device=dev)
        rc = lib.fns_b200_sample_rows_noalloc(
            0, lg.data_ptr(), 0, lg.stride(0), w.vocab, rows, masks.data_ptr(), masks.stride(0), hist.data_ptr(),
            hist.stride(0), hl.data_ptr(), pd.data_ptr(), got.data_ptr(), stream, text, 256)
        assert rc == 0, text.value
        torch.cuda.synchronize()
        assert torch.equal(got, expect), f"call {call}: {got.tolist()} != {expect.tolist()}"
    # more rows than the static scratch holds: refused with a clear text, nothing launched
    rc = lib.fns_b200_sample_rows_noalloc(0, lg.data_ptr(), 0, lg.stride(0), w.vocab, 65, None, 0, None, 0, None,
                                          pd.data_ptr(), got.data_ptr(), stream, text, 256)
    assert rc == 3 and b"64" in text.value
    ref.close()
