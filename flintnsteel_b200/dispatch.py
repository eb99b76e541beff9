"""Multi-GPU dispatcher: one process per GPU.  A thin ctypes layer over ``fns_b200_mg_*`` (csrc/fns_mg.cu); the
partitioning, the exchange and the launch order live in the C++ library, so a C++ engine calls the same code.

The reference is single-GPU, one row per call (its docs/ENGINE.md:132); this layer is new.  Two partitions:

* ``RowSharded``   - independent sessions.  Every rank samples the rows its own LM head produced, with its own
                     workspace and stream.  No collective on the data path (tokens can be gathered afterwards:
                     4 bytes per row).
* ``VocabSharded`` - one very large vocabulary split evenly over the ranks on 32-id boundaries.  Each rank selects
                     the top-k_cap (value, id) candidates of its shard of every row, ONE NCCL all-gather brings
                     the lists into local memory (k_cap * 8 bytes per row and rank), and every rank runs the same
                     merge + draw, so all ranks hold the same tokens without a broadcast.  Exact for the reason the
                     reference's 128 slices are (src/kernels.cu:594-597).

``torch.distributed`` is used for one thing only: to hand rank 0's NCCL unique id to the other ranks when the
dispatcher is created.  The library then owns its communicator.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import sampler as _s

ROWS, VOCAB = 0, 1
ID_BYTES = 128


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous near-even split: the first ``total % world`` ranks get one more (the rule of fns_b200_mg_range)."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def vocab_shard(vocab: int, rank: int, world: int) -> tuple[int, int]:
    """Even split whose boundaries fall on 32-id words, so that every shard owns whole bitmask words."""
    words = (vocab + 31) // 32
    wlo, whi = shard_range(words, rank, world)
    return wlo * 32, min(vocab, whi * 32)


def _exchange_unique_id(rank: int, world: int, group=None) -> bytes:
    """Rank 0 asks NCCL for a unique id; every rank gets the same 128 bytes (through the caller's process group)."""
    import torch
    import torch.distributed as dist

    lib = _s.load_library()
    buf = (ctypes.c_ubyte * ID_BYTES)()
    if rank == 0:
        rc = lib.fns_b200_mg_unique_id(buf)
        if rc != _s.OK:
            raise _s.SamplerError(rc, "fns_b200_mg_unique_id failed (libnccl.so.2 not loadable?)")
    t = torch.tensor(list(buf), dtype=torch.uint8)
    if dist.get_backend(group) == "nccl":
        t = t.cuda()
    dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    return bytes(t.cpu().tolist())


class _Dispatcher:
    mode = ROWS

    def __init__(self, device: int, vocab: int, k_cap: int, rank: int = 0, world: int = 1, max_rows: int = 256,
                 max_history: int = 0, group=None, ops=None):
        self.lib = _s.load_library()
        self.device, self.vocab, self.k_cap, self.rank, self.world = device, vocab, k_cap, rank, world
        h = ctypes.c_void_p()
        self._host_only = ops is not None
        if ops is not None:  # a table of stand-ins (tests): no GPU, no NCCL
            self._ops = ops
            rc = self.lib.fns_b200_mg_create_with_ops(rank, world, self.mode, max_rows, vocab, k_cap, max_history,
                                                      ctypes.addressof(ops), ctypes.byref(h))
        else:
            uid = _exchange_unique_id(rank, world, group) if world > 1 else None
            rc = self.lib.fns_b200_mg_create(device, rank, world, self.mode, max_rows, vocab, k_cap, max_history, uid,
                                             None, ctypes.byref(h))
        if rc != _s.OK:
            raise _s.SamplerError(rc, "fns_b200_mg_create failed")
        self.handle = h

    def close(self):
        if getattr(self, "handle", None):
            self.lib.fns_b200_mg_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != _s.OK:
            raise _s.SamplerError(rc, self.lib.fns_b200_mg_last_error(self.handle).decode())

    def range(self, total_rows: int = 0) -> tuple[int, int]:
        lo, hi = ctypes.c_int(), ctypes.c_int()
        self._check(self.lib.fns_b200_mg_range(self.handle, total_rows, ctypes.byref(lo), ctypes.byref(hi)))
        return lo.value, hi.value

    def _stream(self, stream):
        if stream is not None:
            return stream
        return None if self._host_only else _s._stream()

    def _sample(self, logits, params, out, masks, history, history_len, stream):
        self._check(self.lib.fns_b200_mg_sample_rows(
            self.handle, _s._ptr(logits), _s._dtype_code(logits), logits.stride(0), logits.shape[0],
            _s._ptr(masks), masks.stride(0) if masks is not None else 0,
            _s._ptr(history), history.stride(0) if history is not None else 0, _s._ptr(history_len),
            _s._ptr(params), _s._ptr(out), stream))
        return out

    def profile_begin(self, max_calls: int):
        self._check(self.lib.fns_b200_mg_profile_begin(self.handle, max_calls))

    def profile_end(self):
        """(select_us, exchange_us, finalize_us, calls): device time per call of the three steps."""
        a, b, c, n = ctypes.c_double(), ctypes.c_double(), ctypes.c_double(), ctypes.c_int()
        self._check(self.lib.fns_b200_mg_profile_end(self.handle, _s._stream(), ctypes.byref(a), ctypes.byref(b),
                                                     ctypes.byref(c), ctypes.byref(n)))
        return a.value, b.value, c.value, n.value


class RowSharded(_Dispatcher):
    """Independent sessions: this rank owns rows ``shard_range(total_rows, rank, world)``."""

    mode = ROWS

    def rows(self, total_rows: int) -> tuple[int, int]:
        return self.range(total_rows)

    def sample(self, logits, params, out, masks=None, history=None, history_len=None, stream=None):
        """``logits`` etc. hold THIS rank's rows only (the LM head that produced them ran here)."""
        return self._sample(logits, params, out, masks, history, history_len, self._stream(stream))

    def gather_tokens(self, local_tokens, total_rows: int, out=None, stream=None):
        """Optional: every rank receives all tokens, in row order."""
        import torch

        if out is None:
            out = torch.empty(total_rows, dtype=torch.int32, device=local_tokens.device)
        self._check(self.lib.fns_b200_mg_gather_tokens(self.handle, _s._ptr(local_tokens), total_rows, _s._ptr(out),
                                                       self._stream(stream)))
        return out


class VocabSharded(_Dispatcher):
    """One vocabulary over ``world`` ranks; this rank owns ids ``[self.lo, self.hi)``."""

    mode = VOCAB

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.lo, self.hi = self.range()

    def sample(self, logits_shard, params, out, masks_shard=None, history=None, history_len=None, stream=None):
        """``logits_shard``: [rows][hi - lo] of this rank's ids; ``masks_shard``: the matching words
        [rows][(hi - lo + 31) // 32]; ``history`` holds GLOBAL ids; ``out``: int32 [rows], the same on every rank."""
        return self._sample(logits_shard, params, out, masks_shard, history, history_len, self._stream(stream))
