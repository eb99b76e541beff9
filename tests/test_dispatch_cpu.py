"""The multi-GPU dispatcher without GPUs: two gloo ranks on CPU.

The dispatcher is C++ (csrc/fns_mg.cu, behind fns_b200_mg_*): it partitions, lays out the exchange buffers, calls
the kernels and the collective through a table of function pointers, and hands the merge its strides.  Here that
table is filled with stand-ins built on the CPU oracle (test infrastructure, never shipped) and a gloo all-gather,
so the dispatcher's own code runs exactly as it does on GPUs with NCCL, on host memory.
"""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.dispatch import RowSharded, VocabSharded, shard_range, vocab_shard
from flintnsteel_b200.sampler import CAND_DTYPE, PARAMS_DTYPE

vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
ALLOC = ctypes.CFUNCTYPE(i32, vp, sz, ctypes.POINTER(vp))
RELEASE = ctypes.CFUNCTYPE(i32, vp, vp)
COPY = ctypes.CFUNCTYPE(i32, vp, vp, vp, sz, vp)
SELECT = ctypes.CFUNCTYPE(i32, vp, vp, i32, i64, i32, i32, ctypes.c_int32, vp, i64, vp, i64, vp, vp, vp, vp)
FINALIZE = ctypes.CFUNCTYPE(i32, vp, vp, i32, i32, i64, i64, i32, vp, vp, vp)
SAMPLE = ctypes.CFUNCTYPE(i32, vp, vp, i32, i64, i32, i32, vp, i64, vp, i64, vp, vp, vp, vp)
ALLGATHER = ctypes.CFUNCTYPE(i32, vp, vp, vp, sz, vp)


class Ops(ctypes.Structure):  # fns_b200_mg_ops (csrc/fns_internal.h)
    _fields_ = [("user", vp), ("alloc", ALLOC), ("release", RELEASE), ("copy", COPY), ("select_rows", SELECT),
                ("finalize_rows", FINALIZE), ("sample_rows", SAMPLE), ("allgather", ALLGATHER)]


def view(ptr, dtype, count):
    """numpy view of ``count`` items of ``dtype`` at a raw address."""
    if not ptr or count == 0:
        return None
    nbytes = np.dtype(dtype).itemsize * count
    return np.frombuffer((ctypes.c_ubyte * nbytes).from_address(ptr), dtype=dtype, count=count)


class OracleOps:
    """The dispatcher's table on host memory: kernels = the CPU oracle, collective = gloo (or none for one rank)."""

    def __init__(self, k_cap, world):
        from oracle.binding import Oracle

        self.o, self.k_cap, self.world, self.keep = Oracle(), k_cap, world, {}
        self.table = Ops(None, ALLOC(self.alloc), RELEASE(self.release), COPY(self.copy), SELECT(self.select_rows),
                         FINALIZE(self.finalize_rows), SAMPLE(self.sample_rows), ALLGATHER(self.allgather))

    def alloc(self, user, nbytes, out):
        buf = (ctypes.c_ubyte * max(int(nbytes), 1))()
        self.keep[ctypes.addressof(buf)] = buf
        out[0] = ctypes.addressof(buf)
        return 0

    def release(self, user, p):
        self.keep.pop(p, None)
        return 0

    def copy(self, user, dst, src, nbytes, stream):
        ctypes.memmove(dst, src, nbytes)
        return 0

    def _k(self, p):
        return 1 if p["temperature"][0] <= 0 else self.o.clamp_k(int(p["top_k"][0]), self.k_cap)

    def _rows(self, logits, dtype, row_stride, vocab, rows):
        assert dtype == 0  # fp32 on the host
        return np.stack([view(logits + 4 * r * row_stride, np.float32, vocab) for r in range(rows)])

    def select_rows(self, user, logits, dtype, row_stride, vocab, rows, id_base, masks, mstride, hist, hstride, hlen, params,
                    out, stream):
        x = self._rows(logits, dtype, row_stride, vocab, rows)
        p = view(params, PARAMS_DTYPE, rows)
        cands = view(out, CAND_DTYPE, rows * self.k_cap).reshape(rows, self.k_cap)
        lens = view(hlen, np.int32, rows)
        for r in range(rows):
            row = x[r]
            if hist:
                h = view(hist + 4 * r * hstride, np.int32, int(lens[r]))
                if h is not None:
                    row = self.o.penalize(row, h - id_base, None, float(p["repetition"][r]), float(p["presence"][r]),
                                          float(p["frequency"][r]))
            m = view(masks + 4 * r * mstride, np.uint32, (vocab + 31) // 32) if masks else None
            v, i, _ = self.o.topk(row, m, self._k(p[r:r + 1]), id_base)
            cands["value"][r] = -np.finfo(np.float32).max
            cands["id"][r] = 0x7FFFFFFF
            cands["value"][r, : v.size] = v
            cands["id"][r, : i.size] = i
        return 0

    def finalize_rows(self, user, cands, lists, list_len, list_stride, row_stride, rows, params, out_tokens, stream):
        p = view(params, PARAMS_DTYPE, rows)
        tok = view(out_tokens, np.int32, rows)
        for r in range(rows):
            at = [cands + 8 * (r * row_stride + l * list_stride) for l in range(lists)]
            v = np.stack([view(a, CAND_DTYPE, list_len)["value"] for a in at])
            i = np.stack([view(a, CAND_DTYPE, list_len)["id"] for a in at])
            mv, mi, nk = self.o.merge(v, i, self._k(p[r:r + 1]))
            tok[r] = self.o.draw(mv, mi, nk, p[r:r + 1])
        return 0

    def sample_rows(self, user, logits, dtype, row_stride, vocab, rows, masks, mstride, hist, hstride, hlen, params, out,
                    stream):
        x = self._rows(logits, dtype, row_stride, vocab, rows)
        p = view(params, PARAMS_DTYPE, rows)
        m = np.stack([view(masks + 4 * r * mstride, np.uint32, (vocab + 31) // 32) for r in range(rows)]) if masks else None
        h = np.stack([view(hist + 4 * r * hstride, np.int32, hstride) for r in range(rows)]) if hist else None
        tok, _ = self.o.sample_rows(x, p.copy(), self.k_cap, m, h, view(hlen, np.int32, rows) if hist else None)
        view(out, np.int32, rows)[:] = tok
        return 0

    def allgather(self, user, send, recv, nbytes, stream):
        mine = torch.from_numpy(view(send, np.uint8, nbytes).copy())
        everything = torch.empty(self.world * nbytes, dtype=torch.uint8)
        dist.all_gather_into_tensor(everything, mine)
        view(recv, np.uint8, self.world * nbytes)[:] = everything.numpy()
        return 0


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- vocabulary shards: rows with a 50 % mask, history with global ids, k_cap 128
        w = wl.large_vocab(seed=5, rows=6, vocab=20_000 + 64)  # 627 words: does not split evenly
        w.params["top_k"], w.params["repetition"], w.params["presence"] = 100, 1.2, 0.3
        hist = wl.rng(9).integers(0, w.vocab, size=(6, 50), dtype=np.int32)
        hlen = np.array([50, 0, 7, 50, 1, 33], np.int32)
        ops = OracleOps(128, world)
        vs = VocabSharded(-1, w.vocab, 128, rank, world, max_rows=6, max_history=50, ops=ops.table)
        lo, hi = vs.lo, vs.hi
        x = torch.from_numpy(w.logits_f32()[:, lo:hi].copy())
        m = torch.from_numpy(np.ascontiguousarray(w.masks[:, lo // 32:(hi + 31) // 32]).view(np.int32))
        params = torch.from_numpy(w.params.view(np.uint8).reshape(-1).copy())
        out = torch.empty(6, dtype=torch.int32)
        vs.sample(x, params, out, masks_shard=m, history=torch.from_numpy(hist), history_len=torch.from_numpy(hlen))
        expect, _ = ops.o.sample_rows(w.logits_f32(), w.params, 128, w.masks, hist, hlen)
        results[f"vocab{rank}"] = (out.numpy().tolist(), expect.tolist(), (lo, hi))
        vs.close()
        # ---- row shards: 7 rows over 2 ranks (4 + 3), tokens gathered on every rank
        b = wl.session_batch(seed=8, rows=7, vocab=4096, history=32)
        ops2 = OracleOps(64, world)
        rs = RowSharded(-1, 4096, 64, rank, world, max_rows=7, max_history=32, ops=ops2.table)
        a, z = rs.rows(7)
        mine = torch.empty(z - a, dtype=torch.int32)
        rs.sample(torch.from_numpy(b.logits[a:z].copy()), torch.from_numpy(b.params[a:z].view(np.uint8).reshape(-1).copy()), mine,
                  masks=torch.from_numpy(b.masks[a:z].view(np.int32).copy()), history=torch.from_numpy(b.history[a:z].copy()),
                  history_len=torch.from_numpy(b.history_len[a:z].copy()))
        everything = rs.gather_tokens(mine, 7)
        expect, _ = ops2.o.sample_rows(b.logits, b.params, 64, b.masks, b.history, b.history_len)
        results[f"rows{rank}"] = (everything.numpy().tolist(), expect.tolist(), (a, z))
        rs.close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
        results = dict(results)
    assert results["vocab0"][2] == (0, 10048) and results["vocab1"][2] == (10048, 20064)
    for r in range(world):
        got, expect, _ = results[f"vocab{r}"]
        assert got == expect, f"vocab-sharded tokens differ on rank {r}"
        got, expect, _ = results[f"rows{r}"]
        assert got == expect, f"row-sharded tokens differ on rank {r}"
    assert results["rows0"][2] == (0, 4) and results["rows1"][2] == (4, 7)


def test_shard_arithmetic():
    assert [shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [shard_range(256, r, 8) for r in range(8)] == [(32 * r, 32 * r + 32) for r in range(8)]
    for vocab, world in ((262_144, 8), (151_936, 4), (151_936, 8), (1000, 3), (33, 2)):
        edges = [vocab_shard(vocab, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == vocab
        for (a, b), (c, d) in zip(edges, edges[1:]):
            assert b == c and b % 32 == 0  # whole bitmask words
    assert vocab_shard(262_144, 3, 8) == (98_304, 131_072)


def test_the_library_splits_as_the_python_helpers_do():
    """fns_b200_mg_range against shard_range / vocab_shard, and the refusal of a shard without a bitmask word."""
    ops = OracleOps(64, 1)
    for vocab, world in ((262_144, 8), (151_936, 8), (1000, 3), (20_064, 2)):
        for rank in range(world):
            vs = VocabSharded(-1, vocab, 64, rank, world, max_rows=4, ops=OracleOps(64, world).table)
            assert (vs.lo, vs.hi) == vocab_shard(vocab, rank, world)
            vs.close()
            rs = RowSharded(-1, vocab, 64, rank, world, max_rows=64, ops=OracleOps(64, world).table)
            assert rs.rows(37) == shard_range(37, rank, world)
            rs.close()
    with pytest.raises(Exception):
        VocabSharded(-1, 33, 64, 0, 3, max_rows=4, ops=ops.table)  # 2 words for 3 ranks: one shard would be empty


def test_single_rank_is_the_plain_path():
    ops = OracleOps(64, 1)
    w = wl.session_batch(seed=3, rows=3, vocab=2048, history=16)
    vs = VocabSharded(-1, w.vocab, 64, max_rows=3, max_history=16, ops=ops.table)
    out = torch.empty(3, dtype=torch.int32)
    vs.sample(torch.from_numpy(w.logits), torch.from_numpy(w.params.view(np.uint8).reshape(-1).copy()), out,
              masks_shard=torch.from_numpy(w.masks.view(np.int32)), history=torch.from_numpy(w.history),
              history_len=torch.from_numpy(w.history_len))
    expect, _ = ops.o.sample_rows(w.logits, w.params, 64, w.masks, w.history, w.history_len)
    assert out.numpy().tolist() == expect.tolist()
