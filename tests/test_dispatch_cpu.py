"""The multi-GPU dispatcher without GPUs: two gloo ranks on CPU.

The dispatcher (flintnsteel_b200/dispatch.py) only allocates tensors and calls collectives; the kernels come from
its backend.  Here the backend is a stand-in built on the CPU oracle (test infrastructure, never shipped), so the
sharding arithmetic, the all-gather layout and the strides handed to the merge are exercised exactly as on NCCL.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flintnsteel_b200 import workloads as wl
from flintnsteel_b200.dispatch import RowSharded, VocabSharded, shard_range, vocab_shard
from flintnsteel_b200.sampler import PARAMS_DTYPE


class OracleBackend:
    """select_rows / finalize_rows / sample_rows with the Sampler's signatures, on CPU tensors."""

    def __init__(self, k_cap):
        from oracle.binding import Oracle

        self.o, self.k_cap = Oracle(), k_cap

    @staticmethod
    def _params(t):
        return t.numpy().view(PARAMS_DTYPE)

    def _k(self, p):
        return 1 if p["temperature"][0] <= 0 else self.o.clamp_k(int(p["top_k"][0]), self.k_cap)

    def select_rows(self, logits, params, out_cands, id_base=0, masks=None, history=None, history_len=None, vocab=None):
        p = self._params(params)
        x = logits.float().numpy()
        for r in range(x.shape[0]):
            row = x[r, :vocab]
            if history is not None:
                h = history[r, : int(history_len[r])].numpy() - id_base
                row = self.o.penalize(row, h, None, float(p["repetition"][r]), float(p["presence"][r]), float(p["frequency"][r]))
            m = None if masks is None else masks[r].numpy().view(np.uint32)
            v, i, _ = self.o.topk(row, m, self._k(p[r:r + 1]), id_base)
            out_cands[r, :, 0] = torch.from_numpy(np.full(self.k_cap, -np.finfo(np.float32).max, np.float32).view(np.int32))
            out_cands[r, :, 1] = 0x7FFFFFFF
            out_cands[r, : v.size, 0] = torch.from_numpy(v.view(np.int32).copy())
            out_cands[r, : i.size, 1] = torch.from_numpy(i.copy())

    def finalize_rows(self, cands, lists, list_len, rows, params, out_tokens=None, out_cands=None, list_stride=None,
                      row_stride=None):
        p = self._params(params)
        flat = cands.reshape(-1, 2).numpy()
        for r in range(rows):
            at = [r * row_stride + l * list_stride for l in range(lists)]
            v = np.stack([flat[a:a + list_len, 0].view(np.float32) for a in at])
            i = np.stack([flat[a:a + list_len, 1] for a in at])
            k = self._k(p[r:r + 1])
            mv, mi, nk = self.o.merge(v, i, k)
            out_tokens[r] = self.o.draw(mv, mi, nk, p[r:r + 1])

    def sample_rows(self, logits, params, out, masks=None, history=None, history_len=None):
        p = self._params(params)
        tok, _ = self.o.sample_rows(logits.float().numpy(), p, self.k_cap,
                                    None if masks is None else masks.numpy().view(np.uint32),
                                    None if history is None else history.numpy(),
                                    None if history is None else history_len.numpy())
        out.copy_(torch.from_numpy(tok))
        return out


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- vocabulary shards: bf16 rows, 50 % mask, history with global ids, k_cap 128
        w = wl.large_vocab(seed=5, rows=6, vocab=20_000 + 64)  # 627 words: does not split evenly
        w.params["top_k"], w.params["repetition"], w.params["presence"] = 100, 1.2, 0.3
        hist = wl.rng(9).integers(0, w.vocab, size=(6, 50), dtype=np.int32)
        hlen = np.array([50, 0, 7, 50, 1, 33], np.int32)
        be = OracleBackend(128)
        vs = VocabSharded(be, w.vocab, 128, rank, world)
        lo, hi = vs.lo, vs.hi
        x = torch.from_numpy(w.logits_f32()[:, lo:hi].copy())
        m = torch.from_numpy(np.ascontiguousarray(w.masks[:, lo // 32:(hi + 31) // 32]).view(np.int32))
        params = torch.from_numpy(w.params.view(np.uint8).reshape(-1).copy())
        out = torch.empty(6, dtype=torch.int32)
        vs.sample(x, params, out, masks_shard=m, history=torch.from_numpy(hist), history_len=torch.from_numpy(hlen))
        expect, _ = be.o.sample_rows(w.logits_f32(), w.params, 128, w.masks, hist, hlen)
        results[f"vocab{rank}"] = (out.numpy().tolist(), expect.tolist(), (lo, hi))
        # ---- row shards: 7 rows over 2 ranks (4 + 3), tokens gathered on every rank
        b = wl.session_batch(seed=8, rows=7, vocab=4096, history=32)
        rs = RowSharded(OracleBackend(64), rank, world)
        a, z = rs.rows(7)
        mine = torch.empty(z - a, dtype=torch.int32)
        rs.sample(torch.from_numpy(b.logits[a:z]), torch.from_numpy(b.params[a:z].view(np.uint8).reshape(-1).copy()), mine,
                  masks=torch.from_numpy(b.masks[a:z].view(np.int32)), history=torch.from_numpy(b.history[a:z]),
                  history_len=torch.from_numpy(b.history_len[a:z]))
        everything = rs.gather_tokens(mine, 7)
        expect, _ = be.o.sample_rows(b.logits, b.params, 64, b.masks, b.history, b.history_len)
        results[f"rows{rank}"] = (everything.numpy().tolist(), expect.tolist(), (a, z))
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


def test_single_rank_is_the_plain_path():
    be = OracleBackend(64)
    w = wl.session_batch(seed=3, rows=3, vocab=2048, history=16)
    vs = VocabSharded(be, w.vocab, 64)
    out = torch.empty(3, dtype=torch.int32)
    vs.sample(torch.from_numpy(w.logits), torch.from_numpy(w.params.view(np.uint8).reshape(-1).copy()), out,
              masks_shard=torch.from_numpy(w.masks.view(np.int32)), history=torch.from_numpy(w.history),
              history_len=torch.from_numpy(w.history_len))
    expect, _ = be.o.sample_rows(w.logits, w.params, 64, w.masks, w.history, w.history_len)
    assert out.numpy().tolist() == expect.tolist()
