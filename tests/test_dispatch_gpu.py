"""The multi-GPU dispatcher (fns_b200_mg_*, C++) on real GPUs: two ranks, the library's own NCCL communicator.

Skipped on a machine with one GPU (the same dispatcher code runs on two gloo ranks in test_dispatch_cpu.py).
Rows shard with no collective; a vocabulary shard exchanges (value, id) candidates with ONE all-gather and every
rank must end up with the oracle's tokens.
"""
import os
import socket

import numpy as np
import pytest

from flintnsteel_b200 import workloads as wl

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, results):
    import torch.distributed as dist

    from flintnsteel_b200.dispatch import RowSharded, VocabSharded
    from flintnsteel_b200.sampler import params_to_device

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # ---- one vocabulary over the ranks: bf16 rows, 50 % mask, k_cap 128
        w = wl.large_vocab(seed=5, rows=6, vocab=20_000 + 64)
        w.params["top_k"] = 100
        vs = VocabSharded(rank, w.vocab, 128, rank, world, max_rows=6)
        lo, hi = vs.lo, vs.hi
        lg = torch.from_numpy(np.ascontiguousarray(w.logits[:, lo:hi]).view(np.int16)).to(dev).view(torch.bfloat16)
        m = torch.from_numpy(np.ascontiguousarray(w.masks[:, lo // 32:(hi + 31) // 32]).view(np.int32)).to(dev)
        out = torch.empty(6, dtype=torch.int32, device=dev)
        vs.sample(lg, params_to_device(w.params, dev), out, masks_shard=m)
        torch.cuda.synchronize()
        results[f"vocab{rank}"] = out.cpu().numpy().tolist()
        vs.close()
        # ---- the benchmark's shape in small: k_cap 1024 (k_ring under a mask), history with global ids
        w2 = wl.large_vocab(seed=6, rows=8, vocab=65_536)
        w2.params["repetition"], w2.params["presence"] = 1.1, 0.2
        hist = wl.rng(3).integers(0, w2.vocab, size=(8, 40), dtype=np.int32)
        hl = torch.full((8,), 40, dtype=torch.int32, device=dev)
        vs = VocabSharded(rank, w2.vocab, 1024, rank, world, max_rows=8, max_history=40)
        lo, hi = vs.lo, vs.hi
        lg = torch.from_numpy(np.ascontiguousarray(w2.logits[:, lo:hi]).view(np.int16)).to(dev).view(torch.bfloat16)
        m = torch.from_numpy(np.ascontiguousarray(w2.masks[:, lo // 32:(hi + 31) // 32]).view(np.int32)).to(dev)
        out = torch.empty(8, dtype=torch.int32, device=dev)
        vs.profile_begin(4)
        for _ in range(2):
            vs.sample(lg, params_to_device(w2.params, dev), out, masks_shard=m, history=torch.from_numpy(hist).to(dev),
                      history_len=hl)
        results[f"stages{rank}"] = vs.profile_end()
        results[f"vocab_big{rank}"] = out.cpu().numpy().tolist()
        vs.close()
        # ---- independent sessions: 7 rows over 2 ranks (4 + 3), tokens gathered on every rank
        b = wl.session_batch(seed=8, rows=7, vocab=4096, history=32)
        rs = RowSharded(rank, 4096, 64, rank, world, max_rows=7, max_history=32)
        a, z = rs.rows(7)
        mine = torch.empty(z - a, dtype=torch.int32, device=dev)
        rs.sample(torch.from_numpy(b.logits[a:z]).to(dev), params_to_device(b.params[a:z], dev), mine,
                  masks=torch.from_numpy(b.masks[a:z].view(np.int32)).to(dev),
                  history=torch.from_numpy(b.history[a:z]).to(dev),
                  history_len=torch.from_numpy(b.history_len[a:z]).to(dev))
        results[f"rows{rank}"] = rs.gather_tokens(mine, 7).cpu().numpy().tolist()
        rs.close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_nccl(oracle):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
        results = dict(results)
    w = wl.large_vocab(seed=5, rows=6, vocab=20_000 + 64)
    w.params["top_k"] = 100
    want_vocab, _ = oracle.sample_rows(w.logits_f32(), w.params, 128, w.masks, None, None)
    b = wl.session_batch(seed=8, rows=7, vocab=4096, history=32)
    want_rows, _ = oracle.sample_rows(b.logits, b.params, 64, b.masks, b.history, b.history_len)
    w2 = wl.large_vocab(seed=6, rows=8, vocab=65_536)
    w2.params["repetition"], w2.params["presence"] = 1.1, 0.2
    hist = wl.rng(3).integers(0, w2.vocab, size=(8, 40), dtype=np.int32)
    want_big, _ = oracle.sample_rows(w2.logits_f32(), w2.params, 1024, w2.masks, hist, np.full(8, 40, np.int32))
    for r in range(world):
        assert results[f"vocab{r}"] == want_vocab.tolist(), f"vocabulary-sharded tokens differ on rank {r}"
        assert results[f"vocab_big{r}"] == want_big.tolist(), f"vocabulary-sharded tokens (k_cap 1024) differ on rank {r}"
        sel, exch, fin, calls = results[f"stages{r}"]
        assert calls == 2 and sel > 0 and exch > 0 and fin > 0
        assert results[f"rows{r}"] == want_rows.tolist(), f"row-sharded tokens differ on rank {r}"
