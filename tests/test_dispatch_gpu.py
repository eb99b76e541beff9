"""The multi-GPU dispatcher on real GPUs: two NCCL ranks, the CUDA sampler as the backend.

Skipped on a machine with one GPU (the same dispatcher logic runs on two gloo ranks in test_dispatch_cpu.py).
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
    from flintnsteel_b200.sampler import Sampler, params_to_device

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # ---- one vocabulary over the ranks: bf16 rows, 50 % mask, k_cap 128
        w = wl.large_vocab(seed=5, rows=6, vocab=20_000 + 64)
        w.params["top_k"] = 100
        s = Sampler(rank, max_rows=6, max_vocab=w.vocab, k_cap=128, max_history=0)
        vs = VocabSharded(s, w.vocab, 128, rank, world)
        lo, hi = vs.lo, vs.hi
        lg = torch.from_numpy(np.ascontiguousarray(w.logits[:, lo:hi]).view(np.int16)).to(dev).view(torch.bfloat16)
        m = torch.from_numpy(np.ascontiguousarray(w.masks[:, lo // 32:(hi + 31) // 32]).view(np.int32)).to(dev)
        out = torch.empty(6, dtype=torch.int32, device=dev)
        vs.sample(lg, params_to_device(w.params, dev), out, masks_shard=m)
        torch.cuda.synchronize()
        results[f"vocab{rank}"] = out.cpu().numpy().tolist()
        s.close()
        # ---- independent sessions: 7 rows over 2 ranks (4 + 3), tokens gathered on every rank
        b = wl.session_batch(seed=8, rows=7, vocab=4096, history=32)
        s = Sampler(rank, max_rows=7, max_vocab=4096, k_cap=64, max_history=32)
        rs = RowSharded(s, rank, world)
        a, z = rs.rows(7)
        mine = torch.empty(z - a, dtype=torch.int32, device=dev)
        rs.sample(torch.from_numpy(b.logits[a:z]).to(dev), params_to_device(b.params[a:z], dev), mine,
                  masks=torch.from_numpy(b.masks[a:z].view(np.int32)).to(dev),
                  history=torch.from_numpy(b.history[a:z]).to(dev),
                  history_len=torch.from_numpy(b.history_len[a:z]).to(dev))
        results[f"rows{rank}"] = rs.gather_tokens(mine, 7).cpu().numpy().tolist()
        s.close()
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
    for r in range(world):
        assert results[f"vocab{r}"] == want_vocab.tolist(), f"vocabulary-sharded tokens differ on rank {r}"
        assert results[f"rows{r}"] == want_rows.tolist(), f"row-sharded tokens differ on rank {r}"
