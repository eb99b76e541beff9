#!/usr/bin/env python
"""Benchmark of the sampler hot path (logits -> token) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("sessions256"): 256 independent sessions per GPU per step, V = 151,936 fp32 logits, xgrammar-style
bitmask, 2,048-id histories with repetition / presence / frequency penalties, per-row temperature / top-k /
top-p (the batched configuration of the headline metric).  A step is one pass of the sampler over one batch;
several distinct batches rotate so that every step's inputs (155 MB of logits per batch, larger than the
126 MB L2) come from HBM.  Rows shard across GPUs with no data-path collective ("weak" scaling: 256 rows per
GPU).  One JSON line is printed by rank 0.

--impl reference times the CPU restatement of the reference's sampler (oracle/, OpenMP over rows on every
host core) on the same workload, a bounded sample per step; the reference's own CUDA kernels, recompiled for
sm_100a, are timed beside it (they are GPU code, so they are reported as an extra, not as the CPU arm).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sampler rows/s (V=151936 fp32, mask+penalties+top-k/p, 256 sessions per GPU)"
WORKLOAD = "sessions256"
# dram__bytes_read.sum + dram__bytes_write.sum per k_select launch, from the ncu captures summarised under profiles/
NCU_TRAFFIC_BYTES = 25.3e6
NCU_TRAFFIC_BYTES_DENSE = 162.8e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def pinned(a: np.ndarray):
    import torch

    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.pin_memory()


def run_b200(args):
    import torch
    import torch.distributed as dist

    from flintnsteel_b200 import workloads as wl
    from flintnsteel_b200.sampler import Engine, Sampler, params_to_device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    json_fd = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # stdout carries ONE JSON line: NCCL's banner and anything else a library prints go to stderr
        sys.stdout.flush()
        json_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl b200 needs a CUDA device: the sampler has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    rows, K, W = args.rows, args.steps, args.warmup

    if args.only_batch1:  # profiler runs of the few-row kernel: ten plain launches per case and nothing else
        res = {}
        cases = {"single_row_T0.7": wl.single_row(), "single_row_greedy": wl.single_row(greedy=True), "grammar_row": wl.grammar_row()}
        for name, w in cases.items():
            s = Sampler(local, max_rows=1, max_vocab=w.vocab, k_cap=64, max_history=4096)
            lg = torch.from_numpy(w.logits).to(dev)
            masks = None if w.masks is None else torch.from_numpy(w.masks.view(np.int32)).to(dev)
            hist, hl = torch.from_numpy(w.history).to(dev), torch.from_numpy(w.history_len).to(dev)
            pd = params_to_device(w.params, dev)
            out1 = torch.empty(1, dtype=torch.int32, device=dev)
            for _ in range(10):
                s.sample_rows(lg, pd, out1, masks=masks, history=hist, history_len=hl)
            torch.cuda.synchronize()
            s.device_status()
            res[name] = int(out1.item())
            s.close()
        print(json.dumps({"note": "--only-batch1: a profiler run, not a benchmark line", "tokens": res}))
        return
    # ---- inputs: `batches` distinct 256-row batches per rank, resident in HBM --------------------------------
    host = [wl.session_batch(seed=1000 * rank + b, rows=rows) for b in range(args.batches)]
    vocab = host[0].vocab
    row_bytes = host[0].row_bytes() - (4 * host[0].masks.shape[1] if args.no_masks else 0)
    dev_in = []
    for w in host:
        dev_in.append(dict(
            logits=torch.from_numpy(w.logits).to(dev), masks=torch.from_numpy(w.masks.view(np.int32)).to(dev),
            history=torch.from_numpy(w.history).to(dev), history_len=torch.from_numpy(w.history_len).to(dev),
            params=params_to_device(w.params, dev)))
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    sampler = Sampler(local, max_rows=rows, max_vocab=vocab, k_cap=64, max_history=host[0].history.shape[1])

    def step(i, masked=not args.no_masks):
        d = dev_in[i % len(dev_in)]
        sampler.sample_rows(d["logits"], d["params"], out, masks=d["masks"] if masked else None, history=d["history"],
                            history_len=d["history_len"])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_region(fn, steps):
        """Exactly `steps` calls of fn(i), device time, bracketed by barrier + synchronise, max over ranks."""
        for i in range(3):  # re-warm right before the clock starts: nothing idles between warm-up and the region
            fn(i)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for i in range(steps):
            fn(i)
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(W):
        step(i)
    barrier()
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    # ---- timed regions: exactly K steps each, repeated; the median region is the value ----------------------
    launches0 = sampler.launch_count()
    regions = [timed_region(step, K) for _ in range(args.repeats)]
    launches = (sampler.launch_count() - launches0) * K // (args.repeats * (K + 3))
    total_ms = float(np.median(regions))
    if args.only_headline:  # profiler runs: the timed regions and nothing else
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": world * rows * K / (total_ms / 1e3), "unit": "rows/s",
                              "ms_per_step": total_ms / K, "config": {"workload": WORKLOAD + ("_all_ids_allowed" if args.no_masks else "")},
                              "note": "--only-headline: a profiler run, not a benchmark line"}))
        if world > 1:
            dist.destroy_process_group()
        return
    # a longer untimed stretch of the same steps so that the clock record has samples under load
    if rank == 0:
        t_end = time.time() + 1.0
        i = 0
        while time.time() < t_end:
            step(i)
            i += 1
            if i % 64 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
    clock_info = clocks.stop() if rank == 0 else None
    sampler.device_status()

    # ---- the dominant kernel: its launch duration is the timed region's device time per launch (the region holds
    # nothing but K back-to-back k_select launches, counted below); event pairs around every single launch, which put
    # gaps between the launches, are reported beside it
    peak, peak_kind = measured_peaks()
    sel_avg_s = total_ms / max(launches, 1) / 1e3
    achieved = rows * row_bytes / sel_avg_s / 1e9 if sel_avg_s > 0 else 0.0
    sampler.profile_begin(K)
    for i in range(K):
        step(i)
    sel_ms, fin_ms, calls = sampler.profile_end()
    isolated_us = sel_ms / max(calls, 1) * 1e3
    # the same rows with every id allowed: no vector can be skipped, so every logit byte comes from HBM
    dense_regions = [timed_region(lambda i: step(i, masked=False), K) for _ in range(max(3, args.repeats // 3))]
    dense_s = float(np.median(dense_regions)) / K / 1e3
    dense_bytes = rows * (host[0].row_bytes() - 4 * host[0].masks.shape[1])
    # the same densities with the allowed ids scattered instead of in 20 runs: nearly every 16-byte vector holds one
    scat = []
    for b, w in enumerate(host):
        g = wl.rng(77 + b)
        m = np.stack([wl.random_mask(g, vocab, float(f)) for f in w.meta["allowed_fraction"]])
        scat.append(torch.from_numpy(m.view(np.int32)).to(dev))

    def step_scattered(i):
        d = dev_in[i % len(dev_in)]
        sampler.sample_rows(d["logits"], d["params"], out, masks=scat[i % len(scat)], history=d["history"], history_len=d["history_len"])

    scat_s = float(np.median([timed_region(step_scattered, K) for _ in range(3)])) / K / 1e3
    del scat
    # strong scaling of the same fixed batch: 256 rows in all, rows / world per rank
    strong = None
    if world > 1:
        share = max(1, rows // world)
        lo = (rank * share) % rows

        def step_strong(i):
            d = dev_in[i % len(dev_in)]
            sampler.sample_rows(d["logits"][lo:lo + share], d["params"][lo * 48:(lo + share) * 48], out[:share],
                                masks=d["masks"][lo:lo + share], history=d["history"][lo:lo + share],
                                history_len=d["history_len"][lo:lo + share])

        strong_ms = float(np.median([timed_region(step_strong, K) for _ in range(3)]))
        strong = {"rows_total": share * world, "rows_per_gpu": share, "ms_per_step": strong_ms / K,
                  "rows_per_s": share * world * K / (strong_ms / 1e3),
                  "note": "the fixed 256-row batch split over the GPUs (strong scaling) next to the weak figure above"}

    # ---- end to end through the engine glue: host buffers in, tokens out to the host, every step -----------
    eng = Engine(local, max_rows=rows, vocab=vocab, k_cap=64, max_history=host[0].history.shape[1])
    host_pin = [dict(logits=pinned(w.logits), masks=pinned(w.masks.view(np.int32)), history=pinned(w.history),
                     history_len=pinned(w.history_len), params=pinned(w.params.view(np.uint8))) for w in host[:2]]

    def e2e(steps, logits_on_host, history_on_device=False, cached_masks=False):
        """Steps through the engine glue with host inputs: step i + 1 is queued (pick_async) before the host waits for
        step i (pick_wait), as the reference chains its decode (src/engine.cu:796-852); two slots alternate."""
        def queue(i):
            h, d = host_pin[i % 2], dev_in[i % 2]
            if cached_masks:
                eng.pick_async_dl(d["logits"], h["params"], masks=h["masks"], mask_states=states[i % 2])
            else:
                eng.pick_async(h["logits"] if logits_on_host else d["logits"], h["params"], masks_host=h["masks"],
                               history_host=None if history_on_device else h["history"],
                               history_len_host=None if history_on_device else h["history_len"],
                               logits_on_host=logits_on_host, host_stable=True)
        for warm in range(2):
            queue(warm)
            eng.pick_wait(rows)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        queue(0)
        for i in range(steps):
            if i + 1 < steps:
                queue(i + 1)
            eng.pick_wait(rows)
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return world * rows * steps / (float(t.item()) / 1e3)

    side_bytes = rows * (host[0].masks.shape[1] * 4 + host[0].history.shape[1] * 4 + 4 + 48)
    # logits that cross PCIe when the kernel reads them from page-locked host memory: the 16-byte vectors (4 ids =
    # one nibble of a mask word) with at least one allowed id, averaged over the two batches the e2e leg alternates
    nib = [np.unpackbits(w.masks.view(np.uint8), bitorder="little").reshape(-1, 4).any(axis=1).sum() for w in host[:2]]
    crossing = int(np.mean(nib)) * 16
    e2e_steps = max(3, min(K, 20))
    e2e_host = e2e(e2e_steps, True)
    e2e_engine = e2e(max(3, min(K, 100)), False)
    # the sessions' histories kept on the device (fns_b200_engine_append), masks from the host: what a decode step uploads
    for b in range(1):
        hd = dev_in[0]["history"]
        eng.reset()
        for c in range(0, hd.shape[1], 64):  # the committed tokens so far, 64 columns at a time
            cols = hd[:, c:c + 64].contiguous()
            counts = np.full(rows, cols.shape[1], np.int32)
            eng.append(cols.data_ptr(), cols.shape[1], rows, counts_host=counts)
        torch.cuda.synchronize()
    e2e_engine_dev_hist = e2e(max(3, min(K, 100)), False, history_on_device=True)
    # ... and the masks kept on the device by grammar state: a state seen before uploads nothing
    eng.mask_cache(2 * rows)
    states = [np.arange(rows, dtype=np.uint64) + np.uint64(1000 * b) for b in range(2)]
    e2e_engine_cached = e2e(max(3, min(K, 100)), False, history_on_device=True, cached_masks=True)
    hits, misses, up_bytes = eng.mask_stats()

    result = {
        "metric": METRIC, "value": world * rows * K / (total_ms / 1e3), "unit": "rows/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD + ("_all_ids_allowed" if args.no_masks else ""), "rows_per_gpu": rows, "vocab": vocab, "k_cap": 64,
                   "history_ids": int(host[0].history.shape[1]), "batches_rotated": len(dev_in),
                   "l2": f"{len(dev_in)} distinct batches of {rows * row_bytes / 1e6:.0f} MB rotate; each exceeds the 126 MB L2",
                   "parallelism": f"rows{world}"},
        "us_per_row": total_ms * 1e3 / (K * rows),
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "k_select", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "frac_of_8TBps_nominal": achieved / 8000.0,
                     "bytes_per_launch": rows * row_bytes, "avg_launch_us": sel_avg_s * 1e6,
                     "isolated_launch_us": isolated_us,
                     "traffic": args.traffic if args.traffic is not None else
                     (NCU_TRAFFIC_BYTES if rows == 256 and not args.no_masks else None),
                     "traffic_note": "ncu dram bytes per launch of the capture summarised under profiles/; below the "
                                     "algorithmic bytes because vectors with no allowed id are never loaded",
                     "bound_note": "frac is algorithmic (dense) bytes over time, as the metric is defined; with this "
                                   "workload's run-structured masks the kernel moves only `traffic` bytes and is "
                                   "latency-bound, not HBM-bound: the HBM-bound figure is all_ids_allowed",
                     "frac_of_traffic": (NCU_TRAFFIC_BYTES / sel_avg_s / 1e9 / peak) if rows == 256 and not args.no_masks else None,
                     "all_ids_allowed": {"kernel": "k_ring", "avg_launch_us": dense_s * 1e6, "bytes_per_launch": dense_bytes,
                                         "achieved": dense_bytes / dense_s / 1e9 if dense_s > 0 else 0.0,
                                         "frac": dense_bytes / dense_s / 1e9 / peak if dense_s > 0 else 0.0,
                                         "traffic": NCU_TRAFFIC_BYTES_DENSE if rows == 256 else None},
                     "scattered_masks": {"avg_launch_us": scat_s * 1e6, "bytes_per_launch": rows * row_bytes,
                                         "achieved": rows * row_bytes / scat_s / 1e9, "frac": rows * row_bytes / scat_s / 1e9 / peak,
                                         "note": "the same per-row densities with random bits instead of 20 runs"}},
        "value_stats": {"regions": len(regions), "ms_per_step_min": min(regions) / K, "ms_per_step_median": total_ms / K,
                        "ms_per_step_max": max(regions) / K},
        "strong256": strong,
        "e2e": {"value": e2e_host, "unit": "rows/s", "h2d_bytes_per_step": int(crossing + side_bytes),
                "d2h_bytes_per_step": rows * 4, "steps": e2e_steps,
                "host_input_bytes_per_step": int(rows * vocab * 4 + side_bytes),
                "note": "engine pick (pick_async + pick_wait), every input in pinned host memory every step, tokens "
                        "read back to the host: masks, histories and parameters are copied by DMA, the logits are "
                        "read over PCIe by the kernel itself, which loads only the 16-byte vectors holding an "
                        "allowed id (h2d_bytes_per_step counts those; host_input_bytes_per_step is the full size)"},
        "e2e_engine": {"value": e2e_engine, "unit": "rows/s", "h2d_bytes_per_step": int(side_bytes),
                       "d2h_bytes_per_step": rows * 4,
                       "note": "as the reference's Engine::pick_async is used: logits already on the GPU (the LM "
                               "head wrote them), masks / histories / parameters from host memory, tokens back",
                       "device_histories": {"value": e2e_engine_dev_hist, "unit": "rows/s",
                                            "h2d_bytes_per_step": int(rows * (host[0].masks.shape[1] * 4 + 48)),
                                            "note": "session histories kept on the device (fns_b200_engine_append): a step "
                                                    "uploads masks and parameters only"},
                       "device_histories_cached_masks": {
                           "value": e2e_engine_cached, "unit": "rows/s", "h2d_bytes_per_step": int(rows * (48 + 4)),
                           "mask_cache": {"hits": hits, "misses": misses, "bytes_uploaded_in_all": up_bytes},
                           "note": "masks through fns_b200_engine_pick_async_dl with grammar-state ids: every state was "
                                   "seen in the warm-up, so a step uploads parameters and 4-byte slot numbers only"}},
    }
    if rank == 0:
        result["clocks"] = clock_info
    if rank == 0 and not args.skip_extras:
        result["batch1"] = batch1_latency(torch, dev, local)
        result["config5_one_gpu"] = config5_one_gpu(torch, dev, local)
    if rank == 0 and world == 1 and not args.skip_extras:
        result["cpu_baseline"] = cpu_baseline(host[0], budget_s=args.cpu_seconds)
        result["reference_gpu_kernels"] = reference_gpu(torch, dev, host[0], dev_in[0])
    if world > 1 and not args.skip_extras:
        vs = vocab_sharded(torch, dist, dev, local, rank, world)
        if rank == 0:
            result["vocab_sharded"] = vs
    if rank == 0:
        line = json.dumps(result)
        if json_fd is None:
            print(line)
        else:
            sys.stdout.flush()
            os.write(json_fd, (line + "\n").encode())
    if world > 1:
        dist.destroy_process_group()


def batch1_latency(torch, dev, local):
    """Device time per row at batch 1: a CUDA graph of 50 back-to-back calls replayed 40 times (no host launch
    gaps), and plain stream launches for comparison."""
    from flintnsteel_b200 import workloads as wl
    from flintnsteel_b200.sampler import Sampler, params_to_device

    res = {}
    cases = {"single_row_T0.7_k40_p0.95_rep1.1_h512": wl.single_row(), "single_row_greedy": wl.single_row(greedy=True),
             "grammar_row_mask1.5pct_h4096_allpen_k20": wl.grammar_row()}
    for name, w in cases.items():
        s = Sampler(local, max_rows=1, max_vocab=w.vocab, k_cap=64, max_history=4096)
        lg = torch.from_numpy(w.logits).to(dev)
        masks = None if w.masks is None else torch.from_numpy(w.masks.view(np.int32)).to(dev)
        hist, hl = torch.from_numpy(w.history).to(dev), torch.from_numpy(w.history_len).to(dev)
        pd = params_to_device(w.params, dev)
        out = torch.empty(1, dtype=torch.int32, device=dev)

        def call():
            s.sample_rows(lg, pd, out, masks=masks, history=hist, history_len=hl)

        for _ in range(5):
            call()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            call()
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(50):
                    call()
        torch.cuda.synchronize()
        for _ in range(3):
            graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(40):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        graph_us = a.elapsed_time(b) * 1e3 / (40 * 50)
        a.record()
        for _ in range(200):
            call()
        b.record()
        torch.cuda.synchronize()
        res[name] = {"us_per_row_graph": graph_us, "us_per_row_stream": a.elapsed_time(b) * 1e3 / 200,
                     "bytes_per_row": w.row_bytes(), "plan": s.plan(0, w.vocab, 1, w.history.shape[1])}
        s.close()
    # a small batch: 8 sessions of the headline workload (masks, 2,048-id histories, all penalties) in one call
    w = wl.session_batch(seed=77, rows=8)
    s = Sampler(local, max_rows=8, max_vocab=w.vocab, k_cap=64, max_history=w.history.shape[1])
    lg, mk = torch.from_numpy(w.logits).to(dev), torch.from_numpy(w.masks.view(np.int32)).to(dev)
    hist, hl = torch.from_numpy(w.history).to(dev), torch.from_numpy(w.history_len).to(dev)
    pd = params_to_device(w.params, dev)
    out8 = torch.empty(8, dtype=torch.int32, device=dev)
    for _ in range(5):
        s.sample_rows(lg, pd, out8, masks=mk, history=hist, history_len=hl)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(50):
                s.sample_rows(lg, pd, out8, masks=mk, history=hist, history_len=hl)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(40):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    res["sessions8_masked_penalised"] = {"us_per_call_graph": a.elapsed_time(b) * 1e3 / (40 * 50), "rows": 8,
                                         "plan": s.plan(0, w.vocab, 8, w.history.shape[1])}
    s.close()
    # one session through the engine glue, as the reference's decode loop uses Engine::pick: logits on the GPU, the
    # grammar mask from host memory, the history on the device, the token back on the host - wall clock per token
    import time

    from flintnsteel_b200.sampler import Engine
    w = wl.grammar_row()
    eng = Engine(local, max_rows=1, vocab=w.vocab, k_cap=64, max_history=4096)
    lg = torch.from_numpy(w.logits).to(dev)
    pr = w.params.copy()

    def token_step(i):
        pr["counter"] = i
        eng.pick_async(lg, pr, masks_host=w.masks)
        eng.append(eng.device_tokens_ptr(), 1, 1)
        return eng.pick_wait(1)

    for i in range(200):
        token_step(i)
    eng.reset()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(2000):
        token_step(i)
    res["engine_one_session_step"] = {"us_per_token_wall": (time.perf_counter() - t0) / 2000 * 1e6,
                                      "note": "pick_async + append + pick_wait from this Python process (three ctypes "
                                              "calls per token); the kernel's share is the grammar row's figure above"}
    eng.close()
    # config 3: one verification window (3 draft positions + bonus = 4 rows), greedy, accept length on the device
    sw = wl.spec_windows(seed=1, windows=1, n_draft=3)
    s = Sampler(local, max_rows=4, max_vocab=sw.vocab, k_cap=64, max_history=0)
    lg, dr = torch.from_numpy(sw.logits).to(dev), torch.from_numpy(sw.draft).to(dev)
    pd = params_to_device(sw.params, dev)
    toks, acc = torch.empty(4, dtype=torch.int32, device=dev), torch.empty(1, dtype=torch.int32, device=dev)
    for _ in range(5):
        s.verify_accept(lg, dr, pd, toks, acc)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(50):
                s.verify_accept(lg, dr, pd, toks, acc)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(40):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    res["verify_window_4rows_greedy"] = {"us_per_window_graph": a.elapsed_time(b) * 1e3 / (40 * 50), "rows": 4,
                                         "bytes_per_window": 4 * sw.vocab * 4 + 12 + 20,
                                         "note": "select + draw kernel and the accept kernel per window"}
    s.close()
    return res


def config5_one_gpu(torch, dev, local):
    """64 rows x V = 262,144 bf16, 50 % random mask, top-k 1024 / top-p / min-p on ONE GPU (no exchange)."""
    from flintnsteel_b200 import workloads as wl
    from flintnsteel_b200.sampler import Sampler, params_to_device

    w = wl.large_vocab(seed=0, rows=64)
    s = Sampler(local, max_rows=64, max_vocab=w.vocab, k_cap=1024, max_history=0)
    lg = torch.from_numpy(w.logits.view(np.int16)).to(dev).view(torch.bfloat16)
    m = torch.from_numpy(w.masks.view(np.int32)).to(dev)
    pd = params_to_device(w.params, dev)
    out = torch.empty(64, dtype=torch.int32, device=dev)
    for _ in range(5):
        s.sample_rows(lg, pd, out, masks=m)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(50):
        s.sample_rows(lg, pd, out, masks=m)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1e3 / 50
    s.close()
    return {"us_per_call": us, "rows": 64, "vocab": w.vocab, "k": 1024, "bytes_per_call": 64 * w.row_bytes(),
            "achieved_GBps": 64 * w.row_bytes() / us / 1e3}


def host_threads() -> int:
    """Every core this process may run on (launchers such as torchrun set OMP_NUM_THREADS=1, which is not that)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_baseline(w, budget_s: float):
    """The CPU oracle (a port of the reference's sampler, not the product) on this host's cores, same rows."""
    from oracle.binding import Oracle

    o = Oracle()
    cores = host_threads()
    x = w.logits
    t0, done, threads = time.time(), 0, 1
    n = min(32, w.rows)
    while time.time() - t0 < budget_s:
        lo = done % w.rows
        hi = min(w.rows, lo + n)
        _, threads = o.sample_rows(x[lo:hi], w.params[lo:hi], 64, w.masks[lo:hi], w.history[lo:hi], w.history_len[lo:hi],
                                   threads=cores)
        done += hi - lo
    dt = time.time() - t0
    return {"value": done / dt, "unit": "rows/s", "cores": threads, "kind": "port",
            "sample": f"{done} rows of the same batch in {dt:.1f} s, OpenMP over rows"}


def reference_gpu(torch, dev, w, d):
    """The reference's own CUDA sampler (src/kernels.cu, unmodified, built for sm_100a) on this GPU: one row per
    call, two launches per row.  It has no repetition / frequency terms, so it runs the same rows and masks
    without penalties: the same memory traffic and the same selection work."""
    try:
        from oracle.binding import RefGpu

        ref = RefGpu()
    except Exception as exc:  # the checker library is optional for the benchmark
        return {"unavailable": str(exc)}
    out = torch.empty(w.rows, dtype=torch.int32, device=dev)
    ref.sample_rows(d["logits"], d["masks"], w.params, out)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    ref.sample_rows(d["logits"], d["masks"], w.params, out)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    return {"value": w.rows / (ms / 1e3), "unit": "rows/s", "us_per_row": ms * 1e3 / w.rows,
            "note": "reference kernels recompiled for sm_100a, row by row on one stream (they are not re-entrant)"}


def vocab_sharded(torch, dist, dev, local, rank, world):
    """64 rows x V = 262,144 bf16 split evenly by vocabulary through the C++ dispatcher (fns_b200_mg_*): per-shard
    top-1024, one NCCL all-gather of (value, id) candidates, merge + draw on every rank.  The three steps are timed
    with CUDA events inside the library; rank 0's tokens are compared with the unsharded path on the same rows."""
    from flintnsteel_b200 import workloads as wl
    from flintnsteel_b200.dispatch import VocabSharded
    from flintnsteel_b200.sampler import Sampler, params_to_device

    w = wl.large_vocab(seed=0, rows=64)
    vs = VocabSharded(local, w.vocab, 1024, rank, world, max_rows=w.rows)
    lo, hi = vs.lo, vs.hi
    lg = torch.from_numpy(np.ascontiguousarray(w.logits[:, lo:hi]).view(np.int16)).to(dev).view(torch.bfloat16)
    masks = torch.from_numpy(np.ascontiguousarray(w.masks[:, lo // 32:(hi + 31) // 32]).view(np.int32)).to(dev)
    pd = params_to_device(w.params, dev)
    out = torch.empty(w.rows, dtype=torch.int32, device=dev)
    for _ in range(5):
        vs.sample(lg, pd, out, masks_shard=masks)
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = 50
    a.record()
    for _ in range(steps):
        vs.sample(lg, pd, out, masks_shard=masks)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    vs.profile_begin(steps)
    for _ in range(steps):
        vs.sample(lg, pd, out, masks_shard=masks)
    sel_us, exch_us, fin_us, _ = vs.profile_end()
    stage = torch.tensor([sel_us, exch_us, fin_us], dtype=torch.float64, device=dev)
    dist.all_reduce(stage, op=dist.ReduceOp.MAX)
    same = out.clone()
    dist.broadcast(same, 0)
    flag = torch.tensor([1 if torch.equal(same, out) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    matches = None
    if rank == 0:  # the whole rows on one GPU, no exchange: a product-vs-product check that can fail
        s = Sampler(local, max_rows=w.rows, max_vocab=w.vocab, k_cap=1024, max_history=0)
        full = torch.from_numpy(w.logits.view(np.int16)).to(dev).view(torch.bfloat16)
        fm = torch.from_numpy(w.masks.view(np.int32)).to(dev)
        direct = torch.empty(w.rows, dtype=torch.int32, device=dev)
        s.sample_rows(full, pd, direct, masks=fm)
        torch.cuda.synchronize()
        matches = bool(torch.equal(direct, out))
        s.close()
    vs.close()
    ms = float(t.item()) / steps
    return {"rows_per_s": w.rows / (ms / 1e3), "ms_per_step": ms, "rows": w.rows, "vocab": w.vocab, "k": 1024,
            "allgather_bytes_per_rank": w.rows * 1024 * 8, "all_ranks_agree": bool(flag.item()),
            "matches_unsharded": matches, "select_us": float(stage[0]), "allgather_us": float(stage[1]),
            "finalize_us": float(stage[2]), "stage_note": "CUDA events inside the library, max over ranks",
            "scaling": "strong (the vocabulary is split)"}


def run_reference(args):
    """CPU arm: the oracle port with every host thread, on bounded samples of the same workload."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from flintnsteel_b200 import workloads as wl
    from oracle.binding import Oracle

    o = Oracle()
    sample_rows = args.rows  # the same 256-row steps as the GPU arm
    w = wl.session_batch(seed=0, rows=sample_rows)
    threads, cores = 1, host_threads()
    for _ in range(max(args.warmup, 1)):
        _, threads = o.sample_rows(w.logits[:16], w.params[:16], 64, w.masks[:16], w.history[:16], w.history_len[:16],
                                   threads=cores)
    K = min(args.steps, 40)
    t0 = time.time()
    for _ in range(K):
        o.sample_rows(w.logits, w.params, 64, w.masks, w.history, w.history_len, threads=cores)
    dt = time.time() - t0
    value = sample_rows * K / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": K,
        "warmup": max(args.warmup, 1), "ms_per_step": dt / K * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_step": sample_rows, "vocab": w.vocab, "k_cap": 64,
                   "history_ids": int(w.history.shape[1]),
                   "rows_per_gpu": sample_rows, "batches_rotated": 1, "parallelism": f"rows{world}",
                   "note": "the reference's sampler is CUDA code; its CPU form is the restatement in oracle/fns_oracle.c"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port",
                         "sample": f"{K} steps of {sample_rows} rows, OpenMP over rows"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    try:
        import torch

        if torch.cuda.is_available():
            from flintnsteel_b200.sampler import params_to_device  # noqa: F401  (torch plumbing only)

            dev = torch.device("cuda:0")
            d = {"logits": torch.from_numpy(w.logits).to(dev), "masks": torch.from_numpy(w.masks.view(np.int32)).to(dev)}
            line["reference_gpu_kernels"] = reference_gpu(torch, dev, w, d)
    except Exception as exc:
        line["reference_gpu_kernels"] = {"unavailable": str(exc)}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--batches", type=int, default=4)
    ap.add_argument("--repeats", type=int, default=30, help="timed regions of K steps each; the median is the value")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--skip-extras", action="store_true", help="no batch-1 / CPU / reference-kernel legs")
    ap.add_argument("--only-headline", action="store_true", help="the timed regions only (for profiler runs)")
    ap.add_argument("--only-batch1", action="store_true", help="ten launches of each one-row case only (for profiler runs)")
    ap.add_argument("--no-masks", action="store_true", help="every id allowed: the HBM-bound variant of the workload")
    ap.add_argument("--traffic", type=float, default=None,
                    help="dram bytes per select launch from an ncu capture (see profiles/), echoed into the line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
