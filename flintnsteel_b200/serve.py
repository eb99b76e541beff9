"""A sampler-only JSON-lines service: one request per line on stdin, one answer per line on stdout.

The shape of the reference's native driver (NomenAK/FlintNSteel tools/fns_serve/fns_serve.cpp:291-303, 523-538) cut
down to the sampler: the request carries the sampling fields of fns-serve - "temperature", "top_p", "top_k", "seed",
"presence_penalty", with the defaults the reference uses (greedy, 1, 0 = k_cap, 0, 0) - plus the logits to sample
from, since no model runs here:

    {"id": 7, "logits_npy": "/path/row.npy", "temperature": 1.0, "top_p": 0.95, "top_k": 20, "seed": 0,
     "allowed": [1, 5, 9], "history": [5, 5, 2], "draw": 3}

"logits" (a list) or "logits_npy" (a .npy file of one row or [rows][vocab]); "allowed": ids the grammar allows
(absent = all); "history": ids already generated (penalties); "draw": the index of the generated token = the Philox
counter (fns_serve.cpp:326-328).  The answer is {"id": 7, "tokens": [t, ...]}; a failure is {"error": "..."} and the
service keeps running, as fns-serve does (fns_serve.cpp:533-538).  The request fields are parsed by the library
(fns_b200_params_from_json), so this front end and a C++ one read a request the same way.

    python -m flintnsteel_b200.serve [--device 0] [--k-cap 64]
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

from .sampler import Sampler, params_from_json, params_to_device


def answer(line: str, samplers: dict, device: int, k_cap: int) -> dict:
    import torch

    req = json.loads(line)
    if not isinstance(req, dict):
        raise ValueError("a request is a JSON object")
    if "logits_npy" in req:
        x = np.load(req["logits_npy"])
    elif "logits" in req:
        x = np.asarray(req["logits"], dtype=np.float32)
    else:
        raise ValueError("no logits: give \"logits\" or \"logits_npy\"")
    x = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
    rows, vocab = x.shape
    p = np.repeat(params_from_json(line), rows)
    p["counter"] = np.uint64(int(req.get("draw", 0))) + np.arange(rows, dtype=np.uint64)
    dev = torch.device(f"cuda:{device}")
    hist = np.asarray(req.get("history", []), dtype=np.int32).reshape(-1)
    key = (vocab, max(rows, 1), max(hist.size, 1))
    s = samplers.get(key)
    if s is None:
        s = samplers[key] = Sampler(device, max_rows=rows, max_vocab=vocab, k_cap=k_cap, max_history=max(hist.size, 1))
    masks = None
    if req.get("allowed") is not None:
        ids = np.asarray(req["allowed"], dtype=np.int64).reshape(-1)
        if ids.size and (ids.min() < 0 or ids.max() >= vocab):
            raise ValueError("token outside the vocabulary")
        bits = np.zeros(((vocab + 31) // 32) * 32, dtype=bool)
        bits[ids] = True
        words = np.packbits(bits.reshape(-1, 32), axis=1, bitorder="little").view(np.uint32).reshape(1, -1)
        masks = torch.from_numpy(np.repeat(words, rows, axis=0).view(np.int32)).to(dev)
    h = hl = None
    if hist.size:
        h = torch.from_numpy(np.repeat(hist[None, :], rows, axis=0)).to(dev)
        hl = torch.full((rows,), hist.size, dtype=torch.int32, device=dev)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    s.sample_rows(torch.from_numpy(x).to(dev), params_to_device(p, dev), out, masks=masks, history=h, history_len=hl)
    torch.cuda.synchronize()
    return {"id": req.get("id", -1), "tokens": out.cpu().tolist()}


def serve(stdin=sys.stdin, stdout=sys.stdout, device: int = 0, k_cap: int = 64) -> None:
    samplers: dict = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        try:
            reply = answer(line, samplers, device, k_cap)
        except Exception as exc:  # the service survives a bad request
            reply = {"error": str(exc).replace('"', "'")}
        stdout.write(json.dumps(reply) + "\n")
        stdout.flush()
    for s in samplers.values():
        s.close()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--k-cap", type=int, default=64)
    a = ap.parse_args()
    serve(device=a.device, k_cap=a.k_cap)
