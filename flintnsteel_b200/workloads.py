"""Seeded synthetic inputs for the five sampler configurations that the benchmark and the parity tests use.

No dataset is involved: logits are drawn from the stated distributions with numpy's Philox bit generator, so
the same (config, seed) gives the same bytes on every machine.  All arrays are host numpy arrays.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .sampler import PARAMS_DTYPE, make_params

V_QWEN = 151_936
V_LARGE = 262_144


@dataclass
class Workload:
    name: str
    logits: np.ndarray                 # (rows, V) float32, or uint16 holding bf16 bits
    params: np.ndarray                 # (rows,) PARAMS_DTYPE  (per window for a verification workload)
    masks: np.ndarray | None = None    # (rows, ceil(V / 32)) uint32, bit (i & 31) of word (i >> 5); 1 = allowed
    history: np.ndarray | None = None  # (rows, H) int32
    history_len: np.ndarray | None = None
    draft: np.ndarray | None = None    # (windows, n_draft) int32
    bf16: bool = False
    k_cap: int = 64
    meta: dict = field(default_factory=dict)

    @property
    def rows(self) -> int:
        return self.logits.shape[0]

    @property
    def vocab(self) -> int:
        return self.logits.shape[1]

    def logits_f32(self) -> np.ndarray:
        return bf16_bits_to_f32(self.logits) if self.bf16 else self.logits

    def row_bytes(self) -> int:
        """Algorithmic bytes per row: logits + mask words + history ids + the token written."""
        b = self.vocab * (2 if self.bf16 else 4) + 4
        if self.masks is not None:
            b += 4 * self.masks.shape[1]
        if self.history is not None:
            b += 4 * self.history.shape[1]
        return b


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16, returned as uint16 bit patterns."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def gaussian_logits(g: np.random.Generator, rows: int, vocab: int, sigma: float, spikes: int = 8,
                    spike: float = 10.0) -> np.ndarray:
    x = g.standard_normal((rows, vocab), dtype=np.float32) * np.float32(sigma)
    for r in range(rows):
        ids = g.choice(vocab, size=spikes, replace=False)
        x[r, ids] += np.float32(spike)
    return x


def run_mask(g: np.random.Generator, vocab: int, fraction: float, runs: int = 20) -> np.ndarray:
    """Bitmask allowing about ``fraction`` of the vocabulary as ``runs`` random contiguous runs."""
    words = (vocab + 31) // 32
    if fraction >= 0.999:
        bits = np.ones(vocab, dtype=bool)
    else:
        bits = np.zeros(vocab, dtype=bool)
        total = max(1, int(round(fraction * vocab)))
        cuts = np.sort(g.integers(0, total + 1, size=runs - 1))
        lens = np.diff(np.concatenate(([0], cuts, [total])))
        for n in lens:
            if n <= 0:
                continue
            start = int(g.integers(0, vocab - n + 1))
            bits[start:start + n] = True
    padded = np.zeros(words * 32, dtype=bool)
    padded[:vocab] = bits
    return np.packbits(padded.reshape(words, 32), axis=1, bitorder="little").view(np.uint32).reshape(words)


def random_mask(g: np.random.Generator, vocab: int, density: float) -> np.ndarray:
    words = (vocab + 31) // 32
    padded = np.zeros(words * 32, dtype=bool)
    padded[:vocab] = g.random(vocab) < density
    return np.packbits(padded.reshape(words, 32), axis=1, bitorder="little").view(np.uint32).reshape(words)


def mask_allows(mask: np.ndarray, ids: np.ndarray) -> np.ndarray:
    return ((mask[ids >> 5] >> (ids & 31).astype(np.uint32)) & 1).astype(bool)


def single_row(seed: int = 0, vocab: int = V_QWEN, greedy: bool = False) -> Workload:
    """Config 1: one row, repetition 1.1 over 512 history ids, T 0.7, top-k 40, top-p 0.95, Philox seed 0."""
    g = rng(seed)
    x = gaussian_logits(g, 1, vocab, 2.5)
    hist = g.integers(0, vocab, size=(1, 512), dtype=np.int32)
    p = make_params(1, temperature=0.0 if greedy else 0.7, top_k=40, top_p=0.95, repetition=1.1, seed=0, counter=0)
    return Workload("single_row", x, p, None, hist, np.array([512], np.int32), meta={"seed": seed})


def grammar_row(seed: int = 0, vocab: int = V_QWEN) -> Workload:
    """Config 2: the same logits under a 1.5 % bitmask of 20 runs; 4096-id history with all three penalties."""
    g = rng(seed)
    x = gaussian_logits(g, 1, vocab, 2.5)
    g2 = rng(seed + 1_000_003)
    mask = run_mask(g2, vocab, 0.015, 20)[None, :]
    hist = g2.integers(0, vocab, size=(1, 4096), dtype=np.int32)
    p = make_params(1, temperature=0.6, top_k=20, top_p=0.9, min_p=0.05, repetition=1.1, presence=0.5,
                    frequency=0.3, seed=0, counter=0)
    return Workload("grammar_row", x, p, mask, hist, np.array([4096], np.int32), meta={"seed": seed})


def spec_windows(seed: int = 0, windows: int = 1, n_draft: int = 3, vocab: int = V_QWEN,
                 p_match: float = 0.7, temperature: float = 0.0) -> Workload:
    """Config 3: windows of n_draft + 1 rows; each draft id is the row's argmax with probability 0.7, else
    uniform-random."""
    g = rng(seed)
    rows = windows * (n_draft + 1)
    x = gaussian_logits(g, rows, vocab, 2.5)
    arg = x.reshape(windows, n_draft + 1, vocab)[:, :n_draft].argmax(axis=2).astype(np.int32)
    rnd = g.integers(0, vocab, size=(windows, n_draft), dtype=np.int32)
    draft = np.where(g.random((windows, n_draft)) < p_match, arg, rnd).astype(np.int32)
    p = make_params(windows, temperature=temperature, top_k=40, top_p=0.95, seed=seed, counter=0)
    p["counter"] = np.arange(windows, dtype=np.uint64) * np.uint64(n_draft + 1)
    return Workload("spec_windows", x, p, draft=draft, meta={"seed": seed, "n_draft": n_draft})


def session_batch(seed: int = 0, rows: int = 256, vocab: int = V_QWEN, history: int = 2048,
                  k_values=(0, 20, 40, 100)) -> Workload:
    """Config 4: independent sessions.  T ~ U[0.3, 1.2], top_k in {0, 20, 40, 100}, top_p ~ U[0.8, 1], mask
    allowed fraction log-uniform in [0.1 %, 100 %] as 20 runs, 2048-id histories, repetition 1.1 / presence
    0.5 / frequency 0.3."""
    g = rng(seed)
    x = gaussian_logits(g, rows, vocab, 2.5)
    g2 = rng(seed + 2_000_003)
    frac = np.exp(g2.uniform(np.log(1e-3), np.log(1.0), size=rows))
    masks = np.stack([run_mask(g2, vocab, float(f), 20) for f in frac])
    hist = g2.integers(0, vocab, size=(rows, history), dtype=np.int32)
    p = make_params(rows, repetition=1.1, presence=0.5, frequency=0.3)
    p["temperature"] = g2.uniform(0.3, 1.2, size=rows).astype(np.float32)
    p["top_k"] = g2.choice(np.array(k_values, dtype=np.int32), size=rows)
    p["top_p"] = g2.uniform(0.8, 1.0, size=rows).astype(np.float32)
    p["seed"] = np.arange(rows, dtype=np.uint64) + np.uint64(seed)
    p["counter"] = g2.integers(0, 4096, size=rows).astype(np.uint64)
    return Workload("session_batch", x, p, masks, hist, np.full(rows, history, np.int32),
                    meta={"seed": seed, "allowed_fraction": frac})


def large_vocab(seed: int = 0, rows: int = 64, vocab: int = V_LARGE) -> Workload:
    """Config 5: bf16 logits N(0, 3^2) + Zipf(1.1) bias (the log of an unnormalised Zipf law over the ids:
    -1.1 * ln(id + 1)), top-k 1024, top-p 0.9, min-p 0.02, 50 % random bitmask."""
    g = rng(seed)
    x = g.standard_normal((rows, vocab), dtype=np.float32) * np.float32(3.0)
    x += (-1.1 * np.log(np.arange(1, vocab + 1, dtype=np.float64))).astype(np.float32)[None, :]
    bits = f32_to_bf16_bits(x)
    g2 = rng(seed + 3_000_003)
    masks = np.stack([random_mask(g2, vocab, 0.5) for _ in range(rows)])
    p = make_params(rows, temperature=1.0, top_k=1024, top_p=0.9, min_p=0.02)
    p["seed"] = np.arange(rows, dtype=np.uint64) + np.uint64(seed)
    return Workload("large_vocab", bits, p, masks, bf16=True, k_cap=1024, meta={"seed": seed})


def lcg_logits(n: int = 150_144):
    """The inputs of the reference's own sampler test (tests/sample_check.cu:79-88): logits from a 32-bit linear
    congruential generator seeded with 7, thirty spiked ids at (j * 4999) % n with value 8 - 0.25 j, and a mask
    that allows every other spike.  Returns (logits, mask, spike_ids)."""
    rr = 7
    out = np.empty(n, dtype=np.int64)
    for i in range(n):
        rr = (rr * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = rr
    x = ((out >> 9) - (1 << 22)).astype(np.float32) / np.float32(1 << 22) * np.float32(3.0)
    spikes = np.array([(j * 4999) % n for j in range(30)], dtype=np.int64)
    for j, s in enumerate(spikes):
        x[s] = np.float32(8.0 - 0.25 * j)
    mask = np.zeros((n + 31) // 32, dtype=np.uint32)
    for j in range(0, 30, 2):
        s = int(spikes[j])
        mask[s >> 5] |= np.uint32(1 << (s & 31))
    return x, mask, spikes
