"""Multi-GPU dispatcher: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-GPU, one row per call (its docs/ENGINE.md:132); this layer is new.  Two partitions:

* ``RowSharded``   - independent sessions.  Rows [lo, hi) of the batch live on this rank; every rank samples its
                     own rows with its own workspace and stream.  No collective on the data path (tokens can be
                     gathered afterwards: 4 bytes per row).
* ``VocabSharded`` - one very large vocabulary split evenly over the ranks.  Each rank selects the top-k_cap
                     (value, id) candidates of its shard of every row, the lists are exchanged with ONE
                     all-gather (k_cap * 8 bytes per row per rank) into local memory, and every rank runs the
                     same merge + draw on the gathered lists, so all ranks hold the same tokens without a
                     broadcast.  Exact for the same reason the reference's 128 slices are
                     (src/kernels.cu:594-597): the global top-k is contained in the union of the shards' top-k,
                     and the merge orders by (value, id) alone, so the result does not depend on the number of
                     shards.

The kernels come from ``backend`` (a ``flintnsteel_b200.sampler.Sampler``); the dispatcher only allocates
tensors and calls the collective.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous near-even split: the first ``total % world`` ranks get one more."""
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def vocab_shard(vocab: int, rank: int, world: int) -> tuple[int, int]:
    """Even split whose boundaries fall on 32-id words, so that every shard owns whole bitmask words."""
    words = (vocab + 31) // 32
    wlo, whi = shard_range(words, rank, world)
    return wlo * 32, min(vocab, whi * 32)


class RowSharded:
    """Independent sessions: this rank owns rows ``shard_range(total_rows, rank, world)``."""

    def __init__(self, backend, rank: int = 0, world: int = 1, group=None):
        self.backend, self.rank, self.world, self.group = backend, rank, world, group

    def rows(self, total_rows: int) -> tuple[int, int]:
        return shard_range(total_rows, self.rank, self.world)

    def sample(self, logits, params, out, masks=None, history=None, history_len=None):
        """``logits`` etc. hold THIS rank's rows only (the LM head that produced them ran here)."""
        return self.backend.sample_rows(logits, params, out, masks=masks, history=history, history_len=history_len)

    def gather_tokens(self, local_tokens, total_rows: int):
        """Optional: every rank receives all tokens, in row order.  Shards of unequal size are padded to the
        largest for the collective (equal contributions on every backend) and trimmed afterwards."""
        if self.world == 1:
            return local_tokens
        sizes = [hi - lo for lo, hi in (shard_range(total_rows, r, self.world) for r in range(self.world))]
        width = max(sizes)
        padded = torch.full((width,), -1, dtype=local_tokens.dtype, device=local_tokens.device)
        padded[: local_tokens.numel()] = local_tokens
        out = torch.empty(self.world * width, dtype=local_tokens.dtype, device=local_tokens.device)
        dist.all_gather_into_tensor(out, padded, group=self.group)
        if all(n == width for n in sizes):
            return out
        return torch.cat([out[r * width: r * width + n] for r, n in enumerate(sizes)])


class VocabSharded:
    """One vocabulary over ``world`` ranks; this rank owns ids ``vocab_shard(vocab, rank, world)``."""

    def __init__(self, backend, vocab: int, k_cap: int, rank: int = 0, world: int = 1, group=None):
        self.backend, self.vocab, self.k_cap = backend, vocab, k_cap
        self.rank, self.world, self.group = rank, world, group
        self.lo, self.hi = vocab_shard(vocab, rank, world)
        self._local = None
        self._gathered = None

    def _buffers(self, rows: int, device):
        if self._local is None or self._local.shape[0] != rows or self._local.device != device:
            self._local = torch.empty((rows, self.k_cap, 2), dtype=torch.int32, device=device)
            self._gathered = torch.empty((self.world, rows, self.k_cap, 2), dtype=torch.int32, device=device)
        return self._local, self._gathered

    def sample(self, logits_shard, params, out, masks_shard=None, history=None, history_len=None):
        """``logits_shard``: [rows][hi - lo] of this rank's ids; ``masks_shard``: the matching words
        [rows][(hi - lo + 31) // 32]; ``history`` holds GLOBAL ids; ``out``: int32 [rows], the same on every rank."""
        rows = logits_shard.shape[0]
        local, gathered = self._buffers(rows, logits_shard.device)
        self.backend.select_rows(logits_shard, params, local, id_base=self.lo, masks=masks_shard, history=history,
                                 history_len=history_len, vocab=self.hi - self.lo)
        if self.world > 1:
            # the output is the ranks' [rows][k_cap] blocks one after the other (dim 0 concatenation)
            dist.all_gather_into_tensor(gathered.view(self.world * rows, self.k_cap, 2), local, group=self.group)
        else:
            gathered = local[None]
        # gathered is [world][rows][k_cap]: list l of row r starts at l * rows * k_cap + r * k_cap
        self.backend.finalize_rows(gathered, self.world, self.k_cap, rows, params, out_tokens=out,
                                   list_stride=rows * self.k_cap, row_stride=self.k_cap)
        return out
