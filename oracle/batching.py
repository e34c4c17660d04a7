"""Oracle restatement of the batch-shaping code that decides which (n, L)
shapes reach the kernels: length buckets, the token-budget micro-batch sampler
and the BOS/EOS padding collate.  Integer work: every output must be bit-exact.

Test infrastructure: see the package docstring.
"""
from __future__ import annotations

import bisect
import math
from typing import Iterator, List, Optional, Sequence

import numpy as np

BUCKET_STEP = 50  # train.py:2561


def build_bucket_boundaries(max_seq_len: int) -> List[int]:
    """train.py:2587-2593: multiples of 50 below ``max_seq_len`` then
    ``max_seq_len`` itself; a single bucket when max_seq_len < 50."""
    if max_seq_len < BUCKET_STEP:
        return [max_seq_len]
    return [*range(BUCKET_STEP, max_seq_len, BUCKET_STEP), max_seq_len]


def bucket_of(boundaries: Sequence[int], length: int) -> int:
    """train.py:1060-1076 (FastBucket.get_bucket): the smallest boundary that is
    >= length; lengths above the last boundary map to the last boundary."""
    bs = sorted(boundaries)
    i = bisect.bisect_left(bs, length)
    return bs[min(i, len(bs) - 1)]


def pick_micro_batch(bucket_len: int, target_tokens: int, max_micro_batch: int,
                     samples_per_step: int) -> int:
    """train.py:1770-1779 (_pick_bs): largest micro-batch within the token
    budget whose remainder against the step size is 0 or at least
    max(8, bs//3)."""
    bs = max(1, min(max_micro_batch, target_tokens // max(1, bucket_len)))
    while bs > 1:
        r = samples_per_step % bs
        if r == 0 or r >= max(8, bs // 3):
            return bs
        bs -= 1
    return bs


class BucketedCounts:
    """Minimal stand-in for what the sampler reads from FlatTokenDataset
    (train.py:1662-1688): per-bucket boundaries, sample counts, and the global
    id of each bucket's first sample."""

    def __init__(self, boundaries: Sequence[int], counts: Sequence[int]):
        self.boundaries = list(boundaries)
        self.counts = np.asarray(counts, dtype=np.int64)
        self.starts = np.concatenate(([0], np.cumsum(self.counts)[:-1])).astype(np.int64)
        self.total = int(self.counts.sum())


class TokenBudgetSampler:
    """train.py:1750-1858 (TokenBudgetBatchSampler).

    Per epoch: ``rng = default_rng(seed + epoch)``; one ``rng.permutation(count)``
    per non-empty bucket in boundary order; then, until the data runs out, draw
    a bucket with probability proportional to ``remaining / micro_batch`` by
    ``rng.random() * total`` against the cumulative weights
    (``searchsorted(..., side='right')``) and emit
    ``k = min(micro_batch, remaining, step budget left)`` ids from that bucket's
    permutation.  Each optimiser step consumes exactly ``samples_per_step``
    samples (the last step of an epoch may be short).
    """

    def __init__(self, data: BucketedCounts, samples_per_step: int = 64,
                 target_tokens: int = 12288, max_micro_batch: int = 64, seed: int = 42):
        self.data = data
        self.samples_per_step = int(samples_per_step)
        self.seed = seed
        self.epoch = 0
        self.skip_samples = 0
        self.micro_batch = {b: pick_micro_batch(int(b), target_tokens, max_micro_batch,
                                                samples_per_step)
                            for b in data.boundaries}

    def set_epoch(self, epoch: int, skip_samples: int = 0):
        self.epoch, self.skip_samples = epoch, int(skip_samples)

    def __len__(self):
        return int(math.ceil(self.data.total / self.samples_per_step))

    def __iter__(self) -> Iterator[List[int]]:
        it = self._stream()
        todo = self.skip_samples
        if todo > 0:  # train.py:1793-1808: resume must land on a micro-batch edge
            seen = 0
            for mb in it:
                seen += len(mb)
                if seen >= todo:
                    if seen != todo:
                        raise RuntimeError('resume position is not on a micro-batch boundary')
                    break
            if seen != todo:
                raise RuntimeError('dataset shorter than the resume position')
        yield from it

    def _stream(self):
        d = self.data
        rng = np.random.default_rng(self.seed + self.epoch)
        bounds = d.boundaries
        nb = len(bounds)
        order = [rng.permutation(int(c)) if int(c) > 0 else None for c in d.counts]
        cursor = [0] * nb
        left = d.counts.copy()
        alive = left > 0
        remaining = int(left.sum())
        per_pick = np.array([1.0 / self.micro_batch[b] for b in bounds], dtype=np.float64)
        w = np.zeros(nb, dtype=np.float64)
        cum = np.empty(nb, dtype=np.float64)
        while remaining > 0:
            got = 0
            while got < self.samples_per_step and remaining > 0:
                np.multiply(left, per_pick, out=w)
                w[~alive] = 0.0
                np.cumsum(w, out=cum)
                tot = float(cum[-1])
                if tot <= 0.0:
                    break
                u = rng.random() * tot
                bi = min(int(np.searchsorted(cum, u, side='right')), nb - 1)
                k = min(self.micro_batch[bounds[bi]], int(left[bi]), self.samples_per_step - got)
                if k <= 0:
                    alive[bi] = False
                    continue
                c = cursor[bi]
                yield (order[bi][c:c + k] + int(d.starts[bi])).tolist()
                cursor[bi] = c + k
                left[bi] -= k
                remaining -= k
                if left[bi] == 0:
                    alive[bi] = False
                got += k


def collate_pad(batch: Sequence[np.ndarray], eos_id: Optional[int] = None,
                bos_id: Optional[int] = None, max_len: Optional[int] = None) -> np.ndarray:
    """train.py:1691-1747: ``[BOS] + body + [EOS]`` per row, right-padded with 0
    to the longest row, int64.  Raises when a row would exceed ``max_len``
    (the reference never truncates)."""
    n = len(batch)
    if n == 0:
        return np.zeros((0, 0), dtype=np.int64)
    lens = np.array([len(a) for a in batch], dtype=np.int64)
    extra = (bos_id is not None) + (eos_id is not None)
    if max_len is not None and int((lens + extra).max()) > int(max_len):
        raise RuntimeError('sample longer than max_seq_len after BOS/EOS')
    out = np.zeros((n, int(lens.max()) + extra), dtype=np.int64)
    for i, a in enumerate(batch):
        at = 0
        if bos_id is not None:
            out[i, 0] = bos_id
            at = 1
        out[i, at:at + len(a)] = a
        if eos_id is not None:
            out[i, at + len(a)] = eos_id
    return out
