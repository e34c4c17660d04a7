"""Batch shaping of the reference trainer, host side: length buckets, the
token-budget micro-batch sampler and the BOS/EOS padding collate.  These decide
the (n, L) shapes the kernels see; every result is integer and must equal the
reference's bit for bit (numpy's PCG64 stream is consumed in the same order).

Names follow train.py: build_bucket_boundaries (2587-2593), FastBucket
(1060-1076), TokenBudgetBatchSampler (1750-1858), collate_pad (1691-1747).
``SyntheticBucketDataset`` stands in for FlatTokenDataset (1662-1688) with
seeded token ids instead of a memory-mapped corpus.
"""
import math

import numpy as np
import torch

BUCKET_STEP = 50


def build_bucket_boundaries(max_seq_len: int):
    edges = list(range(BUCKET_STEP, max_seq_len, BUCKET_STEP)) if max_seq_len >= BUCKET_STEP else []
    edges.append(max_seq_len)
    return edges


class FastBucket:
    def __init__(self, boundaries):
        self.boundaries = sorted(boundaries)
        self.max_boundary = self.boundaries[-1]
        self._arr = np.asarray(self.boundaries, dtype=np.int64)

    def get_bucket(self, length: int) -> int:
        if length > self.max_boundary:
            return self.max_boundary
        return int(self._arr[np.searchsorted(self._arr, length, side='left')])

    def bucket_indices(self, lengths):
        """Vector form: index of each length's bucket."""
        idx = np.searchsorted(self._arr, np.asarray(lengths), side='left')
        return np.minimum(idx, len(self._arr) - 1)


class SyntheticBucketDataset:
    """Documents with log-uniform body lengths and uniform token ids, grouped by
    bucket the way the flat cache is (global sample id = bucket start + index)."""

    def __init__(self, n_docs, max_seq_len=4096, vocab=32000, seed=0, lo=64, hi=None):
        hi = max_seq_len - 2 if hi is None else hi
        rng = np.random.default_rng(seed)
        lens = np.floor(np.exp(rng.uniform(np.log(lo), np.log(hi), size=n_docs))).astype(np.int64)
        self.boundaries = build_bucket_boundaries(max_seq_len)
        fb = FastBucket(self.boundaries)
        which = fb.bucket_indices(lens)
        order = np.argsort(which, kind='stable')
        self.lengths = lens[order]
        self.counts = np.bincount(which, minlength=len(self.boundaries)).astype(np.int64)
        self.starts = np.concatenate(([0], np.cumsum(self.counts)[:-1])).astype(np.int64)
        self.total = int(n_docs)
        self.vocab, self.seed = vocab, seed

    def __len__(self):
        return self.total

    def __getitem__(self, i):
        rng = np.random.default_rng((self.seed, int(i)))
        return rng.integers(3, self.vocab, size=int(self.lengths[i])).astype(np.uint16 if self.vocab <= 65536 else np.int64)


class TokenBudgetBatchSampler:
    """Each optimiser step consumes exactly ``samples_per_step`` samples; every
    micro-batch comes from one bucket and holds
    ``min(max_micro_batch, target_tokens // bucket_len)`` samples (shrunk until it
    tiles the step without a tiny tail); buckets are drawn with probability
    proportional to remaining_samples / micro_batch."""

    def __init__(self, dataset, samples_per_step=64, target_tokens=12288, max_micro_batch=64, seed=42):
        self.dataset = dataset
        self.samples_per_step = int(samples_per_step)
        self.seed, self.epoch, self.skip_samples = seed, 0, 0
        self.boundaries = list(dataset.boundaries)
        self.counts = np.array(dataset.counts, dtype=np.int64)
        self.bs_map = {b: self._pick_bs(int(b), target_tokens, max_micro_batch, samples_per_step)
                       for b in self.boundaries}

    @staticmethod
    def _pick_bs(bucket_len, target_tokens, max_micro_batch, samples_per_step):
        bs = max(1, min(max_micro_batch, target_tokens // max(1, bucket_len)))
        for cand in range(bs, 1, -1):
            tail = samples_per_step % cand
            if tail == 0 or tail >= max(8, cand // 3):
                return cand
        return 1

    def set_epoch(self, epoch, skip_samples=0):
        self.epoch, self.skip_samples = epoch, int(skip_samples)

    def __len__(self):
        return int(math.ceil(self.dataset.total / self.samples_per_step))

    def __iter__(self):
        stream = self._generate()
        if self.skip_samples > 0:
            done = 0
            for mb in stream:
                done += len(mb)
                if done >= self.skip_samples:
                    break
            if done != self.skip_samples:
                raise RuntimeError(f'cannot resume at sample {self.skip_samples}: micro-batch boundary is at {done}')
        yield from stream

    def steps(self):
        """Micro-batches grouped per optimiser step."""
        group, have = [], 0
        for mb in self:
            group.append(mb)
            have += len(mb)
            if have >= self.samples_per_step:
                yield group
                group, have = [], 0
        if group:
            yield group

    def _generate(self):
        rng = np.random.default_rng(self.seed + self.epoch)
        nb = len(self.boundaries)
        perm = [rng.permutation(int(c)) if c > 0 else None for c in self.counts]
        used = np.zeros(nb, dtype=np.int64)
        left = self.counts.copy()
        live = left > 0
        todo = int(left.sum())
        k_of = np.array([self.bs_map[b] for b in self.boundaries], dtype=np.int64)
        inv_k = np.array([1.0 / self.bs_map[b] for b in self.boundaries], dtype=np.float64)
        w = np.zeros(nb, dtype=np.float64)
        cum = np.empty(nb, dtype=np.float64)
        starts = self.dataset.starts
        while todo > 0:
            have = 0
            while have < self.samples_per_step and todo > 0:
                np.multiply(left, inv_k, out=w)
                w[~live] = 0.0
                np.cumsum(w, out=cum)
                if cum[-1] <= 0.0:
                    break
                bi = min(int(np.searchsorted(cum, rng.random() * float(cum[-1]), side='right')), nb - 1)
                k = int(min(k_of[bi], left[bi], self.samples_per_step - have))
                if k <= 0:
                    live[bi] = False
                    continue
                u = int(used[bi])
                yield (perm[bi][u:u + k] + int(starts[bi])).tolist()
                used[bi] += k
                left[bi] -= k
                todo -= k
                have += k
                if left[bi] == 0:
                    live[bi] = False


def collate_pad(batch, eos_id=None, bos_id=None, max_len=None):
    """[BOS] + body + [EOS] per row, right-padded with 0 to the longest row; int64
    [n, Lmax].  Never truncates: a row longer than ``max_len`` raises."""
    n = len(batch)
    if n == 0:
        return torch.zeros((0, 0), dtype=torch.long)
    lens = np.fromiter((len(a) for a in batch), dtype=np.int64, count=n)
    head = 0 if bos_id is None else 1
    extra = head + (0 if eos_id is None else 1)
    longest = int(lens.max()) + extra
    if max_len is not None and longest > int(max_len):
        raise RuntimeError(f'a sample needs {longest} tokens with BOS/EOS, more than max_seq_len={max_len}')
    out = np.zeros((n, longest), dtype=np.int64)
    if bos_id is not None:
        out[:, 0] = bos_id
    for i, a in enumerate(batch):
        out[i, head:head + lens[i]] = a
    if eos_id is not None:
        out[np.arange(n), head + lens] = eos_id
    return torch.from_numpy(out)
