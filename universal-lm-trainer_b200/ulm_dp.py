"""Data-parallel optimiser step for the reference's training loop.

The reference is single-GPU: per optimiser step it runs each micro-batch,
weights its mean loss by n/samples_per_step, accumulates gradients, then
unscales, clips and steps (train.py:2341-2375).  Here every rank builds the SAME
micro-batch list (same sampler seed), takes a contiguous slice of the ROWS of
each micro-batch, and computes

    sum over its rows of CE  /  n_tokens(micro-batch, all ranks)  *  n/samples_per_step

so that the sum over ranks equals the reference's weighted loss exactly; rows are
independent through forward and backward, so the summed gradients are the
reference's too.  One all-reduce (SUM) of the fp32 gradients per step over NCCL
follows, on a flat buffer the parameters' .grad tensors are views of; then one
fused pass unscales, checks for inf/nan and accumulates the squared norm
(ulm_grad_unscale_sumsq), and every rank applies the same clip and optimiser
step.  The all-reduce is issued bucket by bucket from gradient-ready hooks during
the backward of the rank's last micro-batch, in a fixed bucket order, so it
overlaps that backward.  No kernel reads another GPU's memory.
"""
import numpy as np
import torch
import torch.distributed as dist

import ulm_ops


def shard_bounds(n_rows: int, rank: int, world: int):
    """Contiguous, balanced row slice of a micro-batch for one rank (may be empty)."""
    return (n_rows * rank) // world, (n_rows * (rank + 1)) // world


def local_rows(micro_batch, rank, world, pad_id=0):
    """Rows [lo, hi) of an int64 [n, L] micro-batch, trimmed to their own longest
    row (trailing pad columns change nothing under a causal mask and are ignored
    by the loss).  Returns None for an empty slice."""
    lo, hi = shard_bounds(micro_batch.shape[0], rank, world)
    if hi <= lo:
        return None
    rows = micro_batch[lo:hi]
    used = int((rows != pad_id).any(dim=0).nonzero().max()) + 1 if bool((rows != pad_id).any()) else 2
    return rows[:, :max(used, 2)]


class FlatGrads:
    """One flat fp32 buffer holding every parameter's gradient (the .grad tensors
    are views), so the all-reduce and the post-pass touch few, large ranges."""

    def __init__(self, params):
        self.params = [p for p in params if p.requires_grad]
        seen, uniq = set(), []
        for p in self.params:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append(p)
        self.params = uniq
        total = sum((p.numel() + 3) // 4 * 4 for p in self.params)
        self.flat = torch.zeros(total, dtype=torch.float32, device=self.params[0].device)
        off = 0
        for p in self.params:
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            off += (p.numel() + 3) // 4 * 4

    def zero_(self):
        self.flat.zero_()

    def buckets(self, bucket_elems):
        """Contiguous slices of the flat buffer, last parameters first (their gradients are
        ready first), as (start, stop, [params])."""
        out, cur, start, off = [], [], 0, 0
        spans = []
        for p in self.params:
            n = (p.numel() + 3) // 4 * 4
            spans.append((off, off + n, p))
            off += n
        for lo, hi, p in spans:
            cur.append(p)
            if hi - start >= bucket_elems:
                out.append((start, hi, cur))
                cur, start = [], hi
        if cur:
            out.append((start, off, cur))
        return out[::-1]


def cuda_grad_post(flat, inv_scale, out2):
    """Default post-pass: the fused CUDA kernel."""
    return ulm_ops.grad_unscale_sumsq_(flat, inv_scale, out2)


class DataParallelStep:
    def __init__(self, model, optimizer, samples_per_step, rank=0, world=1, group=None,
                 autocast_dtype=torch.bfloat16, loss_scale=None, max_grad_norm=1.0,
                 ce_chunk_rows=4096, pad_id=0, bucket_bytes=64 << 20, grad_post=cuda_grad_post,
                 device=None, dynamic_loss_scale=False, growth_interval=2000):
        self.model, self.opt = model, optimizer
        self.spp, self.rank, self.world, self.group = int(samples_per_step), rank, world, group
        self.dtype, self.max_norm = autocast_dtype, max_grad_norm
        self.chunk_rows, self.pad_id = ce_chunk_rows, pad_id
        self.device = device if device is not None else next(model.parameters()).device
        self.grads = FlatGrads(model.parameters())
        self.bucket_elems = max(1, bucket_bytes // 4)
        self.grad_post = grad_post
        # loss scale (fp16): grads are computed on loss*scale and unscaled in the post-pass.  With
        # dynamic_loss_scale it follows torch's GradScaler rule (train.py:2219, 2364-2367): halve on an
        # inf/nan step (which is skipped), double after growth_interval clean steps.
        self.scale = float(loss_scale) if loss_scale else 1.0
        self.dynamic, self.growth_interval, self._clean_steps = bool(dynamic_loss_scale), int(growth_interval), 0
        self.inv_scale = torch.tensor([1.0 / self.scale], dtype=torch.float32, device=self.device)
        self.stats = torch.zeros(2, dtype=torch.float32, device=self.device)
        # gradient-ready bookkeeping for the overlapped all-reduce
        self._buckets = self.grads.buckets(self.bucket_elems)
        self._bucket_of = {}
        for bi, (_, _, ps) in enumerate(self._buckets):
            for p in ps:
                self._bucket_of[id(p)] = bi
        self._armed = False
        self._pending, self._ready, self._next, self._works = [], [], 0, []
        if self.world > 1:
            for p in self.grads.params:
                p.register_post_accumulate_grad_hook(self._on_grad_ready)

    def _arm(self):
        """Called before the backward of this rank's last micro-batch of the step."""
        self._armed = True
        self._pending = [len(ps) for _, _, ps in self._buckets]
        self._ready = [False] * len(self._buckets)
        self._next, self._works = 0, []

    def _launch_ready(self, force=False):
        # strictly in bucket order, so every rank issues the same sequence of collectives
        while self._next < len(self._buckets) and (force or self._ready[self._next]):
            lo, hi, _ = self._buckets[self._next]
            self._works.append(dist.all_reduce(self.grads.flat[lo:hi], op=dist.ReduceOp.SUM, group=self.group,
                                               async_op=True))
            self._next += 1

    def _on_grad_ready(self, p):
        if not self._armed:
            return
        bi = self._bucket_of[id(p)]
        self._pending[bi] -= 1
        if self._pending[bi] == 0:
            self._ready[bi] = True
            self._launch_ready()

    def _forward_backward(self, ids, weight, n_tokens):
        if self.device.type == 'cuda':
            with torch.autocast('cuda', dtype=self.dtype):
                loss = self.model.compute_loss(ids, ignore_index=self.pad_id, chunk_rows=self.chunk_rows,
                                               denominator=n_tokens)
        else:
            loss = self.model.compute_loss(ids, ignore_index=self.pad_id, chunk_rows=self.chunk_rows,
                                           denominator=n_tokens)
        (loss * (weight * self.scale)).backward()
        return loss.detach() * weight

    def step(self, micro_batches):
        """micro_batches: the step's int64 [n, L] tensors (host), identical on every
        rank.  Returns (weighted loss summed over ranks, grad norm, skipped)."""
        self.grads.zero_()
        loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        work = []
        for mb in micro_batches:
            n = mb.shape[0]
            n_tokens = max(1, int((mb[:, 1:] != self.pad_id).sum()))
            rows = local_rows(mb, self.rank, self.world, self.pad_id)
            if rows is not None:
                work.append((rows, n / self.spp, float(n_tokens)))
        for i, (rows, weight, n_tokens) in enumerate(work):
            if self.world > 1 and i == len(work) - 1:
                self._arm()                               # all-reduce buckets as their gradients complete
            ids = rows.to(self.device, non_blocking=True)
            loss_acc += self._forward_backward(ids, weight, n_tokens)
        flat = self.grads.flat
        if self.world > 1:
            if not self._armed:                           # this rank had no rows in the step: nothing was issued
                self._arm()
            self._launch_ready(force=True)                # whatever the hooks have not issued yet, same order
            self._armed = False
            self._works.append(dist.all_reduce(loss_acc, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            for w in self._works:
                w.wait()
        self.stats.zero_()
        self.grad_post(flat, self.inv_scale, self.stats)
        norm = self.stats[0].sqrt()
        skipped = bool(self.stats[1].item() != 0.0) if self.scale != 1.0 else False
        if not skipped:
            if self.max_norm is not None:
                flat.mul_(torch.clamp(self.max_norm / (norm + 1e-6), max=1.0))   # clip_grad_norm_'s factor
            self.opt.step()
        if self.dynamic and self.scale != 1.0:
            if skipped:
                self.scale, self._clean_steps = self.scale * 0.5, 0
            else:
                self._clean_steps += 1
                if self._clean_steps >= self.growth_interval:
                    self.scale, self._clean_steps = self.scale * 2.0, 0
            self.inv_scale.fill_(1.0 / self.scale)
        return loss_acc, norm, skipped
