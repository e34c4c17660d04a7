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
step.  No kernel reads another GPU's memory.
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


def cuda_grad_post(flat, inv_scale, out2):
    """Default post-pass: the fused CUDA kernel."""
    return ulm_ops.grad_unscale_sumsq_(flat, inv_scale, out2)


class DataParallelStep:
    def __init__(self, model, optimizer, samples_per_step, rank=0, world=1, group=None,
                 autocast_dtype=torch.bfloat16, loss_scale=None, max_grad_norm=1.0,
                 ce_chunk_rows=4096, pad_id=0, bucket_bytes=64 << 20, grad_post=cuda_grad_post,
                 device=None):
        self.model, self.opt = model, optimizer
        self.spp, self.rank, self.world, self.group = int(samples_per_step), rank, world, group
        self.dtype, self.max_norm = autocast_dtype, max_grad_norm
        self.chunk_rows, self.pad_id = ce_chunk_rows, pad_id
        self.device = device if device is not None else next(model.parameters()).device
        self.grads = FlatGrads(model.parameters())
        self.bucket_elems = max(1, bucket_bytes // 4)
        self.grad_post = grad_post
        # static loss scale (fp16): grads are computed on loss*scale and unscaled in the post-pass
        self.scale = float(loss_scale) if loss_scale else 1.0
        self.inv_scale = torch.tensor([1.0 / self.scale], dtype=torch.float32, device=self.device)
        self.stats = torch.zeros(2, dtype=torch.float32, device=self.device)

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
        for mb in micro_batches:
            n = mb.shape[0]
            n_tokens = max(1, int((mb[:, 1:] != self.pad_id).sum()))
            rows = local_rows(mb, self.rank, self.world, self.pad_id)
            if rows is None:
                continue
            ids = rows.to(self.device, non_blocking=True)
            loss_acc += self._forward_backward(ids, n / self.spp, float(n_tokens))
        flat = self.grads.flat
        if self.world > 1:
            works = [dist.all_reduce(flat[o:o + self.bucket_elems], op=dist.ReduceOp.SUM, group=self.group,
                                     async_op=True) for o in range(0, flat.numel(), self.bucket_elems)]
            works.append(dist.all_reduce(loss_acc, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            for w in works:
                w.wait()
        self.stats.zero_()
        self.grad_post(flat, self.inv_scale, self.stats)
        norm = self.stats[0].sqrt()
        skipped = bool(self.stats[1].item() != 0.0) if self.scale != 1.0 else False
        if not skipped:
            if self.max_norm is not None:
                flat.mul_(torch.clamp(self.max_norm / (norm + 1e-6), max=1.0))   # clip_grad_norm_'s factor
            self.opt.step()
        return loss_acc, norm, skipped
