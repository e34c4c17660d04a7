"""Data-parallel optimiser step for the reference's training loop.

The reference is single-GPU: per optimiser step it runs each micro-batch,
weights its mean loss by n/samples_per_step, accumulates gradients, then
unscales, clips and steps (train.py:2341-2375).  Here every rank builds the SAME
micro-batch list (same sampler seed), takes a slice of the ROWS of each
micro-batch, and computes

    sum over its rows of CE  /  n_tokens(micro-batch, all ranks)  *  n/samples_per_step

so that the sum over ranks equals the reference's weighted loss exactly; rows are
independent through forward and backward, so the summed gradients are the
reference's too.  One all-reduce (SUM) of the fp32 gradients per step over NCCL
follows, on a flat buffer the parameters' .grad tensors are views of; then one
fused pass unscales, checks for inf/nan and accumulates the squared norm
(ulm_grad_unscale_sumsq, fixed summation order: every rank gets the same bits),
and every rank applies the same clip and optimiser step.  The all-reduce is
issued bucket by bucket from gradient-ready hooks during the backward of the
rank's last micro-batch, in a fixed bucket order (`overlap_allreduce=True`), or -- the
default, and the faster of the two with persistent attention kernels -- as one
all-reduce after it.  No kernel reads another GPU's memory.

Row assignment (`plan_step`): every rank runs a few forward/backward calls, each on
consecutive rows of one micro-batch, chosen so that the ranks' estimated times are equal.
A call costs the GPU c + rows*L*(a + b*L) (linear layers plus causal attention) and the
host a fixed time to launch it; a rank takes max(sum of GPU costs, calls * host cost)
(`CostModel`, measured on B200 for the 100M preset and scaled by the model's size).

Input pipeline (`InputPipeline`): collate, token counting, row assignment and
trimming happen on a worker thread into pinned buffers, a few steps ahead of the
GPU (the reference leaves this to DataLoader worker processes,
train.py:2868-2883); the training thread only issues the async H2D copy.
"""
import collections
import contextlib
import queue
import threading
import time

import torch
import torch.distributed as dist

import ulm_ops



class CostModel(collections.namedtuple('CostModel', 'a b call host')):
    """Estimated time, in milliseconds, of one forward/backward call on `rows` rows of padded length L:
    the GPU needs ``call + rows*L*(a + b*L)``, the host ``host`` to launch it (a few thousand kernel
    launches, whatever the size); a rank's step takes max(sum of GPU times, number of calls * host).

    Measured on one B200 with the 100M preset (d 768, 10 layers, 95.4 M parameters), fp16 autocast, 36 calls of
    16 k to 48 k tokens at L = 128 ... 4096: GPU time = 1.5 ms + tokens * (8.1e-4 + 9.2e-8 * L) ms (rms error
    2.7 %, worst 7.6 %).  Launching a call costs the host 10 ms when its shapes have been seen before and
    22-33 ms when they are new (every library GEMM of a new shape costs its launcher an extra 30-50 us, and a
    training step's calls almost always have new token counts); 20 ms per 10 layers is used.  In flop terms
    the linear layers run at 707 TFLOP/s effective (norms, gates and the loss ride on them) and the attention
    at 584 TFLOP/s."""
    __slots__ = ()

    def row(self, length):
        return float(length) * (self.a + self.b * float(length))

    def load(self, gpu_costs):
        """Estimated time of a rank that runs calls with these GPU costs."""
        return max(sum(gpu_costs), len(gpu_costs) * self.host) if gpu_costs else 0.0

    @classmethod
    def for_model(cls, n_params, d_model, n_layers, checkpointing=False):
        """Scaled from the measured preset: linear work ~ 6 flops per parameter and token, attention
        3.5 * 2 * L * d_model flops per token and layer, per-call costs ~ number of layers.  With activation
        checkpointing the forward runs twice: 4/3 of the GPU work, and twice the host time per call (measured
        on the scaled preset, 24 layers of width 1024: 3.3e-3 + 3.8e-7 * L ms per token and, for repeated
        shapes, 55 ms per call on the host; this formula gives 3.3e-3, 3.9e-7 and, with 1 ms per layer for the
        launches of new shapes, which the recomputation repeats and does not pay again, 72)."""
        r = 4.0 / 3.0 if checkpointing else 1.0
        # wider layers run their GEMMs closer to peak: 707 TFLOP/s effective at width 768, 829 at 1024 (both measured)
        lin_rate = 7.07e11 * (d_model / 768.0) ** 0.55
        return cls(a=r * 6.0 * n_params / lin_rate, b=r * 7.0 * d_model * n_layers / 5.84e11,
                   call=r * 0.15 * n_layers, host=((2.0 if checkpointing else 1.0) + 1.0) * n_layers)


DEFAULT_COST = CostModel.for_model(95.4e6, 768, 10)


def shard_bounds(n_rows: int, rank: int, world: int):
    """Contiguous, balanced row slice of a micro-batch for one rank (may be empty)."""
    return (n_rows * rank) // world, (n_rows * (rank + 1)) // world


def row_cost(length: int, cost: CostModel = DEFAULT_COST) -> float:
    """GPU milliseconds one row of padded length `length` adds to a call."""
    return cost.row(length)


def _split_rows(n, k):
    """k contiguous, balanced slices of n rows."""
    return [((n * i) // k, (n * (i + 1)) // k) for i in range(k)]


def _lpt(units, world, cost):
    """Longest-processing-time assignment of (gpu_cost, payload) units to `world` bins; deterministic."""
    gpu = [[] for _ in range(world)]
    bins = [[] for _ in range(world)]
    for c, payload in sorted(units, key=lambda u: (-u[0], u[1])):
        r = min(range(world), key=lambda i: (cost.load(gpu[i] + [c]), i))
        gpu[r].append(c)
        bins[r].append(payload)
    return [cost.load(g) for g in gpu], bins


def _contiguous_plan(shapes, world, cost):
    """The micro-batches laid end to end and cut into `world` consecutive pieces of (nearly) equal
    estimated time: at most len(shapes) + world - 1 calls in all, so about one more per rank than whole
    micro-batches would need.  The smallest makespan T for which the greedy fill fits is found by
    bisection; returns (loads, bins)."""
    per_row = [cost.row(L) for _, L in shapes]

    def fill(T):
        bins, gpu = [[] for _ in range(world)], [[] for _ in range(world)]
        r = 0
        for m, (n, _) in enumerate(shapes):
            lo = 0
            while lo < n:
                room = T - sum(gpu[r]) - cost.call
                k = min(n - lo, int(room / per_row[m] + 1e-9)) if room > 0 else 0
                if (len(gpu[r]) + 1) * cost.host > T:
                    k = 0                                # one more call would make this rank launch-bound beyond T
                if k <= 0:
                    if not bins[r]:
                        return None                      # not even one row fits an empty rank
                    r += 1
                    if r == world:
                        return None
                    continue
                bins[r].append((m, lo, lo + k))
                gpu[r].append(cost.call + k * per_row[m])
                lo += k
        return [cost.load(g) for g in gpu], bins

    total = sum(n * c for (n, _), c in zip(shapes, per_row))
    lo_t = total / world
    hi_t = total + (len(shapes) + world) * max(cost.call, cost.host) + max(per_row, default=0.0)
    best = fill(hi_t)
    for _ in range(40):
        mid = 0.5 * (lo_t + hi_t)
        got = fill(mid)
        if got is None:
            lo_t = mid
        else:
            best, hi_t = got, mid
    return best


def plan_step(shapes, world: int, max_imbalance: float = 1.04, cost: CostModel = DEFAULT_COST):
    """Which rows of which micro-batch every rank computes in one optimiser step.

    ``shapes``: [(n_rows, padded_length)] in step order.  Returns ``plan[r] = [(m, lo, hi), ...]``: rank r
    runs rows [lo, hi) of micro-batch m as one forward/backward call, in the listed order.

    Rows are independent and the loss of a row subset uses its micro-batch's GLOBAL token count and
    weight, so any partition is exact.  Fewer, larger calls are cheaper (every call costs the host a few
    thousand launches, and a rank whose calls are small becomes launch-bound; small GEMMs run below peak),
    equal loads are what the gradient all-reduce waits for.  Times are estimated with ``cost``
    (`CostModel`).  Candidates: (1) the micro-batches cut into k balanced row chunks each and assigned
    longest-first (good when there are many more micro-batches than ranks: whole micro-batches go to ranks);
    (2) the micro-batches laid end to end and cut into `world` consecutive pieces (about one call more per
    rank than whole micro-batches would need, whatever the ratio).  The candidate with the smallest
    estimated makespan wins, ties going to fewer calls.  A pure function of its arguments: every rank
    computes the same plan."""
    if world == 1:
        return [[(m, 0, n) for m, (n, _) in enumerate(shapes) if n > 0]]
    shapes = [(max(int(n), 0), L) for n, L in shapes]
    costs = [n * cost.row(L) for n, L in shapes]
    total = sum(costs)
    candidates = []
    for units_per_rank in (1, 1.5, 2, 3, 4, 6, 8, 12, 16, 10 ** 9):
        target = total / (world * units_per_rank) if total > 0 else 1.0
        units = []
        for m, ((n, L), c) in enumerate(zip(shapes, costs)):
            if n <= 0:
                continue
            k = max(1, min(n, int(round(c / target)) if units_per_rank < 10 ** 9 else n))
            for lo, hi in _split_rows(n, k):
                units.append(((hi - lo) * cost.row(L) + cost.call, (m, lo, hi)))
        load, bins = _lpt(units, world, cost)
        candidates.append((max(load), len(units), bins))
        mean = sum(load) / world
        if mean > 0 and max(load) / mean <= max_imbalance:
            break
    if total > 0:
        got = _contiguous_plan(shapes, world, cost)
        if got is not None:
            load, bins = got
            candidates.append((max(load), sum(len(b) for b in bins), bins))
    best = min(candidates, key=lambda c: (round(c[0], 6), c[1]))
    # a rank runs its calls in micro-batch order (the order only has to be the same on every run)
    return [sorted(b) for b in best[2]]


def trim_rows(rows, pad_id=0):
    """Rows trimmed to their own longest row (trailing pad columns change nothing under a
    causal mask and are ignored by the loss); at least two columns."""
    nz = (rows != pad_id).any(dim=0).nonzero()
    used = int(nz.max()) + 1 if nz.numel() else 2
    return rows[:, :max(used, 2)]


def local_rows(micro_batch, rank, world, pad_id=0, bounds=None):
    """Rows [lo, hi) of an int64 [n, L] micro-batch for one rank, trimmed.  ``bounds`` is
    a (lo, hi) pair; without it the plain balanced slice is used.  Returns None for an empty slice."""
    lo, hi = bounds if bounds is not None else shard_bounds(micro_batch.shape[0], rank, world)
    if hi <= lo:
        return None
    return trim_rows(micro_batch[lo:hi], pad_id)


def prepare_step(micro_batches, rank, world, samples_per_step, pad_id=0, pin=False, cost=DEFAULT_COST):
    """Everything the host has to work out for one optimiser step on one rank:
    [(local rows int64 [n_r, L_r], loss weight n/samples_per_step, global token count)]."""
    plan = plan_step([(mb.shape[0], mb.shape[1]) for mb in micro_batches], world, cost=cost)[rank]
    n_tokens = {}
    work = []
    for m, lo, hi in plan:
        mb = micro_batches[m]
        if m not in n_tokens:
            n_tokens[m] = max(1, int((mb[:, 1:] != pad_id).sum()))   # train.py:2069, over ALL ranks' rows
        rows = trim_rows(mb[lo:hi], pad_id).contiguous()
        if pin and not rows.is_pinned():
            rows = rows.pin_memory()
        work.append((rows, mb.shape[0] / samples_per_step, float(n_tokens[m])))
    return work


def _pipeline_worker(steps, args, q, received_all):
    """Body of the input worker (thread or forked process): prepare every step, then the end marker.
    A worker process stays alive until the consumer has taken everything out of the queue: tensors
    travel as shared-memory handles that are only valid while their sender lives."""
    rank, world, spp, pad_id, pin, cost = args
    try:
        for st in steps:
            mbs = st() if callable(st) else st
            q.put(('step', prepare_step(mbs, rank, world, spp, pad_id, pin, cost)))
        q.put(('end', None))
    except BaseException as e:  # noqa: BLE001 - re-raised on the training thread
        q.put(('error', f'{type(e).__name__}: {e}'))
    received_all.wait(timeout=600)


class InputPipeline:
    """Turns an iterable of steps (each a list of int64 [n, L] host tensors, or a zero-argument callable
    producing one) into per-rank prepared work lists, ``depth`` steps ahead of the training loop.

    ``mode='process'`` (default on Linux) runs the work in a forked worker process, like the reference's
    DataLoader workers (train.py:2868-2883): collate and trimming are Python/numpy loops, and in a thread
    of the training process they would take the interpreter lock away from the thread that launches the
    kernels.  The worker never touches CUDA; its tensors arrive through shared memory.  ``mode='thread'``
    keeps everything in one process (used where forking is unwanted) and can pin its buffers.  ``cost``: the
    `CostModel` of the model being trained (`DataParallelStep.cost`); every rank must pass the same one."""

    def __init__(self, steps, rank, world, samples_per_step, pad_id=0, depth=2, pin=True, mode='process', cost=DEFAULT_COST):
        self.mode = mode
        args = (rank, world, samples_per_step, pad_id, bool(pin) and mode == 'thread', cost)
        if mode == 'process':
            import torch.multiprocessing as mp
            ctx = mp.get_context('fork')
            self._q = ctx.Queue(maxsize=max(1, depth))
            self._done = ctx.Event()
            self._w = ctx.Process(target=_pipeline_worker, args=(steps, args, self._q, self._done), daemon=True)
        elif mode == 'thread':
            self._q = queue.Queue(maxsize=max(1, depth))
            self._done = threading.Event()
            self._w = threading.Thread(target=_pipeline_worker, args=(steps, args, self._q, self._done), name='ulm-input', daemon=True)
        else:
            raise ValueError("mode must be 'process' or 'thread'")
        self._w.start()

    def __iter__(self):
        while True:
            kind, item = self._q.get()
            if kind == 'end':
                self._done.set()
                self._w.join(timeout=5)
                return
            if kind == 'error':
                self._done.set()
                raise RuntimeError(f'input pipeline worker failed: {item}')
            yield item


class RankFailure(RuntimeError):
    """A peer rank did not reach the step boundary in time."""


class StepHeartbeat:
    """Host-side failure detector for the data-parallel step.  At every step boundary each
    rank publishes ``hb/<step>/<rank>`` in the process group's key-value store and waits, with a
    time limit, for every peer's key of the same step.  A rank that died or left between steps
    is therefore noticed on the host BEFORE anything of the next step is launched -- no
    collective is started that could never complete, no kernel waits on a peer."""

    def __init__(self, store, rank, world, timeout_s=30.0):
        import datetime
        self.store, self.rank, self.world = store, rank, world
        self.timeout = datetime.timedelta(seconds=float(timeout_s))
        self.step_no = 0

    def check(self):
        k = self.step_no
        self.step_no += 1
        self.store.set(f'hb/{k}/{self.rank}', '1')
        peers = [f'hb/{k}/{r}' for r in range(self.world) if r != self.rank]
        if not peers:
            return
        try:
            self.store.wait(peers, self.timeout)
        except Exception as e:  # noqa: BLE001 - the store raises its own error types on expiry
            raise RankFailure(f'rank {self.rank}: a peer did not reach step {k} within {self.timeout.total_seconds():.1f} s: {e}') from e


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


def _check_kernel_status(device):
    """Raise if an attention kernel gave up on a barrier wait during the step."""
    import flash_attn_v100_cuda as fa
    fa.check_status(device)


def cost_model_of(model):
    """`CostModel` for a DecoderOnlyTransformer-like module: the parameters that take part in matrix products
    (all of them when the lm head is tied to the embedding table, all but the table otherwise: a lookup costs
    no flops), width, depth and whether it checkpoints its layers; DEFAULT_COST for anything else."""
    cfg = getattr(model, 'config', None)
    if cfg is None or not hasattr(cfg, 'd_model') or not hasattr(cfg, 'n_layers'):
        return DEFAULT_COST
    emb, head = getattr(model, 'embedding', None), getattr(model, 'fc_out', None)
    tied = emb is not None and head is not None and head.weight is emb.weight
    skip = {id(p) for p in emb.parameters()} if emb is not None and not tied else set()
    n_params = sum(p.numel() for p in model.parameters() if id(p) not in skip)
    return CostModel.for_model(float(n_params), int(cfg.d_model), int(cfg.n_layers),
                               bool(getattr(cfg, 'use_gradient_checkpointing', False)))


class DataParallelStep:
    def __init__(self, model, optimizer, samples_per_step, rank=0, world=1, group=None,
                 autocast_dtype=torch.bfloat16, loss_scale=None, max_grad_norm=1.0,
                 ce_chunk_rows=4096, pad_id=0, bucket_bytes=64 << 20, grad_post=cuda_grad_post,
                 device=None, dynamic_loss_scale=False, growth_interval=2000, profile=False, heartbeat=None,
                 overlap_allreduce=False, amp_scope='step', cost=None):
        self.model, self.opt = model, optimizer
        # the planner's time estimates (`CostModel`), from the model's size unless given; a pure function of
        # the configuration, so every rank derives the same one (pass it to `InputPipeline` too)
        self.cost = cost if cost is not None else cost_model_of(model)
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
        # optional per-step breakdown (CUDA events on the training stream + host clocks)
        self.profile = bool(profile) and self.device.type == 'cuda'
        self.timeline = []
        self.heartbeat = heartbeat                        # optional StepHeartbeat, checked before each step
        # False (default): ONE all-reduce of the whole flat buffer after the last backward.  True: bucket
        # all-reduces issued from gradient-ready hooks during the last backward.  Measured on 2 B200 (100M preset,
        # weak): overlapped 166.8 ms/step, not overlapped 117.9 ms/step.  The attention backward kernels are
        # persistent, one CTA per SM with all of its shared memory and TMEM; a collective kernel that sits on a few
        # SMs waiting for its peer turns their single wave into two (the rank that reaches the collective first
        # lost 50 ms of forward/backward time per step), which costs far more than the 3-6 ms the all-reduce takes
        # on its own.
        self.overlap = bool(overlap_allreduce)
        # 'step': ONE autocast context around all of a step's forward/backward calls -- the 16-bit copies autocast
        # makes of the fp32 weights are cached per context and the weights do not change within a step, so they are
        # cast once per step instead of once per call (and not again by a checkpointed layer's recomputation).
        # 'call': one context per forward, closed before its backward, like the reference's loop (train.py:2351).
        self.amp_scope = amp_scope

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
        if self.amp_scope == 'call' and self.device.type == 'cuda':
            with torch.autocast('cuda', dtype=self.dtype):
                loss = self.model.compute_loss(ids, ignore_index=self.pad_id, chunk_rows=self.chunk_rows, denominator=n_tokens)
        else:
            loss = self.model.compute_loss(ids, ignore_index=self.pad_id, chunk_rows=self.chunk_rows, denominator=n_tokens)
        (loss * (weight * self.scale)).backward()
        return loss.detach() * weight

    def _event(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def accumulate(self, work, reduce=True):
        """Zero the gradients, run forward/backward over the prepared ``work`` list and (with
        ``reduce`` and world > 1) all-reduce; returns the weighted loss summed over ranks.
        Gradients are left in ``self.grads.flat`` still multiplied by the loss scale."""
        prof = self.profile
        t_host0 = time.perf_counter()
        ev = [self._event()] if prof else None
        self.grads.zero_()
        loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        sharded = reduce and self.world > 1
        step_scope = self.device.type == 'cuda' and self.amp_scope == 'step'
        amp = torch.autocast('cuda', dtype=self.dtype) if step_scope else contextlib.nullcontext()
        # weight gradients are added straight into the flat fp32 buffer by their GEMMs (no 16-bit product, no cast
        # and add passes); not with the hook-driven bucket all-reduce, which waits for autograd's accumulation
        in_place = ulm_ops.wgrad_in_place(self.device.type == 'cuda' and not self.overlap)
        # the weights do not change between here and the optimiser step: their 16-bit copies are made once
        # Token ids of ALL of the step's calls go to the device first, through pinned memory: a copy from pageable
        # memory (what a worker process delivers) is not asynchronous, and issued between two calls it would make
        # the launching thread wait for the GPU to finish the previous call.
        if self.device.type == 'cuda':
            dev_ids = [(rows if rows.is_pinned() else rows.pin_memory()).to(self.device, non_blocking=True) for rows, _, _ in work]
        else:
            dev_ids = [rows for rows, _, _ in work]
        with amp, in_place, ulm_ops.weight_cast_scope():
            for i, (rows, weight, n_tokens) in enumerate(work):
                if sharded and self.overlap and i == len(work) - 1:
                    self._arm()                           # all-reduce buckets as their gradients complete
                loss_acc += self._forward_backward(dev_ids[i], weight, n_tokens)
        if prof:
            ev.append(self._event())
        if sharded:
            if self.overlap:
                if not self._armed:                       # this rank had no rows in the step: nothing was issued
                    self._arm()
                self._launch_ready(force=True)            # whatever the hooks have not issued yet, same order
                self._armed = False
            else:
                self._works = [dist.all_reduce(self.grads.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)]
            self._works.append(dist.all_reduce(loss_acc, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            for w in self._works:
                w.wait()
        if prof:
            ev.append(self._event())
            self._prof = (t_host0, ev)
        return loss_acc

    def step(self, micro_batches=None, work=None):
        """One optimiser step.  ``micro_batches``: the step's int64 [n, L] tensors (host),
        identical on every rank; or ``work``: the list `prepare_step` / `InputPipeline` made
        from them for this rank.  Returns (weighted loss summed over ranks, grad norm, skipped)."""
        if self.heartbeat is not None:
            self.heartbeat.check()                        # raises RankFailure before anything is launched
        if work is None:
            work = prepare_step(micro_batches, self.rank, self.world, self.spp, self.pad_id, cost=self.cost)
        loss_acc = self.accumulate(work)
        flat = self.grads.flat
        self.stats.zero_()
        self.grad_post(flat, self.inv_scale, self.stats)
        norm = self.stats[0].sqrt()
        t_enq = time.perf_counter() - self._prof[0] if self.profile else 0.0   # host time to enqueue everything so far
        if self.scale != 1.0:
            # the one host sync of the step (the reference's is loss_accum.item(), train.py:2375); the
            # attention kernels' status word is read under the same sync
            skipped = bool(self.stats[1].item() != 0.0)
        else:
            skipped = False
        if not skipped:
            if self.max_norm is not None:
                flat.mul_(torch.clamp(self.max_norm / (norm + 1e-6), max=1.0))   # clip_grad_norm_'s factor
            self.opt.step()
        if self.profile:
            t_host0, ev = self._prof
            ev.append(self._event())
            ev[-1].synchronize()
            self.timeline.append(dict(fwd_bwd_ms=ev[0].elapsed_time(ev[1]), allreduce_exposed_ms=ev[1].elapsed_time(ev[2]),
                                      post_opt_ms=ev[2].elapsed_time(ev[3]), gpu_ms=ev[0].elapsed_time(ev[3]),
                                      host_enqueue_ms=t_enq * 1e3, host_step_ms=(time.perf_counter() - t_host0) * 1e3, micro_batches=len(work),
                                      rows=sum(int(w[0].shape[0]) for w in work),
                                      tokens_padded=sum(int(w[0].numel()) for w in work)))
        if self.device.type == 'cuda':
            _check_kernel_status(self.device)             # a barrier timeout must not pass as a good step
        if self.dynamic and self.scale != 1.0:
            if skipped:
                self.scale, self._clean_steps = self.scale * 0.5, 0
            else:
                self._clean_steps += 1
                if self._clean_steps >= self.growth_interval:
                    self.scale, self._clean_steps = self.scale * 2.0, 0
            self.inv_scale.fill_(1.0 / self.scale)
        return loss_acc, norm, skipped

    def gradients_of(self, micro_batches, sharded=True):
        """Loss and unscaled gradients of one step WITHOUT touching the optimiser: with
        ``sharded`` the data-parallel way (this rank's rows, all-reduce), otherwise every row
        on this rank alone.  Used to check that the two agree.  Returns (loss, flat clone)."""
        if sharded:
            work = prepare_step(micro_batches, self.rank, self.world, self.spp, self.pad_id, cost=self.cost)
        else:
            work = prepare_step(micro_batches, 0, 1, self.spp, self.pad_id)
        loss = self.accumulate(work, reduce=sharded)
        flat = self.grads.flat * self.inv_scale
        if self.device.type == 'cuda':
            torch.cuda.synchronize()
            _check_kernel_status(self.device)
        return float(loss), flat
