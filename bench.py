#!/usr/bin/env python
"""Benchmark of the hot path: causal attention forward+backward at S=4096, D=64.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = RoPE (768-wide table) + causal attention forward + backward over the
configuration B=8, H=12, S=4096, D=64 per GPU, from unrotated q, k to the gradients
of the unrotated q, k and of v: the stand-alone RoPE kernel on K, the forward kernel
and the dQ and dK/dV kernels (delta is computed inside the dQ kernel) and the RoPE
adjoint on dQ, dK -- as stand-alone RoPE launches or fused into the attention kernels,
whichever flash_attn_v100_cuda.ROPE_FUSION selects (the three placements are timed
side by side in `kernels.step_ms_by_rope_fusion`).
Prints ONE JSON line on rank 0.

  value      whole-job TFLOP/s with inputs resident in HBM; FLOPs are the
             algorithmic 3.5 * 2*B*H*S^2*D (causal-halved forward x (1 + 2.5)).  The timed
             region (exactly K steps between barriers) is taken three times and all are
             listed in ms_per_step_repeats; ms_per_step is the first unless that one is an
             outlier (a stall from outside the process), then the median.
  e2e        the same metric through the public wrapper (rope_flash_attn autograd)
             with HOST buffers: pinned H2D of q,k,v,dO and D2H of o,dq,dk,dv inside
             the timed region (copies overlap compute on separate streams).
  roofline   the slowest kernel of the step, timed alone with CUDA events.
  cpu_baseline  the oracle (the reference's PyTorch path) on the host cores, on
             a bounded sample (one batch element of the same workload).

  train      the data-parallel training step of the 100M preset (weak: 64 samples per
             GPU per step; strong: 64 samples per step in total) and train_scaled, the
             scaled preset with a fixed global batch of 256 sequences (strong), each with
             a per-rank breakdown (GPU time in forward/backward, exposed all-reduce,
             post-pass + optimiser, host enqueue time); at N > 1 dp_check compares one
             step computed sharded over the N ranks with the same step computed whole
             on one rank.
--impl reference times that CPU path alone, K steps of the bounded sample.
Multi-GPU: one process per GPU (torchrun); for the headline ranks hold independent
batches (weak scaling, no data-path collective); time is the max over ranks.
"""
import argparse
import json
import os
import statistics
import subprocess
import threading
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, 'universal-lm-trainer_b200')):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

B, H, S, D, D_MODEL = 8, 12, 4096, 64, 768
FWD_FLOPS = 4.0 * B * H * S * S * D / 2.0           # causal-halved QK^T + PV
STEP_FLOPS = 3.5 * FWD_FLOPS                         # backward counted as 2.5 x forward
METRIC = 'causal attn fwd+bwd TFLOP/s (S=4096,D=64)'
kRepeats = 3                                          # timed regions are taken this many times (outlier guard)
NCU_TRAFFIC = {'attn_fwd': 453.2e6, 'attn_bwd_dq': 738.8e6, 'attn_bwd_dkv': 691.1e6}
WORKLOAD = 'configs[1]: RoPE (768-wide table) + causal attention fwd+bwd, B=8 H=12 S=4096 D=64, unrotated q,k in, gradients of unrotated q,k and v out'


def peaks():
    try:
        with open(os.path.join(ROOT, 'MEASURED_PEAKS.json')) as f:
            p = json.load(f)
        return dict(bf16_burst=p['bf16_tflops'], bf16_sustained=p['bf16_tflops_sustained'],
                    hbm=p['hbm_gbs'], source='measured')
    except Exception:  # noqa: BLE001 - file is written by the driver and may be absent
        return dict(bf16_burst=1590.0, bf16_sustained=1400.0, hbm=6650.0, source='fallback')


class ClockSampler:
    """nvidia-smi clocks/throttle reasons every 200 ms while the timed region runs."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
         'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
         'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines, self.reader = gpu_index, None, [], None

    def start(self, wait_s=15.0):
        """Launch the sampler and wait for its first sample.  Call it BEFORE the warm-up: the tool's start-up
        (process spawn, NVML initialisation) can hold up this process's CUDA calls for seconds on a busy
        host, which must not land inside the timed region; the periodic queries that follow are cheap."""
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '200', '-i', str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.reader = threading.Thread(target=lambda: self.lines.extend(iter(self.proc.stdout.readline, '')), daemon=True)
        self.reader.start()
        t0 = time.perf_counter()
        while not self.lines and time.perf_counter() - t0 < wait_s and self.proc.poll() is None:
            time.sleep(0.02)

    def mark(self):
        """Samples taken before this call are not part of the timed region."""
        self.first = len(self.lines)

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=['nvidia-smi unavailable'])
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            self.proc.wait()
        self.reader.join(timeout=5)
        out = ''.join(self.lines[getattr(self, 'first', 0):])
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(',')]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), f[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def make_inputs(dtype, device, seed):
    """Config-2 inputs: i.i.d. N(0,1) q,k,v,dO from a seed (as one fused qkv buffer,
    the layout the model produces), tables from the 768-wide RoPE."""
    from ulm_model import rope_tables
    g = torch.Generator().manual_seed(seed)
    qkv = torch.randn((B, S, 3 * H * D), generator=g, dtype=torch.float32).to(dtype)
    do = torch.randn((B, S, H, D), generator=g, dtype=torch.float32).to(dtype)
    cos, sin = rope_tables(D_MODEL, S)
    return qkv, do, cos.to(device), sin.to(device)


def views(qkv):
    return tuple(t.view(B, S, H, D).transpose(1, 2) for t in qkv.chunk(3, dim=-1))


def event_time_ms(fn, iters, warm=2, flush=None):
    """Mean device time of ``fn``.  ``flush``: a buffer larger than L2 that is overwritten before every
    iteration (each iteration is then timed with its own pair of events) -- for workloads whose
    footprint would otherwise sit in the 126 MB L2 from one iteration to the next."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    if flush is None:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(iters):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / iters
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        fn()
        t1.record()
        torch.cuda.synchronize()
        total += t0.elapsed_time(t1)
    return total / iters


def cpu_reference_step(dtype, threads):
    """The reference's PyTorch path for one batch element of the workload:
    eager RoPE (train.py:1914-1918) -> cast -> SDPA is_causal (train.py:1956)
    -> backward, on the host cores."""
    from oracle import ops
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(1)
    q, k, v, do = (torch.randn((1, H, S, D), generator=g).to(dtype) for _ in range(4))
    cos, sin = ops.rope_tables_head(D_MODEL, S, D)

    def step():
        t0 = time.perf_counter()
        ops.rope_attention_grads(q, k, v, do, cos, sin, dtype, use_sdpa=True)
        return time.perf_counter() - t0
    return step, STEP_FLOPS / B


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    step, flops = cpu_reference_step(torch.bfloat16, threads)
    for _ in range(args.warmup):
        step()
    times = [step() for _ in range(args.steps)]
    t = sum(times) / len(times)
    val = flops / t / 1e12
    sample = f'one batch element (B=1,H={H},S={S},D={D}) per step, bf16, eager RoPE + SDPA fwd+bwd on CPU'
    _emit(json.dumps({
        'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': 'TFLOP/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': t * 1e3, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
        'config': {'workload': WORKLOAD, 'sample': sample},
        'cpu_baseline': {'value': val, 'unit': 'TFLOP/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                         'sample': sample},
        'e2e': {'value': val, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }))


def bandwidth_bench(dev, pk):
    """configs[3]: RMSNorm over 32768 x 768 bf16 and the cross-entropy row kernels over
    [4096, 32000] bf16 logits tiles (8 chunks = 32768 rows), 5 % ignored targets.  GB/s
    against the measured copy bandwidth; algorithmic bytes: RMSNorm fwd 2*N*d*2, bwd
    3*N*d*2; CE fwd N*V*2, bwd 2*N*V*2."""
    import ulm_ops
    N_, d, V, R = 32768, 768, 32000, 4096
    g = torch.Generator().manual_seed(5)
    x = torch.randn((N_, d), generator=g).to(torch.bfloat16).to(dev)
    dy = torch.randn((N_, d), generator=g).to(torch.bfloat16).to(dev)
    w = (1 + 0.02 * torch.randn((d,), generator=g)).to(dev)
    W = (0.02 * torch.randn((V, d), generator=g)).to(torch.bfloat16).to(dev)
    t = torch.randint(1, V, (N_,), generator=g)
    t[torch.rand(N_, generator=g) < 0.05] = 0
    t = t.to(dev)
    out = {}
    # RMSNorm straight through the C ABI with preallocated outputs: the kernels take ~20-30 us, so
    # per-call tensor allocation on the host would be what gets timed otherwise
    import ctypes as C
    import _native as N
    lib = N.lib()
    y, dx = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(N_, device=dev)
    dw = torch.empty(d, device=dev)
    partial = torch.empty((int(lib.ulm_rmsnorm_bwd_partial_rows(N_)), d), device=dev)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    fa_ = N.RmsFwdArgs(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), d, d, N_, d, N.ULM_BF16, N.ULM_F32, 1e-6, st)
    ba_ = N.RmsBwdArgs(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                       partial.data_ptr(), d, d, d, N_, d, N.ULM_BF16, N.ULM_F32, 1e-6, st)
    # 101 / 151 MB footprints are below the 126 MB L2 or close to it: flush L2 (256 MB write) before every
    # timed launch; the back-to-back time (partly L2-resident) and a plain copy of the same tensors are
    # reported beside it
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    f_fwd = lambda: N.check(lib.ulm_rmsnorm_fwd(C.byref(fa_)), 'rms fwd')    # noqa: E731
    f_bwd = lambda: N.check(lib.ulm_rmsnorm_bwd(C.byref(ba_)), 'rms bwd')    # noqa: E731
    ms = event_time_ms(f_fwd, 20, flush=flush)
    out['rmsnorm_fwd'] = {'ms': ms, 'gbs': 2 * N_ * d * 2 / (ms * 1e-3) / 1e9, 'ms_back_to_back': event_time_ms(f_fwd, 50),
                          'ms_copy_same_bytes': event_time_ms(lambda: y.copy_(x), 20, flush=flush), 'l2': 'flushed before every launch'}
    ms = event_time_ms(f_bwd, 20, flush=flush)
    out['rmsnorm_bwd'] = {'ms': ms, 'gbs': 3 * N_ * d * 2 / (ms * 1e-3) / 1e9, 'ms_back_to_back': event_time_ms(f_bwd, 50),
                          'l2': 'flushed before every launch'}
    # the training layout: fp32 residual stream, 16-bit branch / y / dy, residual add fused in (12 and 16 bytes per element)
    xf, brh = torch.randn(N_, d, device=dev), torch.randn(N_, d, device=dev).to(torch.float16)
    xo, yh, dyh, gadd = torch.empty_like(xf), torch.empty_like(brh), torch.randn(N_, d, device=dev).to(torch.float16), torch.randn(N_, d, device=dev)
    dxf, dbr = torch.empty_like(xf), torch.empty_like(brh)
    fa2 = N.RmsFwdArgs(xf.data_ptr(), w.data_ptr(), yh.data_ptr(), rstd.data_ptr(), d, d, N_, d, N.ULM_F32, N.ULM_F32, 1e-6, st,
                       N.ULM_Y_F16, 0, brh.data_ptr(), xo.data_ptr(), d, d)
    ba2 = N.RmsBwdArgs(xo.data_ptr(), w.data_ptr(), dyh.data_ptr(), rstd.data_ptr(), dxf.data_ptr(), dw.data_ptr(), partial.data_ptr(),
                       d, d, d, N_, d, N.ULM_F32, N.ULM_F32, 1e-6, st, N.ULM_Y_F16, 0, gadd.data_ptr(), dbr.data_ptr(), d, d)
    ms = event_time_ms(lambda: N.check(lib.ulm_rmsnorm_fwd(C.byref(fa2)), 'add rms fwd'), 20, flush=flush)
    out['add_rmsnorm_fwd'] = {'ms': ms, 'gbs': 12 * N_ * d / (ms * 1e-3) / 1e9, 'l2': 'flushed before every launch'}
    ms = event_time_ms(lambda: N.check(lib.ulm_rmsnorm_bwd(C.byref(ba2)), 'add rms bwd'), 20, flush=flush)
    out['add_rmsnorm_bwd'] = {'ms': ms, 'gbs': 16 * N_ * d / (ms * 1e-3) / 1e9, 'l2': 'flushed before every launch'}
    del flush, xf, brh, xo, yh, dyh, gadd, dxf, dbr
    # SwiGLU gate over the 100M preset's feed-forward width: [32768, 2048] bf16 (134 MB per tensor > L2)
    ga, gb, gdy = (torch.randn(N_, 2048, device=dev).to(torch.bfloat16) for _ in range(3))
    gy, gda, gdb = torch.empty_like(ga), torch.empty_like(ga), torch.empty_like(ga)
    sa = N.SwigluArgs(ga.data_ptr(), gb.data_ptr(), gy.data_ptr(), gdy.data_ptr(), gda.data_ptr(), gdb.data_ptr(),
                      ga.numel(), N.ULM_BF16, 0, st)
    ms = event_time_ms(lambda: N.check(lib.ulm_swiglu_fwd(C.byref(sa)), 'swiglu fwd'), 30)
    out['swiglu_fwd'] = {'ms': ms, 'gbs': 3 * ga.numel() * 2 / (ms * 1e-3) / 1e9}
    ms = event_time_ms(lambda: N.check(lib.ulm_swiglu_bwd(C.byref(sa)), 'swiglu bwd'), 30)
    out['swiglu_bwd'] = {'ms': ms, 'gbs': 5 * ga.numel() * 2 / (ms * 1e-3) / 1e9}
    del ga, gb, gdy, gy, gda, gdb
    logits = [(x[i:i + R] @ W.t()) for i in range(0, N_, R)]        # 8 tiles of 262 MB: 2.1 GB > L2
    lses = [None] * len(logits)

    def ce_f():
        for i, lg in enumerate(logits):
            lses[i], _ = ulm_ops.ce_rows_forward(lg, t[i * R:(i + 1) * R], 0)
    ms = event_time_ms(ce_f, 5)
    out['ce_fwd'] = {'ms': ms, 'gbs': N_ * V * 2 / (ms * 1e-3) / 1e9}
    one = torch.ones(1, device=dev)

    def ce_b():
        for i, lg in enumerate(logits):
            ulm_ops.ce_rows_backward_(lg, t[i * R:(i + 1) * R], lses[i], one, 0)
    ms = event_time_ms(ce_b, 3, warm=1)      # in place: values decay towards softmax fixed points, timing is unaffected
    out['ce_bwd'] = {'ms': ms, 'gbs': 2 * N_ * V * 2 / (ms * 1e-3) / 1e9}
    del logits
    # the lm-head GEMM with the statistics in its epilogue (one tcgen05 kernel) against the library GEMM + the row pass
    ms_keep = event_time_ms(lambda: ulm_ops.lm_head_lse(x, W, t, 0, keep_logits=True), 5)
    ms_lse = event_time_ms(lambda: ulm_ops.lm_head_lse(x, W, t, 0, keep_logits=False), 5)
    ms_gemm = event_time_ms(lambda: x @ W.t(), 5)
    gflop = 2.0 * N_ * V * d
    out['lm_head_lse'] = {'ms_logits_stored': ms_keep, 'ms_statistics_only': ms_lse, 'ms_library_gemm_alone': ms_gemm,
                          'ms_library_gemm_plus_ce_fwd': ms_gemm + out['ce_fwd']['ms'],
                          'tflops_statistics_only': gflop / (ms_lse * 1e-3) / 1e12, 'tflops_logits_stored': gflop / (ms_keep * 1e-3) / 1e12,
                          'frac_of_burst_peak': gflop / (ms_lse * 1e-3) / 1e12 / peaks()['bf16_burst']}
    h = x.float().requires_grad_(True)
    Wf = W.float().requires_grad_(True)

    def ce_op():
        loss = ulm_ops.chunked_cross_entropy(h, Wf, t, ignore_index=0, chunk_rows=R, compute_dtype=torch.bfloat16)
        loss.backward()
        return loss
    ms = event_time_ms(ce_op, 6, warm=3)
    out['chunked_ce_fwd_bwd_with_gemms'] = {'ms': ms, 'gemm_tflops': 3 * 2.0 * N_ * V * d / (ms * 1e-3) / 1e12,
                                           'form': 'logits of all rows kept in one 16-bit buffer (fused lm-head GEMM + statistics forward, two library GEMMs backward), no recomputation',
                                           'loss': float(ce_op().detach())}
    ulm_ops.FUSED_LM_HEAD = False
    ms = event_time_ms(ce_op, 6, warm=3)
    ulm_ops.FUSED_LM_HEAD = True
    out['chunked_ce_fwd_bwd_with_gemms_library_forward'] = {'ms': ms, 'form': 'the same with the forward as library GEMM + a pass over the logits (what the fused kernel replaced)'}
    keep_bytes, ulm_ops.KEEP_LOGITS_BYTES = ulm_ops.KEEP_LOGITS_BYTES, 0
    ms = event_time_ms(ce_op, 6, warm=3)
    out['chunked_ce_fwd_bwd_with_gemms_recompute'] = {'ms': ms, 'gemm_tflops': 4 * 2.0 * N_ * V * d / (ms * 1e-3) / 1e12,
                                                     'form': 'chunk by chunk, logits recomputed in the backward: 4 GEMMs per chunk',
                                                     'loss': float(ce_op().detach())}
    ulm_ops.KEEP_LOGITS_BYTES = keep_bytes
    for v_ in out.values():
        if 'gbs' in v_:
            v_['frac_hbm'] = v_['gbs'] / pk['hbm']
    return out


def _gather(obj, world, dist):
    if world == 1:
        return [obj]
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


def train_bench(preset_name, scaling, args, rank, world, dev, dist, pk, warm, timed, base_spp, check=False):
    """Data-parallel training step of a preset.  Every rank draws the same micro-batch list,
    takes its row slices (ulm_dp.plan_step), all-reduces fp32 gradients over NCCL, then the
    fused unscale/norm pass, clip and fused AdamW.  ``scaling`` = 'weak': ``base_spp`` samples
    and a 32768-token / 64-row micro-batch budget PER GPU (the global sampler runs with all
    three multiplied by N); 'strong': ``base_spp`` samples per step in total whatever N.
    Collate, token counts, row assignment and trimming run on the input pipeline's worker
    thread; token ids are copied host->device inside the timed region."""
    import ulm_dp
    import ulm_train
    import _native
    model, preset = ulm_train.build(preset_name, dev, seed=0)
    opt = ulm_train.make_optimizer(model)
    mult = world if scaling == 'weak' else 1
    spp = base_spp * mult
    torch.cuda.empty_cache()       # earlier sections leave multi-GB blocks cached that no step here can reuse
    sources = ulm_train.step_sources(preset_name, spp, warm + timed, target_tokens=32768 * mult,
                                     max_micro_batch=64 * mult, data_seed=7)
    runner = ulm_dp.DataParallelStep(model, opt, samples_per_step=spp, rank=rank, world=world,
                                     autocast_dtype=preset['dtype'], loss_scale=preset['loss_scale'],
                                     dynamic_loss_scale=preset['loss_scale'] is not None,
                                     max_grad_norm=1.0, ce_chunk_rows=4096, pad_id=0, device=dev, profile=True,
                                     overlap_allreduce=args.overlap)
    dp_check = None
    if check and world > 1:
        # one step both ways before any optimiser state exists: sharded over the ranks + all-reduce, and whole
        # on this rank; every rank holds both results and reports its own difference
        mbs = sources[0]()
        loss_s, g_s = runner.gradients_of(mbs, sharded=True)
        loss_u, g_u = runner.gradients_of(mbs, sharded=False)
        rel = float((g_s - g_u).norm() / g_u.norm())
        both = _gather((abs(loss_s - loss_u), rel), world, dist)
        dp_check = {'loss_abs_diff': max(b[0] for b in both), 'grad_rel_diff': max(b[1] for b in both),
                    'what': f'one step of {spp} samples: {world} ranks sharded + NCCL all-reduce vs all rows on one rank, '
                            f'{str(preset["dtype"]).split(".")[-1]} autocast', 'loss': loss_u}
        dp_check['within_tolerance'] = bool(dp_check['loss_abs_diff'] <= 1e-3 and dp_check['grad_rel_diff'] <= 2e-2)
        del g_s, g_u
    # token counts of every step, for the throughput figures (the timed loop gets its batches from the worker process)
    host_steps = [ulm_train.token_counts(s_()) for s_ in sources]
    pipe = iter(ulm_dp.InputPipeline(sources, rank, world, spp, pad_id=0, depth=3, cost=runner.cost))
    for _ in range(warm):
        runner.step(work=next(pipe))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    runner.timeline.clear()
    n0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    e0.record()
    losses = []
    for work in pipe:
        loss, norm, skipped = runner.step(work=work)
        losses.append(loss)
    e1.record()
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall
    if world > 1:
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    n_steps = len(losses)
    ms = float(t.item()) / n_steps
    real = sum(h[0] for h in host_steps[warm:]) / n_steps
    padded = sum(h[1] for h in host_steps[warm:]) / n_steps
    mean_len = padded / spp
    fl = ulm_train.flops_per_token(preset_name, mean_len) * padded
    keys = ('fwd_bwd_ms', 'allreduce_exposed_ms', 'post_opt_ms', 'gpu_ms', 'host_enqueue_ms', 'host_step_ms', 'rows', 'tokens_padded', 'micro_batches')
    mine = {k: sum(st[k] for st in runner.timeline) / max(1, len(runner.timeline)) for k in keys}
    mine['wall_ms'] = t_wall * 1e3 / n_steps
    per_rank = _gather(mine, world, dist)
    out = {'metric': f'{preset_name}-preset training tokens/s', 'value': real / (ms * 1e-3), 'unit': 'tokens/s',
           'padded_tokens_per_s': padded / (ms * 1e-3), 'ms_per_step': ms, 'steps': n_steps, 'warmup': warm,
           'n_gpus': world, 'scaling': scaling, 'our_kernel_launches': int(_native.launch_count() - n0),
           'loss_first_last': [float(losses[0]), float(losses[-1])],
           'model_tflops_per_gpu': fl / (ms * 1e-3) / 1e12 / world,
           'mfu_of_sustained': fl / (ms * 1e-3) / 1e12 / world / pk['bf16_sustained'],
           'per_rank_mean_per_step': per_rank,
           'config': {'preset': str(preset['model']) + f', {str(preset["dtype"]).split(".")[-1]} autocast, '
                                + ('dynamic loss scale from 65536, ' if preset['loss_scale'] else '')
                                + ('gradient checkpointing, ' if preset['checkpointing'] else '') + 'fused AdamW',
                      'samples_per_step': spp, 'target_tokens': 32768 * mult, 'max_micro_batch': 64 * mult, 'ce_chunk_rows': 4096,
                      'lengths': 'log-uniform [64,4094], token ids uniform, seeded',
                      'parallelism': f'dp{world} (rows of each micro-batch sharded, extra rows to the least loaded ranks)',
                      'flops': 'model FLOPs 3 x (linears + lm head) + 3.5 x causal attention; recomputation under checkpointing not counted'}}
    if dp_check is not None:
        out['dp_check'] = dp_check
    if world == 1 and args.kernel_table:
        out['kernel_time_shares'] = kernel_table(runner, [s_() for s_ in sources[:3]])
    del runner, opt, model
    torch.cuda.empty_cache()
    return out


def kernel_table(runner, steps, top=24):
    """Where the GPU time of a training step goes: three more steps under torch.profiler (CUPTI kernel
    records; the step timing above is taken without it), kernels grouped by name."""
    from torch.profiler import profile, ProfilerActivity
    import re
    runner.step(steps[0])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for st in steps:
            runner.step(st)
        torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ev = [e for e in prof.key_averages() if e.device_time_total > 0]
    total = sum(e.device_time_total for e in ev)

    def group(name):
        if name.startswith('nvjet') or 'gemm' in name.lower() or 'cutlass' in name.lower():
            return 'library GEMMs (cuBLAS)'
        m = re.search(r'(attn_\w+_kernel|rope_kernel|rmsnorm_\w+_kernel|swiglu_\w+_kernel|ce_\w+_kernel|unscale_sumsq_kernel|sumsq_reduce_kernel)', name)
        if m:
            return 'ulm::' + m.group(1)
        if 'nccl' in name.lower():
            return 'NCCL'
        return 'PyTorch: ' + re.sub(r'<.*', '', name.replace('void ', '').replace('at::native::', ''))[:60]
    agg = {}
    for e in ev:
        g = group(e.key)
        a = agg.setdefault(g, [0.0, 0])
        a[0] += e.device_time_total
        a[1] += e.count
    rows = sorted(agg.items(), key=lambda kv: -kv[1][0])[:top]
    return {'steps': len(steps), 'gpu_busy_fraction_under_profiler': total / 1e6 / wall,
            'kernel_ms_per_step': total / 1e3 / len(steps),
            'groups': [{'kernel': k, 'share': v[0] / total, 'ms_per_step': v[0] / 1e3 / len(steps), 'launches_per_step': v[1] / len(steps)}
                       for k, v in rows]}


def same_box_training_baseline(dev, warm=1, timed=3):
    """The reference's own PyTorch path for the 100M step (eager RoPE, F.scaled_dot_product_attention,
    F.rms_norm, chunked F.cross_entropy under fp16 autocast with GradScaler and fused AdamW:
    oracle.model.OracleLM, which restates train.py:1920-2082) on this GPU, on the same batches the
    `train` section uses at one GPU.  A library baseline measured beside ours, not part of our path."""
    import ulm_train
    from oracle import model as omodel
    cfg = ulm_train.PRESETS['100m']['model']
    torch.manual_seed(0)
    m = omodel.OracleLM(omodel.OracleModelConfig(**cfg)).to(dev)
    opt = ulm_train.make_optimizer(m)
    scaler = torch.amp.GradScaler('cuda', init_scale=65536.0)
    steps = [s_() for s_ in ulm_train.step_sources('100m', 64, warm + timed, data_seed=7)]
    torch.cuda.reset_peak_memory_stats()

    def one(mbs):
        opt.zero_grad(set_to_none=True)
        for mb in mbs:
            ids = mb.to(dev, non_blocking=True)
            with torch.autocast('cuda', dtype=torch.float16):
                loss = m.compute_loss(ids, ignore_index=0, chunk_rows=4096)
            scaler.scale(loss * (mb.shape[0] / 64)).backward()
        scaler.unscale_(opt)
        torch.nn.utils.clip_grad_norm_(m.parameters(), 1.0)
        scaler.step(opt)
        scaler.update()
    for st in steps[:warm]:
        one(st)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for st in steps[warm:]:
        one(st)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / timed
    real = sum(ulm_train.token_counts(st)[0] for st in steps[warm:]) / timed
    out = {'what': 'reference PyTorch path (oracle.model.OracleLM: eager RoPE, SDPA, F.rms_norm, chunked F.cross_entropy), '
                   '100M preset, fp16 autocast + GradScaler + fused AdamW, same batches as train at 1 GPU',
           'ms_per_step': ms, 'tokens_per_s': real / (ms * 1e-3), 'steps': timed,
           'peak_memory_gb': torch.cuda.max_memory_allocated() / 2 ** 30}
    del m, opt
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--dtype', default='bf16', choices=['bf16', 'fp16'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-train', action='store_true')
    ap.add_argument('--no-scaled', action='store_true')
    ap.add_argument('--no-kernel-table', dest='kernel_table', action='store_false', help='skip the torch.profiler pass over three training steps (1 GPU only)')
    ap.add_argument('--overlap', action='store_true', help='bucket all-reduces during the last backward instead of one all-reduce after it')
    ap.add_argument('--scaled-steps', type=int, default=3)
    ap.add_argument('--train-steps', type=int, default=20)
    ap.add_argument('--lm-head-rows', type=int, default=0,
                    help='time only the fused lm-head kernel on this many rows (V=32000, d=768) and exit: the small case for profiler captures')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if args.impl == 'reference':
        return run_reference(args, rank, world)

    import torch.distributed as dist
    import flash_attn_v100_cuda as fa
    import _native

    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a GPU (there is no CPU path for the kernels)')
    if not fa.is_available():
        raise SystemExit(f'libulm_b200.so unavailable: {fa.build_error()}')
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    dtype = torch.bfloat16 if args.dtype == 'bf16' else torch.float16
    if args.lm_head_rows:
        import ulm_ops
        n, V, d = args.lm_head_rows, 32000, 768
        g = torch.Generator().manual_seed(0)
        x = torch.randn((n, d), generator=g).to(dtype).to(dev)
        W = (0.02 * torch.randn((V, d), generator=g)).to(dtype).to(dev)
        t = torch.randint(1, V, (n,), generator=g).to(dev)
        res = {'rows': n, 'V': V, 'd': d, 'dtype': args.dtype}
        for keep in (True, False):
            ms = event_time_ms(lambda: ulm_ops.lm_head_lse(x, W, t, 0, keep_logits=keep), max(args.steps, 3), warm=args.warmup)
            res['logits_stored' if keep else 'statistics_only'] = {'ms': ms, 'tflops': 2.0 * n * V * d / (ms * 1e-3) / 1e12}
        fa.check_status()
        print(json.dumps({'lm_head_lse': res}))
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- inputs resident in HBM ----------------
    qkv_h, do_h, cos, sin = make_inputs(dtype, dev, seed=1234 + rank)
    qkv_h, do_h = qkv_h.pin_memory(), do_h.pin_memory()
    c2, s2 = cos[:, :D], sin[:, :D]
    qkv_d = qkv_h.to(dev)
    q0, k0, v = views(qkv_d)                   # unrotated q, k: what the qkv projection produces
    do = do_h.to(dev).transpose(1, 2)
    scale = D ** -0.5
    delta = torch.empty((B, H, S), dtype=torch.float32, device=dev)

    def rope_k():                              # K alone through the stand-alone RoPE kernel
        return fa._rope_launch(None, k0, c2, s2, backward=False)[1]

    o, lse, q, k = fa._rope_attn_forward(q0, k0, v, c2, s2, 0.0, True, scale, 0, 'none')

    def step_mode(fuse):
        """Everything from unrotated q,k,v,dO to dq,dk,dv with the RoPE work placed as `fuse` says
        ('none': 5 launches -- RoPE(q,k), forward, dQ, dK/dV, RoPE adjoint; 'fwd': the same 5 with Q rotated
        inside the forward; 'all': 4 launches, the adjoint in the backward kernels' epilogues)."""
        def run():
            o_, lse_, q_, k_ = fa._rope_attn_forward(q0, k0, v, c2, s2, 0.0, True, scale, 0, fuse)
            fa._rope_attn_backward(q_, k_, v, o_, lse_, do, c2, s2, 0.0, True, scale, 0, fuse)
        return run

    step = step_mode(fa.ROPE_FUSION)           # the product's default placement

    def fwd():                                 # forward kernel alone, on rotated inputs
        return fa.attn_forward(q, k, v, 0.0, True, scale, 0)

    def bwd(mode=7):                           # backward kernels alone (mode: 1 delta, 2 dQ, 4 dK/dV)
        return fa.attn_backward(q, k, v, o, lse, do, 0.0, True, scale, 0, mode=mode, delta=delta)

    # ---------------- timed region: K steps, device time, max over ranks ----------------
    sampler = ClockSampler(local)
    sampler.start()                            # before the warm-up: its start-up must not fall into the timed region
    for _ in range(args.warmup):
        step()
    barrier()
    sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(run_steps):
        """Device time of exactly K steps (barrier + synchronize on both sides, max over ranks).  The region
        is taken kRepeats times and all are listed; the FIRST is the result unless it is an outlier (more
        than 1.25x the fastest), in which case the median is.  Later regions run into the power cap and
        are slower, so they are not averaged in; but the GPUs of this pool sit in shared hosts, and a region
        of a few tens of milliseconds is occasionally stretched by seconds by something outside this process
        (seen twice on freshly leased boxes), and one such outlier must not become the result."""
        all_ms = []
        for _ in range(kRepeats):
            barrier()
            e0.record()
            run_steps(args.steps)
            e1.record()
            barrier()
            t_ = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            all_ms.append(float(t_.item()) / args.steps)
        return (all_ms[0] if all_ms[0] <= 1.25 * min(all_ms) else statistics.median(all_ms)), all_ms

    def run_steps(k):
        for _ in range(k):
            step()

    n0 = _native.launch_count()
    ms_step, ms_step_all = timed(run_steps)
    launches = (_native.launch_count() - n0) // kRepeats
    fa.check_status()
    value = world * STEP_FLOPS / (ms_step * 1e-3) / 1e12

    # ---------------- e2e: host buffers, copies inside the timed region ----------------
    outs_h = [torch.empty((B, S, H, D), dtype=dtype).pin_memory() for _ in range(4)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    main_s = torch.cuda.current_stream()
    bufs = [dict(qkv=torch.empty_like(qkv_d), do=torch.empty((B, S, H, D), dtype=dtype, device=dev),
                 ready=torch.cuda.Event(), free=torch.cuda.Event()) for _ in range(2)]
    for b_ in bufs:
        b_['free'].record(main_s)

    def e2e_steps(n):
        pending = []
        for i in range(n):
            b_ = bufs[i % 2]
            with torch.cuda.stream(s_in):
                s_in.wait_event(b_['free'])
                b_['qkv'].copy_(qkv_h, non_blocking=True)
                b_['do'].copy_(do_h, non_blocking=True)
                b_['ready'].record(s_in)
            main_s.wait_event(b_['ready'])
            qq, kk, vv = views(b_['qkv'])
            qq.requires_grad_(True), kk.requires_grad_(True), vv.requires_grad_(True)
            oo = fa.rope_flash_attn(qq, kk, vv, c2, s2, causal=True)
            oo.backward(b_['do'].transpose(1, 2))
            b_['free'].record(main_s)
            res = [oo.detach(), qq.grad, kk.grad, vv.grad]
            done = torch.cuda.Event()
            done.record(main_s)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(outs_h, res):
                    dst.copy_(src.transpose(1, 2) if src.shape[1] == H else src, non_blocking=True)
            pending = res
        main_s.wait_stream(s_out)
        return pending

    e2e_steps(2)
    e2e_ms, e2e_ms_all = timed(e2e_steps)
    clocks = sampler.stop()                # sampled across both timed regions (device-resident and e2e)
    esz = 2
    h2d = (qkv_h.numel() + do_h.numel()) * esz
    d2h = 4 * B * S * H * D * esz
    e2e = {'value': world * STEP_FLOPS / (e2e_ms * 1e-3) / 1e12, 'unit': 'TFLOP/s', 'ms_per_step': e2e_ms,
           'ms_per_step_repeats': e2e_ms_all,
           'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
           'api': 'flash_attn_v100_cuda.rope_flash_attn (autograd fwd+bwd), pinned host buffers'}
    fa.check_status()

    # ---------------- per-kernel timing (alone, burst) and roofline ----------------
    pk = peaks()
    kt = {
        'attn_fwd': (event_time_ms(fwd, 10), FWD_FLOPS),
        'attn_bwd_delta': (event_time_ms(lambda: bwd(1), 10), None),
        'attn_bwd_dq': (event_time_ms(lambda: bwd(2), 10), 0.5 * FWD_FLOPS),     # the dQ GEMM; S, dP are recomputed
        'attn_bwd_dq_with_delta': (event_time_ms(lambda: bwd(3), 10), 0.5 * FWD_FLOPS),   # what a step runs: delta folded in
        'attn_bwd_dkv': (event_time_ms(lambda: bwd(4), 10), 2.0 * FWD_FLOPS),    # S^T, dP^T, dV, dK
        'rope_fwd': (event_time_ms(lambda: fa.rope(q0, k0, c2, s2), 10), None),
        'rope_bwd': (event_time_ms(lambda: fa._rope_launch(q, k, c2, s2, backward=True), 10), None),
        'rope_k_only': (event_time_ms(rope_k, 10), None),
        # the attention kernels with the RoPE work fused in (Q rotation in the forward; adjoint in the epilogues)
        'attn_fwd_rope_fused': (event_time_ms(lambda: fa.attn_forward(q0, k, v, 0.0, True, scale, 0, cos=c2, sin=s2), 10), FWD_FLOPS),
        'attn_bwd_dq_with_delta_rope_fused': (event_time_ms(lambda: fa.attn_backward(q, k, v, o, lse, do, 0.0, True, scale, 0, mode=3, delta=delta, cos=c2, sin=s2), 10), 0.5 * FWD_FLOPS),
        'attn_bwd_dkv_rope_fused': (event_time_ms(lambda: fa.attn_backward(q, k, v, o, lse, do, 0.0, True, scale, 0, mode=4, delta=delta, cos=c2, sin=s2), 10), 2.0 * FWD_FLOPS),
    }
    step_by_fusion = {m: event_time_ms(step_mode(m), 10) for m in ('none', 'fwd', 'all')}
    rope_bytes = 4 * B * H * S * D * esz
    kernels = {}
    for name, (t_ms, fl) in kt.items():
        kernels[name] = {'ms': t_ms}
        if fl:
            kernels[name]['tflops'] = fl / (t_ms * 1e-3) / 1e12
    kernels['rope_fwd']['gbs'] = rope_bytes / (kt['rope_fwd'][0] * 1e-3) / 1e9
    kernels['rope_fwd']['frac_hbm'] = kernels['rope_fwd']['gbs'] / pk['hbm']
    kernels['rope_bwd']['gbs'] = rope_bytes / (kt['rope_bwd'][0] * 1e-3) / 1e9
    kernels['rope_bwd']['frac_hbm'] = kernels['rope_bwd']['gbs'] / pk['hbm']
    kernels['rope_k_only']['gbs'] = rope_bytes / 2 / (kt['rope_k_only'][0] * 1e-3) / 1e9
    kernels['rope_k_only']['frac_hbm'] = kernels['rope_k_only']['gbs'] / pk['hbm']
    # one whole step (unrotated q,k,v,dO -> dq,dk,dv) with the RoPE work placed three ways, and what RoPE
    # costs inside the default step: the step minus the attention kernels on already rotated inputs
    kernels['step_ms_by_rope_fusion'] = dict(step_by_fusion, default=fa.ROPE_FUSION)
    kernels['rope_net_cost_ms'] = step_by_fusion[fa.ROPE_FUSION] - (kt['attn_fwd'][0] + kt['attn_bwd_dq_with_delta'][0] + kt['attn_bwd_dkv'][0])
    kernels['attn_bwd_delta']['gbs'] = (2 * B * H * S * D * esz) / (kt['attn_bwd_delta'][0] * 1e-3) / 1e9
    dom = max(('attn_fwd', 'attn_bwd_dq', 'attn_bwd_dkv'), key=lambda n: kt[n][0])
    ach = kernels[dom]['tflops']
    # DRAM bytes (read + write) of one launch of each kernel at this workload.  NOT measured by this run:
    # constants taken from the ncu capture summarised in profiles/attn_kernels_config2_bf16.md.
    ncu_traffic = NCU_TRAFFIC
    roofline = {'bound': 'tensor', 'kernel': dom, 'achieved': ach, 'peak': pk['bf16_burst'], 'unit': 'TFLOP/s',
                'frac': ach / pk['bf16_burst'], 'traffic': ncu_traffic.get(dom), 'traffic_unit': 'bytes per launch',
                'traffic_source': 'constant from the ncu capture in profiles/attn_kernels_config2_bf16.md (same kernel, same workload), not measured in this run',
                'peak_source': pk['source'] + ' (burst: kernel timed alone)',
                'whole_step_frac_of_sustained': value / world / pk['bf16_sustained'],
                'whole_step_frac_of_nominal_2250': value / world / 2250.0}

    # ---------------- CPU baseline (rank 0, N=1 only) ----------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        stepf, fl = cpu_reference_step(dtype, threads)
        stepf()
        ts, t_start = [], time.perf_counter()
        while len(ts) < 5 and time.perf_counter() - t_start < 20.0:
            ts.append(stepf())
        cpu = {'value': fl / (sum(ts) / len(ts)) / 1e12, 'unit': 'TFLOP/s', 'cores': torch.get_num_threads(),
               'kind': 'port',
               'sample': f'{len(ts)} x one batch element (B=1,H={H},S={S},D={D}), {args.dtype}, eager RoPE + SDPA fwd+bwd'}

    same_box = None
    if rank == 0 and world == 1:
        kernels.update(bandwidth_bench(dev, pk))
        # the reference's own attention call (train.py:1956, F.scaled_dot_product_attention, is_causal) on this
        # GPU with torch's default backend choice: a library baseline on the same box, not part of our path
        import torch.nn.functional as F
        qs, ks, vs = (t.detach().contiguous().requires_grad_(True) for t in (q, k, v))
        dos = do.contiguous()

        def sdpa_step():
            F.scaled_dot_product_attention(qs, ks, vs, is_causal=True).backward(dos)
        t_ms = event_time_ms(sdpa_step, 10, warm=3)
        same_box = {'what': 'torch F.scaled_dot_product_attention fwd+bwd, default backend, same shapes and dtype',
                    'ms_per_step': t_ms, 'tflops': STEP_FLOPS / (t_ms * 1e-3) / 1e12}

    # ---------------- second headline: training tokens/s, data-parallel ----------------
    train = train_strong = train_scaled = None
    if not args.no_train:
        d_ = dist if world > 1 else None
        train = train_bench('100m', 'weak', args, rank, world, dev, d_, pk, warm=3, timed=args.train_steps, base_spp=64)
        if world > 1:      # at one GPU the strong and the weak configuration are the same run
            train_strong = train_bench('100m', 'strong', args, rank, world, dev, d_, pk, warm=3, timed=args.train_steps,
                                       base_spp=64, check=True)
        if not args.no_scaled:
            train_scaled = train_bench('scaled', 'strong', args, rank, world, dev, d_, pk, warm=1, timed=args.scaled_steps,
                                       base_spp=256, check=False)
        if rank == 0 and world == 1 and same_box is not None:
            train['same_box_pytorch'] = same_box_training_baseline(dev)

    if rank == 0:
        _emit(json.dumps({
            'metric': METRIC, 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_step, 'ms_per_step_repeats': ms_step_all,
            'timing': f'{kRepeats} timed regions of exactly {args.steps} steps each, all listed; the first is reported unless it is more than 1.25x the fastest (then the median)',
            'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': args.dtype, 'data': 'synthetic',
            'config': {'workload': WORKLOAD, 'per_gpu': {'B': B, 'H': H, 'S': S, 'D': D}, 'parallelism': f'dp{world}',
                       'l2': 'inputs (201 MB per step) larger than L2', 'flops_per_step_per_gpu': STEP_FLOPS},
            'clocks': clocks, 'e2e': e2e, 'gpu_launches': int(launches), 'roofline': roofline,
            'cpu_baseline': cpu, 'kernels': kernels, 'train': train, 'train_strong': train_strong,
            'train_scaled': train_scaled, 'same_box_pytorch': same_box,
        }))
    if world > 1:
        dist.destroy_process_group()


def _emit(line):
    os.write(_JSON_FD, (line + '\n').encode())


if __name__ == '__main__':
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; keep it for the JSON
    # line alone and send everything else to stderr.
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    main()
