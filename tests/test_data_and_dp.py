"""Host-side batch shaping against the reference's golden vectors, and the
data-parallel identity on CPU ranks (gloo): the sum over ranks of the sharded
step equals the single-process reference step."""
import hashlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ulm_data
import ulm_dp
from oracle import batching, model as omodel
from tests.golden import inputs


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_buckets_match_reference(golden):
    meta, _ = golden
    for m, want in meta['boundaries'].items():
        assert ulm_data.build_bucket_boundaries(int(m)) == want
    fb = ulm_data.FastBucket(ulm_data.build_bucket_boundaries(4096))
    for n, want in meta['bucket_of'].items():
        assert fb.get_bucket(int(n)) == want
    lens = np.array([int(n) for n in meta['bucket_of']])
    got = [fb.boundaries[i] for i in fb.bucket_indices(lens)]
    assert got == [meta['bucket_of'][str(n)] for n in lens]
    for name, (tt, mmb, spp) in {'c3': (32768, 64, 64), 'c5': (32768, 64, 256), 'ref100m': (12288, 64, 64)}.items():
        assert [ulm_data.TokenBudgetBatchSampler._pick_bs(b, tt, mmb, spp) for b in fb.boundaries] == meta['pick_bs'][name]


@pytest.mark.parametrize('case', sorted(inputs.SAMPLER_CASES))
def test_sampler_bit_exact(golden, case):
    meta, _ = golden
    n_docs, seed_len, spp, tt, seed = inputs.SAMPLER_CASES[case]
    want = meta['sampler'][case]
    ds = ulm_data.SyntheticBucketDataset(n_docs, 4096, seed=seed_len)
    assert sha(ds.counts) == want['counts_sha']
    s = ulm_data.TokenBudgetBatchSampler(ds, samples_per_step=spp, target_tokens=tt, max_micro_batch=64, seed=seed)
    for epoch in (0, 1):
        s.set_epoch(epoch)
        mbs = list(s)
        w = want[str(epoch)]
        assert len(mbs) == w['n_mb'] and mbs[0] == w['first_mb'] and mbs[-1] == w['last_mb']
        assert sha(np.array([i for mb in mbs for i in mb], dtype=np.int64)) == w['ids_sha']
        assert sha(np.array([len(mb) for mb in mbs], dtype=np.int64)) == w['sizes_sha']
    s.set_epoch(0, skip_samples=3 * spp)
    assert sha(np.array([i for mb in s for i in mb], dtype=np.int64)) == want['resume3_sha']
    s.set_epoch(0)
    steps = list(s.steps())
    assert all(sum(len(mb) for mb in g) == spp for g in steps[:-1])
    # every micro-batch is drawn from one bucket and respects the token budget
    fb = ulm_data.FastBucket(ds.boundaries)
    for g in steps[:20]:
        for mb in g:
            bs = {fb.get_bucket(int(ds.lengths[i])) for i in mb}
            assert len(bs) == 1 and len(mb) * bs.pop() <= max(tt, 4096)
    # identical to the oracle's stream as well
    o = batching.TokenBudgetSampler(batching.BucketedCounts(ds.boundaries, ds.counts), spp, tt, 64, seed)
    assert list(o) == list(s)


def test_collate_matches_reference(golden):
    meta, arr = golden
    rows = inputs.collate_rows()
    np.testing.assert_array_equal(ulm_data.collate_pad(rows, eos_id=3, bos_id=2, max_len=256).numpy(), arr['collate_bos_eos'])
    np.testing.assert_array_equal(ulm_data.collate_pad(rows, eos_id=3, max_len=256).numpy(), arr['collate_eos_only'])
    np.testing.assert_array_equal(ulm_data.collate_pad(rows, max_len=256).numpy(), arr['collate_plain'])
    with pytest.raises(RuntimeError):
        ulm_data.collate_pad(rows, eos_id=3, bos_id=2, max_len=34)
    assert tuple(ulm_data.collate_pad([]).shape) == (0, 0)


def test_row_sharding_covers_every_row_once():
    for n in (1, 2, 3, 7, 8, 14, 64):
        for world in (1, 2, 3, 4, 8):
            got = []
            for r in range(world):
                lo, hi = ulm_dp.shard_bounds(n, r, world)
                got += list(range(lo, hi))
            assert got == list(range(n))
            sizes = [ulm_dp.shard_bounds(n, r, world)[1] - ulm_dp.shard_bounds(n, r, world)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    # the step plan: every row of every micro-batch exactly once, contiguous chunks, balanced loads
    def check_plan(shapes, world, bound):
        plan = ulm_dp.plan_step(shapes, world)
        assert len(plan) == world and plan == ulm_dp.plan_step(shapes, world)
        seen = {m: [] for m in range(len(shapes))}
        load = []
        for units in plan:
            load.append(sum((hi - lo) * ulm_dp.row_cost(shapes[m][1]) for m, lo, hi in units))
            for m, lo, hi in units:
                assert 0 <= lo < hi <= shapes[m][0]
                seen[m] += list(range(lo, hi))
        for m, (n, _) in enumerate(shapes):
            assert sorted(seen[m]) == list(range(n))
        # balanced GPU work wherever the GPU work, not the launching, is what a rank's time consists of
        if sum(n for n, _ in shapes) >= 2 * world and sum(load) / world >= 3 * ulm_dp.DEFAULT_COST.host:
            assert max(load) <= bound * sum(load) / world, (shapes, world, load)
        # the estimate the planner minimises: GPU time of the calls, or their launch time if that is longer
        cost = ulm_dp.DEFAULT_COST
        est = [cost.load([cost.call + (hi - lo) * cost.row(shapes[m][1]) for m, lo, hi in units]) for units in plan]
        naive = [cost.load([cost.call + (b - a) * cost.row(L) for (n, L) in shapes
                            for a, b in [ulm_dp.shard_bounds(n, r, world)] if b > a]) for r in range(world)]
        assert max(est) <= max(naive) * 1.0001, (shapes, world, est, naive)      # never worse than splitting every micro-batch evenly
        return plan
    few_large = [(64 * 8, 512), (14 * 8, 2052), (8 * 8, 4096)]            # weak scaling at 8 GPUs: 3 micro-batches, 8x rows
    many = [(8, 4096), (14, 2052), (32, 1000), (64, 300), (16, 2000), (8, 4000), (21, 1500), (64, 500), (10, 3000),
            (42, 750), (8, 4050), (64, 400), (12, 2600)]                  # strong scaling: 13 micro-batches of one budget
    for world in (1, 2, 3, 4, 8):
        check_plan(few_large, world, 1.08)
        plan = check_plan(many, world, 1.10)
        if world == 8:      # whole micro-batches or large chunks, not 13 slivers per rank
            assert max(len(u) for u in plan) <= 5
        check_plan([(14, 2052), (8, 4096), (3, 600), (64, 300), (1, 80)], world, 1.35)
        check_plan([(1, 100)], world, 99.0)
    mb = torch.tensor([[2, 5, 6, 3, 0, 0], [2, 7, 3, 0, 0, 0], [2, 8, 9, 4, 5, 3]])
    assert ulm_dp.local_rows(mb, 0, 2).tolist() == [[2, 5, 6, 3]]
    assert ulm_dp.local_rows(mb, 1, 2).shape == (2, 6)
    assert ulm_dp.local_rows(mb[:1], 0, 2) is None and ulm_dp.local_rows(mb[:1], 1, 2).shape == (1, 4)
    # a step with fewer rows than ranks leaves some ranks without work; the others still cover every row
    work = [ulm_dp.prepare_step([mb[:1]], r, 4, 8) for r in range(4)]
    assert sum(len(w) for w in work) == 1


# ---------------------------------------------------------------- gloo ranks ----
def _torch_grad_post(flat, inv_scale, out2):
    """What the CUDA post-pass computes, in torch, for the CPU ranks of this test."""
    flat.mul_(inv_scale[0])
    out2[0] += flat.double().pow(2).sum().float()
    out2[1] = 0.0 if bool(torch.isfinite(flat).all()) else 1.0
    return out2


def _tiny_step_batches(seed=3):
    rng = np.random.default_rng(seed)
    mbs = []
    for n, hi in ((5, 40), (2, 90), (1, 30)):           # 8 samples per step; one micro-batch has fewer rows than ranks
        rows = [rng.integers(3, 512, size=int(L)).astype(np.int64) for L in rng.integers(8, hi, size=n)]
        mbs.append(ulm_data.collate_pad(rows, eos_id=3, bos_id=2, max_len=128))
    return mbs


def _make_model():
    torch.manual_seed(0)
    return omodel.OracleLM(omodel.OracleModelConfig(vocab_size=512, d_model=64, n_heads=2, n_layers=2,
                                                    d_ff=96, max_seq_len=128))


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    torch.set_num_threads(1)
    m = _make_model()
    opt = torch.optim.SGD(m.parameters(), lr=0.0)
    step = ulm_dp.DataParallelStep(m, opt, samples_per_step=8, rank=rank, world=world, max_grad_norm=None,
                                   ce_chunk_rows=64, grad_post=_torch_grad_post, loss_scale=1024.0,
                                   bucket_bytes=8192,   # many buckets: exercises the in-order overlapped all-reduce
                                   device=torch.device('cpu'))
    loss, norm, skipped = step.step(_tiny_step_batches())
    if rank == 0:
        torch.save(dict(flat=step.grads.flat.clone(), loss=float(loss), norm=float(norm), skipped=skipped),
                   os.path.join(out_dir, f'dp{world}.pt'))
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


@pytest.mark.parametrize('world', [1, 2, 3, 4, 8])
def test_dp_step_equals_single_process_reference(tmp_path, world):
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = torch.load(os.path.join(tmp_path, f'dp{world}.pt'))
    torch.set_num_threads(1)
    ref = _make_model()
    ref_loss = omodel.step_loss_and_grads(ref, _tiny_step_batches(), samples_per_step=8, chunk_rows=64)
    want = ulm_dp.FlatGrads  # layout helper only
    uniq, seen = [], set()
    for p in ref.parameters():
        if id(p) not in seen:
            seen.add(id(p))
            uniq.append(p)
    off = 0
    for p in uniq:
        g = got['flat'][off:off + p.numel()].view_as(p)
        assert float((g - p.grad).norm() / p.grad.norm().clamp(min=1e-12)) < 1e-5
        off += (p.numel() + 3) // 4 * 4
    assert abs(got['loss'] - ref_loss) <= 1e-5
    total = torch.sqrt(sum((p.grad.double() ** 2).sum() for p in uniq))
    assert abs(got['norm'] - float(total)) <= 1e-4 * float(total)
    assert got['skipped'] is False


def test_dynamic_loss_scale_backs_off_and_skips():
    torch.manual_seed(0)
    m = _make_model()
    before = [p.detach().clone() for p in m.parameters()]
    opt = torch.optim.SGD(m.parameters(), lr=0.1)

    def post_with_overflow(flat, inv_scale, out2):
        flat[0] = float('inf')
        return _torch_grad_post(flat, inv_scale, out2)
    step = ulm_dp.DataParallelStep(m, opt, samples_per_step=8, max_grad_norm=1.0, ce_chunk_rows=64,
                                   grad_post=post_with_overflow, loss_scale=1024.0, dynamic_loss_scale=True,
                                   growth_interval=2, device=torch.device('cpu'))
    _, _, skipped = step.step(_tiny_step_batches())
    assert skipped and step.scale == 512.0
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))     # the overflowing step changed nothing
    step.grad_post = _torch_grad_post
    for _ in range(2):
        _, _, skipped = step.step(_tiny_step_batches())
        assert not skipped
    assert step.scale == 1024.0                                                # two clean steps: grown back
    assert any(not torch.equal(a, b) for a, b in zip(before, m.parameters()))


def test_input_pipeline_yields_what_prepare_step_makes():
    steps = [_tiny_step_batches(seed=s) for s in (1, 2, 3)]
    for rank, world in ((0, 1), (1, 2), (2, 3)):
        got = list(ulm_dp.InputPipeline(steps, rank, world, samples_per_step=8, pin=False,
                                        mode='thread' if rank == 0 else 'process'))
        assert len(got) == 3
        for st, work in zip(steps, got):
            want = ulm_dp.prepare_step(st, rank, world, 8)
            assert len(work) == len(want)
            for (r1, w1, n1), (r2, w2, n2) in zip(work, want):
                assert torch.equal(r1, r2) and w1 == w2 and n1 == n2
    # token counts are global (all ranks' rows), weights n / samples_per_step
    mbs = steps[0]
    w0 = ulm_dp.prepare_step(mbs, 0, 2, 8)
    units = ulm_dp.plan_step([(mb.shape[0], mb.shape[1]) for mb in mbs], 2)[0]
    assert [w for _, w, _ in w0] == [mbs[m].shape[0] / 8 for m, _, _ in units]
    assert [n for _, _, n in w0] == [float((mbs[m][:, 1:] != 0).sum()) for m, _, _ in units]

    def boom():
        raise ValueError('collate failed')
    for mode in ('thread', 'process'):
        with pytest.raises(RuntimeError, match='collate failed'):
            list(ulm_dp.InputPipeline([boom], 0, 1, samples_per_step=8, pin=False, mode=mode))


# ------------------------------------------------- a rank leaves between steps ----
def _leaving_rank_main(rank, world, port, out_dir):
    """Rank `world-1` exits after the first step; the others must get an error on the host
    instead of waiting forever: from the heartbeat (before anything is launched) when it is on,
    else from the process group's timeout on the gradient all-reduce."""
    import datetime
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    torch.set_num_threads(1)
    use_hb = out_dir.endswith('hb')
    m = _make_model()
    opt = torch.optim.SGD(m.parameters(), lr=0.0)
    hb = ulm_dp.StepHeartbeat(dist.distributed_c10d._get_default_store(), rank, world, timeout_s=3.0) if use_hb else None
    step = ulm_dp.DataParallelStep(m, opt, samples_per_step=8, rank=rank, world=world, max_grad_norm=None,
                                   ce_chunk_rows=64, grad_post=_torch_grad_post, device=torch.device('cpu'),
                                   heartbeat=hb)
    step.step(_tiny_step_batches())
    dist.barrier()
    if rank == world - 1:
        os._exit(0)                                       # gone between steps, nothing of its own in flight
    outcome = 'no error'
    try:
        step.step(_tiny_step_batches())
    except ulm_dp.RankFailure as e:
        outcome = f'RankFailure: {e}'
    except Exception as e:  # noqa: BLE001 - gloo reports a lost peer or an expired timeout as RuntimeError
        outcome = f'{type(e).__name__}: {e}'
    with open(os.path.join(out_dir, f'rank{rank}.txt'), 'w') as f:
        f.write(outcome)
    os._exit(0)                                           # do not try to tear the broken group down


@pytest.mark.parametrize('mode', ['pg', 'hb'])
def test_survivors_surface_an_error_when_a_rank_leaves(tmp_path, mode):
    out = tmp_path / mode
    out.mkdir()
    world = 3
    mp.spawn(_leaving_rank_main, args=(world, _free_port(), str(out)), nprocs=world, join=True)
    for rank in range(world - 1):
        text = (out / f'rank{rank}.txt').read_text()
        assert text != 'no error', text
        if mode == 'hb':
            assert text.startswith('RankFailure'), text


def test_cost_model_scales_with_the_model_and_prefers_few_calls_when_launch_bound():
    """`CostModel.for_model`: the 100M preset reproduces the measured constants, a wider / deeper / checkpointed
    model costs more per token and per call; `cost_model_of` reads them off a module; and where the GPU work of
    a step is small against the host's cost of launching a call, the planner gives every rank one call."""
    import ulm_model
    c = ulm_dp.CostModel.for_model(95.4e6, 768, 10)
    assert c == ulm_dp.DEFAULT_COST
    assert abs(c.a - 8.1e-4) < 2e-5 and abs(c.b - 9.2e-8) < 2e-9 and c.call == 1.5 and c.host == 20.0
    big = ulm_dp.CostModel.for_model(341e6, 1024, 24, checkpointing=True)
    assert big.a > 3 * c.a and big.b > 3 * c.b and big.host > 3 * c.host
    assert abs(big.a - 3.3e-3) < 1e-4 and abs(big.b - 3.9e-7) < 1e-8          # the second measured preset
    cfg = ulm_model.ModelConfig(vocab_size=1000, d_model=128, n_heads=2, n_layers=3, d_ff=256, max_seq_len=64, dropout=0.0)
    m = ulm_model.DecoderOnlyTransformer(cfg)
    got = ulm_dp.cost_model_of(m)
    n_params = sum(p.numel() for p in m.parameters())                          # tied head: every parameter multiplies
    assert got == ulm_dp.CostModel.for_model(float(n_params), 128, 3, False)
    assert ulm_dp.cost_model_of(torch.nn.Linear(4, 4)) == ulm_dp.DEFAULT_COST
    # 64 short samples over 8 ranks: ~10 ms of GPU work per rank against 20 ms per launched call
    shapes = [(27, 300), (14, 520), (15, 450), (8, 1000)]
    plan = ulm_dp.plan_step(shapes, 8)
    assert max(len(u) for u in plan) == 1
    # a large step is balanced on GPU work instead
    plan = ulm_dp.plan_step([(64, 4096)] * 12, 4)
    load = [sum((hi - lo) * ulm_dp.row_cost(4096) for m_, lo, hi in u) for u in plan]
    assert max(load) <= 1.02 * sum(load) / 4
