"""The CPU oracle against vectors produced by the reference itself
(tests/golden/make_golden.py).  Integer work must match bit for bit."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import batching, model as omodel, ops
from tests.golden import inputs


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_bucket_boundaries(golden):
    meta, _ = golden
    for m, want in meta['boundaries'].items():
        assert batching.build_bucket_boundaries(int(m)) == want
    b = batching.build_bucket_boundaries(4096)
    assert len(b) == 82 and b[0] == 50 and b[-2] == 4050 and b[-1] == 4096
    for n, want in meta['bucket_of'].items():
        assert batching.bucket_of(b, int(n)) == want


def test_pick_micro_batch(golden):
    meta, _ = golden
    b = batching.build_bucket_boundaries(4096)
    for name, (tt, mmb, spp) in {'c3': (32768, 64, 64), 'c5': (32768, 64, 256),
                                 'ref100m': (12288, 64, 64)}.items():
        got = [batching.pick_micro_batch(x, tt, mmb, spp) for x in b]
        assert got == meta['pick_bs'][name]
    # the sizes quoted for the 100M preset: 4096 -> 8, 2050 -> 14, 1000 -> 32, <=512 -> 64
    assert batching.pick_micro_batch(4096, 32768, 64, 64) == 8
    assert batching.pick_micro_batch(1000, 32768, 64, 64) == 32
    assert batching.pick_micro_batch(500, 32768, 64, 64) == 64


def _counts(lens):
    b = batching.build_bucket_boundaries(4096)
    c = np.zeros(len(b), dtype=np.int64)
    for L in lens:
        c[b.index(batching.bucket_of(b, int(L)))] += 1
    return b, c


@pytest.mark.parametrize('case', sorted(inputs.SAMPLER_CASES))
def test_sampler_stream_bit_exact(golden, case):
    meta, _ = golden
    n_docs, seed_len, spp, tt, seed = inputs.SAMPLER_CASES[case]
    want = meta['sampler'][case]
    b, c = _counts(inputs.log_uniform_lengths(n_docs, seed_len))
    assert sha(c) == want['counts_sha']
    s = batching.TokenBudgetSampler(batching.BucketedCounts(b, c), samples_per_step=spp,
                                    target_tokens=tt, max_micro_batch=64, seed=seed)
    for epoch in (0, 1):
        s.set_epoch(epoch)
        mbs = list(s)
        w = want[str(epoch)]
        assert len(mbs) == w['n_mb']
        assert mbs[0] == w['first_mb'] and mbs[-1] == w['last_mb']
        assert sha(np.array([i for mb in mbs for i in mb], dtype=np.int64)) == w['ids_sha']
        assert sha(np.array([len(mb) for mb in mbs], dtype=np.int64)) == w['sizes_sha']
        # every optimiser step consumes exactly samples_per_step samples (except the last)
        run, steps = 0, []
        for mb in mbs:
            run += len(mb)
            if run >= spp:
                steps.append(run)
                run = 0
        assert all(x == spp for x in steps)
    s.set_epoch(0, skip_samples=3 * spp)
    assert sha(np.array([i for mb in s for i in mb], dtype=np.int64)) == want['resume3_sha']
    s.set_epoch(0, skip_samples=3 * spp + 1)
    with pytest.raises(RuntimeError):
        list(s)


def test_collate(golden):
    meta, arr = golden
    rows = inputs.collate_rows()
    np.testing.assert_array_equal(batching.collate_pad(rows, eos_id=3, bos_id=2, max_len=256),
                                  arr['collate_bos_eos'])
    np.testing.assert_array_equal(batching.collate_pad(rows, eos_id=3, max_len=256),
                                  arr['collate_eos_only'])
    np.testing.assert_array_equal(batching.collate_pad(rows, max_len=256), arr['collate_plain'])
    assert meta['collate_overflow_raises']
    with pytest.raises(RuntimeError):
        batching.collate_pad(rows, eos_id=3, bos_id=2, max_len=34)
    assert batching.collate_pad([]).shape == (0, 0)


def test_rope_tables_bit_exact(golden):
    meta, arr = golden
    for key, want in meta['rope_tables'].items():
        d_model, S, hd = map(int, key.split('_'))
        c, s = ops.rope_tables_head(d_model, S, hd)
        assert sha(c.contiguous().numpy()) == want['cos_sha']
        assert sha(s.contiguous().numpy()) == want['sin_sha']
    c, s = ops.rope_tables_head(768, 4096, 64)
    rows = [0, 1, 2, 63, 1000, 4095]
    np.testing.assert_array_equal(c[rows].numpy(), arr['rope768_cos_rows'])
    np.testing.assert_array_equal(s[rows].numpy(), arr['rope768_sin_rows'])
    # the quirk: 64 distinct angles per position, not 32 pairs
    assert len(set(c[1].tolist())) == 64


@pytest.mark.parametrize('name,dt', [('f16', torch.float16), ('bf16', torch.bfloat16)])
def test_rope_apply_bit_exact(golden, name, dt):
    _, arr = golden
    q, k = inputs.rope_qk()
    c, s = ops.rope_tables_head(768, q.shape[2], 64)
    qo, ko = ops.apply_rope(q.to(dt), k.to(dt), c, s, out_dtype=dt)
    np.testing.assert_array_equal(qo.view(torch.int16).numpy(), arr[f'rope_q_{name}'])
    np.testing.assert_array_equal(ko.view(torch.int16).numpy(), arr[f'rope_k_{name}'])
    gq, gk = inputs.rope_grads()
    dq, dk = ops.rope_backward(gq.to(dt), gk.to(dt), c, s)
    # autograd's adjoint sums the two products in the same order; allow 1 ulp of fp32
    np.testing.assert_allclose(dq.numpy(), arr[f'rope_dq_{name}'], rtol=2e-7, atol=1e-7)
    np.testing.assert_allclose(dk.numpy(), arr[f'rope_dk_{name}'], rtol=2e-7, atol=1e-7)


def test_attention_matches_reference_sdpa(golden):
    _, arr = golden
    q, k, v, do = inputs.attn_small()
    o, lse = ops.attention_explicit(q, k, v)
    np.testing.assert_allclose(o.numpy(), arr['attn_o'], rtol=1e-5, atol=2e-6)
    dq, dk, dv, _ = ops.attention_bwd_explicit(q, k, v, o, lse, do)
    for got, key in ((dq, 'attn_dq'), (dk, 'attn_dk'), (dv, 'attn_dv')):
        np.testing.assert_allclose(got.numpy(), arr[key], rtol=1e-4, atol=2e-5)
    # lse really is the log-sum-exp of the masked scaled scores
    s = (q @ k.transpose(-1, -2)) * 64 ** -0.5
    s = s.masked_fill(torch.ones(150, 150, dtype=torch.bool).triu(1), float('-inf'))
    np.testing.assert_allclose(lse.numpy(), torch.logsumexp(s, -1).numpy(), rtol=1e-6, atol=1e-6)


def test_rmsnorm(golden):
    _, arr = golden
    x, w, dy = inputs.rms_small()
    np.testing.assert_allclose(ops.rms_norm(x, w).numpy(), arr['rms_y'], rtol=1e-6, atol=1e-6)
    dx, dw = ops.rms_norm_backward(x, w, dy)
    np.testing.assert_allclose(dx.numpy(), arr['rms_dx'], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(dw.numpy(), arr['rms_dw'], rtol=1e-5, atol=1e-5)


def test_chunked_ce(golden):
    meta, arr = golden
    h, W, t = inputs.ce_small()
    h.requires_grad_(True), W.requires_grad_(True)
    loss = ops.chunked_ce(h, W, t, ignore_index=0, chunk_rows=64)
    assert abs(float(loss) - meta['ce_loss']) <= 1e-6
    loss.backward()
    np.testing.assert_allclose(h.grad.numpy(), arr['ce_dh'], rtol=1e-5, atol=1e-8)
    np.testing.assert_allclose(W.grad.numpy(), arr['ce_dw'], rtol=1e-5, atol=1e-8)
    # the per-row pieces the kernels are checked against add up to the same loss
    lse, loss_sum, dl = ops.ce_rows(h.detach() @ W.detach().t(), t)
    n_tok = int((t != 0).sum())
    assert abs(float(loss_sum) / n_tok - meta['ce_loss']) <= 1e-5
    np.testing.assert_allclose((dl @ W.detach() / n_tok).numpy(), arr['ce_dh'], rtol=1e-4, atol=1e-7)


def test_tiny_model_step(golden):
    meta, arr = golden
    torch.set_num_threads(1)
    m = omodel.OracleLM(omodel.OracleModelConfig(**inputs.TINY_MODEL))
    inputs.load_seeded_weights_into_oracle(m)
    ids = torch.from_numpy(batching.collate_pad(inputs.tiny_batch(), eos_id=3, bos_id=2, max_len=256))
    assert sha(ids.numpy()) == meta['tiny_ids_sha']
    loss = m.compute_loss(ids, ignore_index=0, chunk_rows=256)
    assert abs(float(loss) - meta['tiny_loss']) <= 1e-5
    loss.backward()
    np.testing.assert_allclose(m.embedding.weight.grad[:8].numpy(), arr['tiny_emb_grad_rows'],
                               rtol=1e-3, atol=1e-7)
    want = meta['tiny_grad_norms']
    assert abs(float(m.norm_f.grad.norm()) - want['norm.weight']) <= 1e-4 * want['norm.weight']
    assert abs(float(m.wqkv[1].weight.grad.norm()) - want['layers.1.self_attn.wqkv.weight']) \
        <= 1e-4 * want['layers.1.self_attn.wqkv.weight']


def test_dropout_hash_properties():
    # no reference vector exists for the hash (it lives in CUDA only): check the
    # restatement's own invariants -- determinism, keep rate, p=0 keeps all.
    m = ops.dropout_keep_mask(1234, 256, 256, 5, 0.1)
    assert m.dtype == np.bool_ and m.shape == (256, 256)
    assert abs(m.mean() - 0.9) < 0.01
    assert np.array_equal(m, ops.dropout_keep_mask(1234, 256, 256, 5, 0.1))
    assert not np.array_equal(m, ops.dropout_keep_mask(1235, 256, 256, 5, 0.1))
    assert ops.dropout_keep_mask(1, 8, 8, 0, 0.0).all()
    # one value worked by hand from the formula
    h = (7 * 0x9E3779B1) & 0xFFFFFFFF
    h ^= (3 * 0x85EBCA6B) & 0xFFFFFFFF
    h ^= (5 * 0xC2B2AE35) & 0xFFFFFFFF
    h ^= (2 * 0x27D4EB2F) & 0xFFFFFFFF
    h ^= h >> 16; h = (h * 0x7FEB352D) & 0xFFFFFFFF
    h ^= h >> 15; h = (h * 0x846CA68B) & 0xFFFFFFFF
    h ^= h >> 16
    assert bool(ops.dropout_keep_mask(7, 3, 5, 1, 0.5)[2, 4]) == ((h >> 8) / 16777216.0 >= 0.5)


def test_dropout_hash_matches_the_reference_fixture(golden):
    """Keep-mask blocks and hash values written by tests/golden/make_golden.py from the reference's
    own source (csrc/flash_attn_v100/fa_common.cuh:21-38, compiled for the host): the numpy
    restatement must reproduce every bit."""
    meta, arrays = golden
    for x, want in meta['hash_u32'].items():
        assert ops.hash_u32(int(x)) == want
    for i, c in enumerate(meta['dropout_keep_cases']):
        n = c['nrows'] * c['ncols']
        want = np.unpackbits(arrays[f'dropout_keep_{i}'])[:n].reshape(c['nrows'], c['ncols']).astype(bool)
        assert int(want.sum()) == c['kept']
        full = ops.dropout_keep_mask(c['seed'], c['row0'] + c['nrows'], c['col0'] + c['ncols'], c['bh'], c['p'])
        assert np.array_equal(full[c['row0']:, c['col0']:], want), c


def test_dropout_hash_matches_the_compiled_reference_when_present():
    """Where oracle/_ref has been built (it is wherever the reference checkout is available), compare
    the restatement with the reference's code directly on fresh random cases."""
    from oracle import ref_build
    lib = ref_build.load_ref()
    if lib is None:
        pytest.skip('oracle/_ref not built on this machine')
    rng = np.random.default_rng(0)
    for _ in range(20):
        seed, bh = int(rng.integers(0, 2 ** 32)), int(rng.integers(0, 4096))
        p = float(rng.choice([0.0, 0.05, 0.1, 0.5, 0.99]))
        got = ops.dropout_keep_mask(seed, 70, 90, bh, p)
        assert np.array_equal(got, ref_build.ref_keep_block(lib, seed, bh, p, 0, 70, 0, 90))
    for x in rng.integers(0, 2 ** 32, size=50):
        assert ops.hash_u32(int(x)) == lib.ref_hash_u32(int(x))


def test_product_rope_tables_bit_exact(golden):
    """The product's own table builder (ulm_model.rope_tables, not the oracle's twin) against the
    reference's RotaryPositionalEmbedding hashes."""
    import hashlib
    import ulm_model
    meta, arrays = golden

    def sha(a):
        return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    for key, want in meta['rope_tables'].items():
        d_model, S, hd = (int(x) for x in key.split('_'))
        c, s = ulm_model.rope_tables(d_model, S)
        assert sha(c[:, :hd].contiguous().numpy()) == want['cos_sha'] and sha(s[:, :hd].contiguous().numpy()) == want['sin_sha']


def test_product_model_state_dict_is_the_references(golden):
    """Names, shapes and dtypes of every state_dict entry equal the reference model's (parameters and
    the three persistent RoPE buffers), the RoPE buffers carry the same bits, and a state_dict with
    the reference's layout loads with strict=True."""
    import hashlib
    import ulm_model
    meta, _ = golden
    m = ulm_model.DecoderOnlyTransformer(ulm_model.ModelConfig(**inputs.TINY64_MODEL))
    sd = m.state_dict()
    want = meta['state_dict_tiny64']
    assert {k: [list(v.shape), str(v.dtype)] for k, v in sd.items()} == want
    for k, h in meta['state_dict_tiny64_rope_sha'].items():
        assert hashlib.sha256(np.ascontiguousarray(sd[k].numpy()).tobytes()).hexdigest() == h, k
    ref_like = {k: torch.zeros(shape, dtype=getattr(torch, dt.split('.')[1])) for k, (shape, dt) in want.items()}
    m.load_state_dict(ref_like, strict=True)
