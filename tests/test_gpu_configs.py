"""The benchmark configurations at their own sizes: the chunked cross-entropy of
configuration 4 (32768 x 768 hidden, vocabulary 32000, chunks of 4096 rows, bf16), one
micro-batch of the 100M preset under fp16 autocast (configuration 3), and the scaled preset
(d_model 1024, 16 heads, d_ff 2816, bf16, gradient checkpointing) at reduced depth
(configuration 5) -- the product path against the oracle run on the same GPU in the same dtype.
"""
import numpy as np
import pytest
import torch

from oracle import model as omodel, ops
from tests.golden import inputs

pytestmark = pytest.mark.gpu


def relerr(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp(min=1e-30))


@pytest.mark.parametrize('form', ['kept', 'chunked'])
def test_config4_chunked_ce_full_size(form, monkeypatch):
    """hidden [32768, 768] N(0,1) bf16, W [32000, 768] N(0,0.02) bf16, 5 % of the targets ignored
    (id 0), chunks of 4096 rows: loss within 1e-4 of the reference's loop (train.py:2059-2082) run
    in the same dtype on this GPU; dH and dW norm-wise.  Both forms of the op: logits of all rows kept
    in one 16-bit buffer (2.1 GB here), and the chunk-by-chunk form with recomputation."""
    import ulm_ops
    if form == 'chunked':
        monkeypatch.setattr(ulm_ops, 'KEEP_LOGITS_BYTES', 0)
    N, d, V, R = 32768, 768, 32000, 4096
    g = torch.Generator().manual_seed(4)
    h = torch.randn((N, d), generator=g).to(torch.bfloat16).cuda()
    W = (0.02 * torch.randn((V, d), generator=g)).to(torch.bfloat16).cuda()
    t = torch.randint(1, V, (N,), generator=g)
    t[torch.rand(N, generator=g) < 0.05] = 0
    t = t.cuda()
    h1, W1 = h.clone().requires_grad_(True), W.clone().requires_grad_(True)
    loss = ulm_ops.chunked_cross_entropy(h1, W1, t, ignore_index=0, chunk_rows=R, compute_dtype=torch.bfloat16)
    loss.backward()
    h2, W2 = h.clone().requires_grad_(True), W.clone().requires_grad_(True)
    ref = ops.chunked_ce(h2, W2, t, ignore_index=0, chunk_rows=R, logits_dtype=torch.bfloat16)
    ref.backward()
    assert abs(float(loss) - float(ref)) <= 1e-4, (float(loss), float(ref))
    # gradients pass through bf16 dlogits on both sides (ours: one rounding of the fp32 value; the
    # reference: autograd's cast of the fp32 gradient) and bf16 GEMMs with fp32 accumulation
    assert relerr(h1.grad, h2.grad) < 1e-2 and relerr(W1.grad, W2.grad) < 1e-2
    # and against fp32 arithmetic on the same bf16 values, one chunk's worth of rows
    h3, W3 = h[:R].float().requires_grad_(True), W.float().requires_grad_(True)
    l3 = ops.chunked_ce(h3, W3, t[:R], ignore_index=0, chunk_rows=R)
    h4, W4 = h[:R].clone().requires_grad_(True), W.clone().requires_grad_(True)
    l4 = ulm_ops.chunked_cross_entropy(h4, W4, t[:R], ignore_index=0, chunk_rows=R, compute_dtype=torch.bfloat16)
    assert abs(float(l3) - float(l4)) <= 2e-3            # bf16 logits: 8 mantissa bits


def _pair(cfg, dtype, seed=0):
    import ulm_model
    prod = ulm_model.DecoderOnlyTransformer(ulm_model.ModelConfig(**cfg)).cuda()
    sd = inputs.seeded_weights(seed, cfg)
    missing, unexpected = prod.load_state_dict(sd, strict=False)
    assert set(missing) <= {'fc_out.weight', 'rope.inv_freq', 'rope.cos_cached', 'rope.sin_cached'} and not unexpected
    orc = omodel.OracleLM(omodel.OracleModelConfig(**cfg))
    inputs.load_seeded_weights_into_oracle(orc, seed)
    return prod, orc.cuda()


def _micro_batch(n, lo, hi, vocab, max_len, seed):
    import ulm_data
    rng = np.random.default_rng(seed)
    rows = [rng.integers(3, vocab, size=int(L) - 2).astype(np.uint16 if vocab <= 65536 else np.int64)
            for L in rng.integers(lo, hi + 1, size=n)]
    return ulm_data.collate_pad(rows, eos_id=3, bos_id=2, max_len=max_len).cuda()


def _compare(prod, orc, ids, dtype, loss_tol, grad_tol, chunk_rows=4096, loss_scale=1.0):
    with torch.autocast('cuda', dtype=dtype):
        lp = prod.compute_loss(ids, ignore_index=0, chunk_rows=chunk_rows)
        lo = orc.compute_loss(ids, ignore_index=0, chunk_rows=chunk_rows)
    assert abs(float(lp) - float(lo)) <= loss_tol, (float(lp), float(lo))
    # fp16 gradients of a mean over ~30000 tokens underflow without the loss scale the training loop
    # applies (GradScaler's initial 65536, train.py:2219); both sides get the same scale
    (lp * loss_scale).backward()
    (lo * loss_scale).backward()
    last = len(prod.layers) - 1
    pairs = [('embedding', prod.embedding.weight.grad, orc.embedding.weight.grad),
             ('wqkv0', prod.layers[0].self_attn.wqkv.weight.grad, orc.wqkv[0].weight.grad),
             ('wo_last', prod.layers[last].self_attn.wo.weight.grad, orc.wo[last].weight.grad),
             ('w2_last', prod.layers[last].ff.w2.weight.grad, orc.w2[last].weight.grad),
             ('norm1_last', prod.layers[last].norm1.weight.grad, orc.norm1[last].grad),
             ('norm_f', prod.norm.weight.grad, orc.norm_f.grad)]
    for name, a, b in pairs:
        assert relerr(a, b) < grad_tol, (name, relerr(a, b))
    import flash_attn_v100_cuda as fa
    fa.check_status()


def test_config3_100m_preset_micro_batch_fp16():
    """One micro-batch of the 100M preset (d_model 768, 10 layers, 12 heads, d_ff 2048, vocabulary
    32000; 16 rows of up to 2050 tokens = one 32768-token budget) under fp16 autocast: loss within
    1e-4 of the reference's PyTorch path with the same weights, gradients norm-wise."""
    import ulm_train
    cfg = dict(ulm_train.PRESETS['100m']['model'])
    prod, orc = _pair(cfg, torch.float16)
    ids = _micro_batch(16, 1500, 2050, cfg['vocab_size'], cfg['max_seq_len'], seed=11)
    _compare(prod, orc, ids, torch.float16, loss_tol=1e-4, grad_tol=2e-2, loss_scale=65536.0)


def test_config5_scaled_preset_reduced_depth_bf16_checkpointing():
    """The scaled preset's layer shape (d_model 1024, 16 heads, d_ff 2816, vocabulary 32000) at 4 of
    its 24 layers, bf16 autocast, gradient checkpointing on (train.py:2044-2049): loss within 1e-3
    (bf16 logits), gradients norm-wise; and checkpointing changes no bit of the result."""
    import ulm_train
    cfg = dict(ulm_train.PRESETS['scaled']['model'], n_layers=4)
    prod, orc = _pair(cfg, torch.bfloat16)
    prod.use_gradient_checkpointing = True
    prod.train()
    ids = _micro_batch(8, 900, 1300, cfg['vocab_size'], cfg['max_seq_len'], seed=12)
    _compare(prod, orc, ids, torch.bfloat16, loss_tol=1e-3, grad_tol=6e-2)
    g_ck = prod.layers[0].self_attn.wqkv.weight.grad.clone()
    prod.zero_grad(set_to_none=True)
    prod.use_gradient_checkpointing = False
    with torch.autocast('cuda', dtype=torch.bfloat16):
        prod.compute_loss(ids, ignore_index=0, chunk_rows=4096).backward()
    assert torch.equal(g_ck, prod.layers[0].self_attn.wqkv.weight.grad)
