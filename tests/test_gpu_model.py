"""Kernels in the loop: the product model (fused RoPE, FlashAttention, RMSNorm,
chunked CE kernels) against the oracle model (plain PyTorch: SDPA, F.rms_norm,
F.cross_entropy) with identical weights and batches, under the same autocast."""
import numpy as np
import pytest
import torch

from oracle import model as omodel
from tests.golden import inputs

pytestmark = pytest.mark.gpu

CFG = dict(vocab_size=4096, d_model=128, n_heads=2, n_layers=2, d_ff=344, max_seq_len=256)   # head_dim 64


def _models():
    import ulm_model
    prod = ulm_model.DecoderOnlyTransformer(ulm_model.ModelConfig(**CFG)).cuda()
    sd = inputs.seeded_weights(0, CFG)
    missing, unexpected = prod.load_state_dict(sd, strict=False)
    # the seeded set holds the trainable tensors only: the tied head and the RoPE buffers keep their own values
    assert set(missing) <= {'fc_out.weight', 'rope.inv_freq', 'rope.cos_cached', 'rope.sin_cached'} and not unexpected
    orc = omodel.OracleLM(omodel.OracleModelConfig(**CFG))
    inputs.load_seeded_weights_into_oracle(orc)
    return prod, orc.cuda()


def _batch():
    import ulm_data
    rows = inputs.tiny_batch(seed=1, n=8, lo=32, hi=256)
    return ulm_data.collate_pad(rows, eos_id=3, bos_id=2, max_len=256).cuda()


@pytest.mark.parametrize('dtype,tol', [(torch.float16, 1e-4), (torch.bfloat16, 1e-3)])
def test_loss_and_grads_match_oracle_under_autocast(dtype, tol):
    prod, orc = _models()
    ids = _batch()
    with torch.autocast('cuda', dtype=dtype):
        lp = prod.compute_loss(ids, ignore_index=0, chunk_rows=256)
        lo = orc.compute_loss(ids, ignore_index=0, chunk_rows=256)
    # fp32 loss: 1e-4 in fp16; bf16 logits carry 8 mantissa bits, the loss moves by ~1e-3
    assert abs(float(lp) - float(lo)) <= tol, (float(lp), float(lo))
    lp.backward()
    lo.backward()
    pairs = [(prod.embedding.weight.grad, orc.embedding.weight.grad),
             (prod.layers[0].self_attn.wqkv.weight.grad, orc.wqkv[0].weight.grad),
             (prod.layers[1].ff.w2.weight.grad, orc.w2[1].weight.grad),
             (prod.layers[1].norm1.weight.grad, orc.norm1[1].grad),
             (prod.norm.weight.grad, orc.norm_f.grad)]
    for a, b in pairs:
        rel = float((a - b).norm() / b.norm())
        assert rel < (2e-2 if dtype == torch.float16 else 6e-2), rel
    import flash_attn_v100_cuda as fa
    fa.check_status()


def test_dp_step_single_gpu_reduces_loss():
    import ulm_dp
    import ulm_train
    model, preset = ulm_train.build('tiny64', torch.device('cuda'), seed=0)
    opt = ulm_train.make_optimizer(model, lr=3e-3)
    steps = ulm_train.step_batches('tiny64', 16, 8, target_tokens=2048, max_micro_batch=16, n_docs=16, data_seed=3)
    runner = ulm_dp.DataParallelStep(model, opt, samples_per_step=16, autocast_dtype=torch.bfloat16,
                                     ce_chunk_rows=512, device=torch.device('cuda'))
    losses = []
    for _ in range(4):                                   # the same 16 documents every step: loss must fall
        for st in steps[:1]:
            loss, norm, skipped = runner.step(st)
            losses.append(float(loss))
            assert not skipped and float(norm) > 0
    assert losses[-1] < losses[0] - 0.05, losses


def test_checkpointing_matches_plain():
    import ulm_model
    torch.manual_seed(0)
    m = ulm_model.DecoderOnlyTransformer(ulm_model.ModelConfig(**CFG)).cuda()
    ids = _batch()
    out = []
    for ck in (False, True):
        m.use_gradient_checkpointing = ck
        m.zero_grad(set_to_none=True)
        with torch.autocast('cuda', dtype=torch.bfloat16):
            loss = m.compute_loss(ids, chunk_rows=512)
        loss.backward()
        out.append((float(loss), m.layers[0].self_attn.wqkv.weight.grad.clone()))
    assert out[0][0] == out[1][0]
    assert torch.equal(out[0][1], out[1][1])


@pytest.mark.gpu
def test_token_padding_changes_nothing_but_the_row_count():
    """compute_loss pads the flattened token dimension to a multiple of ulm_model.TOKEN_QUANTUM so that the
    library GEMMs see repeating row counts: loss and gradients must equal the unpadded computation (up to the
    GEMMs' choice of algorithm for a different row count)."""
    import ulm_model
    torch.manual_seed(3)
    cfg = ulm_model.ModelConfig(vocab_size=512, d_model=128, n_heads=2, n_layers=2, d_ff=256, max_seq_len=128, dropout=0.0)
    dev = torch.device('cuda')
    m = ulm_model.DecoderOnlyTransformer(cfg).to(dev)
    ids = torch.randint(1, 512, (5, 77), device=dev)
    ids[2, 50:] = 0                                             # padded tail of a shorter document
    outs = []
    old = ulm_model.TOKEN_QUANTUM
    try:
        for q in (0, 1024, 64):
            ulm_model.TOKEN_QUANTUM = q
            for p in m.parameters():
                p.grad = None
            with torch.autocast('cuda', dtype=torch.bfloat16):
                loss = m.compute_loss(ids, ignore_index=0, chunk_rows=128)
            loss.backward()
            outs.append((float(loss), {n: p.grad.clone() for n, p in m.named_parameters()}))
    finally:
        ulm_model.TOKEN_QUANTUM = old
    for loss, grads in outs[1:]:
        assert abs(loss - outs[0][0]) <= 2e-5
        for n, g in grads.items():
            ref = outs[0][1][n]
            assert float((g - ref).norm()) <= 2e-3 * float(ref.norm()) + 1e-7, n
    # the public hidden-state accessor is unpadded
    with torch.no_grad(), torch.autocast('cuda', dtype=torch.bfloat16):
        assert m.forward_hidden(ids).shape == (5, 77, 128)
