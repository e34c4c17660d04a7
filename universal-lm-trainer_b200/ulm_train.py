"""Training-step harness mirroring the reference's loop (train.py:2134-2424) on
top of the data-parallel step: builds a preset model, draws token-budget
micro-batches from a synthetic bucketed corpus and runs optimiser steps.

Presets follow the benchmark configurations (not the reference's configs/*.json,
which use other d_ff / vocab / budget values):
  100m    d_model 768, 10 layers, 12 heads, d_ff 2048, vocab 32000, fp16 autocast
  scaled  d_model 1024, 24 layers, 16 heads, d_ff 2816, vocab 32000, bf16, checkpointing
"""
import torch

import ulm_data
import ulm_dp
import ulm_model

PRESETS = {
    '100m': dict(model=dict(vocab_size=32000, d_model=768, n_heads=12, n_layers=10, d_ff=2048, max_seq_len=4096),
                 dtype=torch.float16, loss_scale=65536.0, checkpointing=False),
    'scaled': dict(model=dict(vocab_size=32000, d_model=1024, n_heads=16, n_layers=24, d_ff=2816, max_seq_len=4096),
                   dtype=torch.bfloat16, loss_scale=None, checkpointing=True),
    'tiny64': dict(model=dict(vocab_size=4096, d_model=128, n_heads=2, n_layers=2, d_ff=344, max_seq_len=256),
                   dtype=torch.bfloat16, loss_scale=None, checkpointing=False),
}
BOS, EOS, PAD = 2, 3, 0


def build(preset, device, seed=0):
    p = PRESETS[preset]
    torch.manual_seed(seed)
    cfg = ulm_model.ModelConfig(**p['model'], dropout=0.0, use_gradient_checkpointing=p['checkpointing'])
    model = ulm_model.DecoderOnlyTransformer(cfg).to(device)
    model.train()
    return model, p


def make_optimizer(model, lr=3e-4, weight_decay=0.01):
    # train.py:2188-2192
    return torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=weight_decay, betas=(0.9, 0.95),
                             fused=next(model.parameters()).is_cuda)


def step_sources(preset, samples_per_step, n_steps, target_tokens=32768, max_micro_batch=64,
                 n_docs=None, data_seed=0, sampler_seed=42):
    """``n_steps`` zero-argument callables, each of which draws the documents of one optimiser
    step and collates its micro-batches (train.py:1691-1747) when called -- the form
    `ulm_dp.InputPipeline` takes, so that the collate work runs on its worker thread."""
    cfg = PRESETS[preset]['model']
    n_docs = n_docs or max(20000, samples_per_step * (n_steps + 1))
    ds = ulm_data.SyntheticBucketDataset(n_docs, cfg['max_seq_len'], vocab=cfg['vocab_size'], seed=data_seed,
                                         lo=min(64, cfg['max_seq_len'] // 4))
    sampler = ulm_data.TokenBudgetBatchSampler(ds, samples_per_step=samples_per_step, target_tokens=target_tokens,
                                               max_micro_batch=max_micro_batch, seed=sampler_seed)
    out = []
    for group in sampler.steps():
        if len(out) == n_steps:
            break
        out.append(lambda group=group: [ulm_data.collate_pad([ds[i] for i in mb], eos_id=EOS, bos_id=BOS,
                                                             max_len=cfg['max_seq_len']) for mb in group])
    return out


def step_batches(preset, samples_per_step, n_steps, target_tokens=32768, max_micro_batch=64,
                 n_docs=None, data_seed=0, sampler_seed=42):
    """Collated micro-batches (host int64 tensors) for ``n_steps`` optimiser steps."""
    cfg = PRESETS[preset]['model']
    # a corpus large enough that buckets are well filled and micro-batches reach their budgeted size
    n_docs = n_docs or max(20000, samples_per_step * (n_steps + 1))
    ds = ulm_data.SyntheticBucketDataset(n_docs, cfg['max_seq_len'], vocab=cfg['vocab_size'], seed=data_seed,
                                         lo=min(64, cfg['max_seq_len'] // 4))
    sampler = ulm_data.TokenBudgetBatchSampler(ds, samples_per_step=samples_per_step, target_tokens=target_tokens,
                                               max_micro_batch=max_micro_batch, seed=sampler_seed)
    out = []
    for group in sampler.steps():
        if len(out) == n_steps:
            break
        out.append([ulm_data.collate_pad([ds[i] for i in mb], eos_id=EOS, bos_id=BOS,
                                         max_len=cfg['max_seq_len']).pin_memory()
                    if torch.cuda.is_available() else
                    ulm_data.collate_pad([ds[i] for i in mb], eos_id=EOS, bos_id=BOS, max_len=cfg['max_seq_len'])
                    for mb in group])
    return out


def token_counts(step):
    real = sum(int((mb != PAD).sum()) for mb in step)
    padded = sum(mb.numel() for mb in step)
    return real, padded


def flops_per_token(preset, seq_len):
    """Model FLOPs per token, forward + backward: 3 x (linears + lm head) plus
    3.5 x the causal attention matmuls at this length."""
    m = PRESETS[preset]['model']
    d, L, ff, V = m['d_model'], m['n_layers'], m['d_ff'], m['vocab_size']
    lin = 2 * L * (4 * d * d + 3 * d * ff)
    head = 2 * d * V
    attn = 2 * seq_len * d * L
    return 3.0 * (lin + head) + 3.5 * attn
