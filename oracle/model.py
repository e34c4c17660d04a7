"""Oracle restatement of the reference's decoder-only model and its per-step
loss weighting, in plain PyTorch (no custom kernels).  Used as the parity
target for the tiny CPU config and for the data-parallel identity tests.

Test infrastructure: see the package docstring.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


@dataclass
class OracleModelConfig:  # mirrors train.py:725-737 (ModelConfig), used fields only
    vocab_size: int = 4096
    d_model: int = 128
    n_heads: int = 4
    n_layers: int = 2
    d_ff: int = 344
    max_seq_len: int = 256
    tie_weights: bool = True


class OracleLM(nn.Module):
    """train.py:1920-2082 with dropout 0: pre-norm blocks of
    RMSNorm -> fused-QKV attention with the d_model-wide RoPE table -> residual,
    RMSNorm -> SwiGLU -> residual; final RMSNorm; tied lm head; chunked CE."""

    def __init__(self, cfg: OracleModelConfig):
        super().__init__()
        self.cfg = cfg
        d, L = cfg.d_model, cfg.n_layers
        self.embedding = nn.Embedding(cfg.vocab_size, d)
        self.wqkv = nn.ModuleList(nn.Linear(d, 3 * d, bias=False) for _ in range(L))
        self.wo = nn.ModuleList(nn.Linear(d, d, bias=False) for _ in range(L))
        self.w1 = nn.ModuleList(nn.Linear(d, cfg.d_ff, bias=False) for _ in range(L))
        self.w3 = nn.ModuleList(nn.Linear(d, cfg.d_ff, bias=False) for _ in range(L))
        self.w2 = nn.ModuleList(nn.Linear(cfg.d_ff, d, bias=False) for _ in range(L))
        self.norm1 = nn.ParameterList(nn.Parameter(torch.ones(d)) for _ in range(L))
        self.norm2 = nn.ParameterList(nn.Parameter(torch.ones(d)) for _ in range(L))
        self.norm_f = nn.Parameter(torch.ones(d))
        self.fc_out = nn.Linear(d, cfg.vocab_size, bias=False)
        if cfg.tie_weights:
            self.fc_out.weight = self.embedding.weight
        for m in self.modules():  # train.py:2015-2022
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)
        cos, sin = ops.rope_tables(d, cfg.max_seq_len)
        self.register_buffer('cos', cos, persistent=False)
        self.register_buffer('sin', sin, persistent=False)

    def hidden(self, ids):
        cfg = self.cfg
        n, L = ids.shape
        H, D = cfg.n_heads, cfg.d_model // cfg.n_heads
        x = self.embedding(ids)
        cos, sin = self.cos[:L, :D], self.sin[:L, :D]
        for i in range(cfg.n_layers):
            h = F.rms_norm(x, (cfg.d_model,), self.norm1[i], 1e-6)
            q, k, v = self.wqkv[i](h).chunk(3, dim=-1)
            q, k, v = (t.view(n, L, H, D).transpose(1, 2) for t in (q, k, v))
            q, k = ops.apply_rope(q, k, cos, sin)
            a = F.scaled_dot_product_attention(q.to(v.dtype), k.to(v.dtype), v, is_causal=True)
            x = x + self.wo[i](a.transpose(1, 2).reshape(n, L, cfg.d_model))
            h = F.rms_norm(x, (cfg.d_model,), self.norm2[i], 1e-6)
            x = x + self.w2[i](F.silu(self.w1[i](h)) * self.w3[i](h))
        return F.rms_norm(x, (cfg.d_model,), self.norm_f, 1e-6)

    def compute_loss(self, ids, ignore_index=0, chunk_rows=2048, denominator=None):
        h = self.hidden(ids)[:, :-1, :]
        t = ids[:, 1:]
        return ops.chunked_ce(h.reshape(-1, h.shape[-1]), self.fc_out.weight, t.reshape(-1),
                              ignore_index=ignore_index, chunk_rows=chunk_rows, denominator=denominator)


def step_loss_and_grads(model: OracleLM, micro_batches, samples_per_step, ignore_index=0,
                        chunk_rows=2048):
    """train.py:2351-2358: each micro-batch's mean loss is weighted by
    ``n / samples_per_step`` before backward; grads accumulate.  Returns the
    weighted loss sum (what the reference logs as the step loss)."""
    model.zero_grad(set_to_none=True)
    total = 0.0
    for ids in micro_batches:
        w = ids.shape[0] / samples_per_step
        loss = model.compute_loss(ids, ignore_index=ignore_index, chunk_rows=chunk_rows)
        (loss * w).backward()
        total += float(loss.detach()) * w
    return total
