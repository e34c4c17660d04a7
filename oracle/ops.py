"""Oracle restatements of the numeric ops on the hot path (CPU, torch/numpy).

Test infrastructure: see the package docstring.  All math runs in fp32 (or fp64
where stated) and is rounded the way the reference's autocast path rounds.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------
# RoPE -- train.py:1877-1918 (RotaryPositionalEmbedding, rotate_half,
# apply_rotary_pos_emb) and csrc/flash_attn_v100/fast_ops.cu:31-68.
# --------------------------------------------------------------------------
def rope_tables(d_model: int, seq_len: int, base: float = 10000.0):
    """cos/sin tables exactly as train.py:1878-1891 builds them.

    The reference derives ``inv_freq`` from the *model* width, not the head
    width: ``inv_freq[i] = base ** -(2 i / d_model)`` for i < d_model/2, and the
    table ``cat(freqs, freqs)`` is d_model wide.  ``apply_rotary_pos_emb`` then
    keeps only the first ``head_dim`` columns (train.py:1903-1906), so column j
    of a 64-wide head rotates by ``pos * base ** -(2 j / d_model)`` for every
    j < 64 (as long as head_dim <= d_model/2): dims j and j+32 do not share an
    angle.  Returned tables are fp32 ``[seq_len, d_model]``.
    """
    inv_freq = 1.0 / (base ** (torch.arange(0, d_model, 2).float() / d_model))
    t = torch.arange(seq_len, dtype=inv_freq.dtype)
    freqs = torch.einsum('i,j->ij', t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rope_tables_head(d_model: int, seq_len: int, head_dim: int, base: float = 10000.0):
    """The ``[S, head_dim]`` views (row stride d_model) the kernels receive."""
    cos, sin = rope_tables(d_model, seq_len, base)
    return cos[:, :head_dim], sin[:, :head_dim]


def _swap_halves_neg(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(q, k, cos2d, sin2d, out_dtype=None):
    """Eager branch of apply_rotary_pos_emb (train.py:1914-1918).

    q, k: ``(B, H, S, D)`` in any float dtype; cos2d/sin2d fp32 ``[S, D]``.
    The products and the sum are formed in fp32 (type promotion against the fp32
    tables) and, when ``out_dtype`` is 16-bit, rounded once -- what autocast's
    later cast (train.py:103-113) does, and what fast_ops.cu:44-48 reproduces
    bit for bit.
    """
    c = cos2d.float()[None, None].to(q.device)
    s = sin2d.float()[None, None].to(q.device)
    qf, kf = q.float(), k.float()
    qo = (qf * c) + (_swap_halves_neg(qf) * s)
    ko = (kf * c) + (_swap_halves_neg(kf) * s)
    if out_dtype is not None:
        qo, ko = qo.to(out_dtype), ko.to(out_dtype)
    return qo, ko


def rope_backward(gq, gk, cos2d, sin2d, out_dtype=None):
    """Adjoint of :func:`apply_rope` as fast_ops.cu:51-68 computes it.

    ``dq[d] = g[d] cos[d] + sgn * g[p] sin[p]`` with partner ``p = d +- D/2``:
    the sine is read at the *partner's* column and sgn is +1 for d < D/2.
    fp32 multiply, multiply, add without contraction, one rounding.
    """
    c = cos2d.float()[None, None].to(gq.device)
    s = sin2d.float()[None, None].to(gq.device)
    half = gq.shape[-1] // 2

    def one(g):
        g = g.float()
        gs = g * s  # g[p] * sin[p], still indexed by p
        partner = torch.cat((gs[..., half:], -gs[..., :half]), dim=-1)
        return (g * c) + partner

    dq, dk = one(gq), one(gk)
    if out_dtype is not None:
        dq, dk = dq.to(out_dtype), dk.to(out_dtype)
    return dq, dk


# --------------------------------------------------------------------------
# Dropout hash -- csrc/flash_attn_v100/fa_common.cuh:21-38.
# --------------------------------------------------------------------------
def hash_u32(x: int) -> int:
    """The integer mix of fa_common.cuh:21-26 on one uint32."""
    x &= 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x ^= x >> 15
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def dropout_keep_mask(seed: int, n_rows: int, n_cols: int, bh: int, p: float) -> np.ndarray:
    """Boolean ``[n_rows, n_cols]`` keep mask of head ``bh`` (b*H + h).

    Pure uint32 arithmetic: ``h = seed*0x9E3779B1 ^ (row+1)*0x85EBCA6B ^
    (col+1)*0xC2B2AE35 ^ (bh+1)*0x27D4EB2F``, a 3-round xorshift-multiply mix,
    then keep iff ``(h >> 8) * 2**-24 >= p`` (fp32 compare).
    """
    m32 = np.uint64(0xFFFFFFFF)
    rows = (np.arange(n_rows, dtype=np.uint64) + np.uint64(1)) * np.uint64(0x85EBCA6B) & m32
    cols = (np.arange(n_cols, dtype=np.uint64) + np.uint64(1)) * np.uint64(0xC2B2AE35) & m32
    h = (np.uint64(seed & 0xFFFFFFFF) * np.uint64(0x9E3779B1)) & m32
    h = h ^ rows[:, None] ^ cols[None, :] ^ ((np.uint64(bh + 1) * np.uint64(0x27D4EB2F)) & m32)
    h ^= h >> np.uint64(16)
    h = (h * np.uint64(0x7FEB352D)) & m32
    h ^= h >> np.uint64(15)
    h = (h * np.uint64(0x846CA68B)) & m32
    h ^= h >> np.uint64(16)
    u = (h >> np.uint64(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    return u >= np.float32(p)


# --------------------------------------------------------------------------
# Attention -- train.py:1955-1961 (SDPA, is_causal=True) is the parity target;
# flash_attn_v100.cu:40-309 / flash_attn_v100_bwd.cu:42-428 define LSE, delta
# and the dropout convention.
# --------------------------------------------------------------------------
def sdpa_causal(q, k, v, scale=None):
    """The reference's own attention call (train.py:1956-1961, dropout 0)."""
    return F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale)


def attention_explicit(q, k, v, scale=None, causal=True, dropout_p=0.0, seed=0,
                       dtype=torch.float32):
    """Dense softmax attention in ``dtype`` (fp32/fp64) math with the kernel's
    conventions; returns ``(o, lse)``.

    * LSE is the natural-log logsumexp of the scaled, masked scores
      (flash_attn_v100.cu:298-302).
    * With dropout, the softmax denominator is the *undropped* sum and kept
      probabilities are scaled by 1/(1-p) (flash_attn_v100.cu:205-232); the
      mask is :func:`dropout_keep_mask`.
    Differentiable through torch autograd (the mask is a constant).
    """
    B, H, S, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    s = torch.matmul(q.to(dtype), k.to(dtype).transpose(-1, -2)) * scale
    if causal:
        tri = torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1)
        s = s.masked_fill(tri, float('-inf'))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    if dropout_p > 0.0:
        keep = np.stack([dropout_keep_mask(seed, S, S, bh, dropout_p) for bh in range(B * H)])
        keep = torch.from_numpy(keep).view(B, H, S, S).to(q.device)
        p = p * keep.to(dtype) / (1.0 - dropout_p)
    o = torch.matmul(p, v.to(dtype))
    return o, lse


def rope_attention_grads(q, k, v, do, cos2d, sin2d, dtype, scale=None, use_sdpa=True):
    """Config-2 parity target: eager RoPE -> cast to ``dtype`` -> causal SDPA,
    gradients w.r.t. the *pre-RoPE* q, k and v by autograd.

    ``dtype`` fp16/bf16 gives the same-precision oracle; fp32/fp64 with
    ``use_sdpa=False`` gives the high-precision truth that bounds both
    implementations' error.  Returns dict(o, lse, dq, dk, dv, q_rot, k_rot).
    """
    q0 = q.detach().clone().requires_grad_(True)
    k0 = k.detach().clone().requires_grad_(True)
    v0 = v.detach().clone().requires_grad_(True)
    qf, kf = apply_rope(q0, k0, cos2d, sin2d)
    qr, kr, vr = qf.to(dtype), kf.to(dtype), v0.to(dtype)
    if use_sdpa:
        o = sdpa_causal(qr, kr, vr, scale)
        with torch.no_grad():
            _, lse = attention_explicit(qr.float(), kr.float(), vr.float(), scale)
    else:
        o, lse = attention_explicit(qr, kr, vr, scale, dtype=dtype)
    o.backward(do.to(o.dtype))
    return dict(o=o.detach(), lse=lse.detach(), dq=q0.grad, dk=k0.grad, dv=v0.grad,
                q_rot=qr.detach(), k_rot=kr.detach())


def attention_bwd_explicit(q, k, v, o, lse, do, scale=None, causal=True,
                           dropout_p=0.0, seed=0):
    """Backward restated from flash_attn_v100_bwd.cu:10-15 in fp32:
    ``P = exp(S - lse)``, ``P_d = keep*P/(1-p)``, ``delta = rowsum(O*dO)``,
    ``dV = P_d^T dO``, ``dP = dO V^T``, ``dS = P_d*dP - P*delta``,
    ``dQ = scale dS K``, ``dK = scale dS^T Q``.  Returns (dq, dk, dv, delta).
    """
    B, H, S, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    qf, kf, vf, of, dof = (t.float() for t in (q, k, v, o, do))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1), float('-inf'))
    p = torch.exp(s - lse.float()[..., None])
    pd = p
    if dropout_p > 0.0:
        keep = np.stack([dropout_keep_mask(seed, S, S, bh, dropout_p) for bh in range(B * H)])
        pd = p * torch.from_numpy(keep).view(B, H, S, S).float().to(q.device) / (1.0 - dropout_p)
    delta = (of * dof).sum(-1)
    dv = torch.matmul(pd.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = pd * dp - p * delta[..., None]
    dq = torch.matmul(ds, kf) * scale
    dk = torch.matmul(ds.transpose(-1, -2), qf) * scale
    return dq, dk, dv, delta


# --------------------------------------------------------------------------
# RMSNorm -- train.py:1862-1875 (F.rms_norm); manual form inf.py:58-67.
# --------------------------------------------------------------------------
def rms_norm(x, weight, eps: float = 1e-6):
    """``w * x * rsqrt(mean(x^2) + eps)`` with an fp32 reduction; the result is
    returned in x's dtype (what F.rms_norm does for 16-bit inputs)."""
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * weight.float()).to(x.dtype)


def rms_norm_backward(x, weight, dy, eps: float = 1e-6):
    """fp32 gradients of :func:`rms_norm`: returns (dx in x.dtype, dw fp32)."""
    xf, wf, g = x.float(), weight.float(), dy.float()
    d = xf.shape[-1]
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    xhat = xf * inv
    gw = g * wf
    dx = inv * (gw - xhat * (gw * xhat).sum(-1, keepdim=True) / d)
    dw = (g * xhat).reshape(-1, d).sum(0)
    return dx.to(x.dtype), dw


# --------------------------------------------------------------------------
# Chunked cross-entropy -- train.py:2059-2082 (compute_loss body after
# forward_hidden).
# --------------------------------------------------------------------------
def chunked_ce(hidden, weight, target, ignore_index=0, chunk_rows=2048, logits_dtype=None,
               denominator=None):
    """Mean CE over targets != ignore_index, computed chunk by chunk.

    ``hidden`` is ``[rows, d]``, ``weight`` ``[V, d]``, ``target`` int64 ``[rows]``
    (the caller has already applied the one-token shift of train.py:2066-2067).
    ``denominator`` overrides the count of valid targets (used to check the
    data-parallel identity, where a rank divides by the whole micro-batch's count).
    ``logits_dtype`` is the dtype the lm-head GEMM produces under autocast
    (fp16/bf16); F.cross_entropy then runs in fp32 (autocast promotes it).
    """
    n_tokens = (target != ignore_index).sum().clamp(min=1) if denominator is None else denominator
    total = None
    for i in range(0, hidden.shape[0], chunk_rows):
        h = hidden[i:i + chunk_rows]
        if logits_dtype is not None:
            logits = (h.to(logits_dtype) @ weight.to(logits_dtype).t()).float()
        else:
            logits = h @ weight.t()
        part = F.cross_entropy(logits, target[i:i + chunk_rows],
                               ignore_index=ignore_index, reduction='sum')
        total = part if total is None else total + part
    if total is None:
        return torch.zeros((), requires_grad=True)
    return total / n_tokens


def ce_rows(logits, target, ignore_index=0):
    """Per-row pieces of the CE over a logits tile in fp32: returns
    (lse[rows], loss_sum, dlogits for upstream grad 1 on loss_sum)."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    valid = target != ignore_index
    tgt = target.clamp(min=0)
    picked = lf.gather(1, tgt[:, None]).squeeze(1)
    loss_sum = ((lse - picked) * valid).sum()
    dl = torch.exp(lf - lse[:, None])
    dl[torch.arange(lf.shape[0], device=lf.device), tgt] -= 1.0
    dl = dl * valid[:, None]
    return lse, loss_sum, dl
