"""Forward-only use of the attention kernels: the reference's inference model, its perplexity
scoring and its Hugging Face attention module all call F.scaled_dot_product_attention directly
(inf.py:119-135, 866-937; hf_template/modeling_universal_lm.py:117-156).  This module gives the
same three places the sm_100a forward kernel:

    causal_attention(qkv, n_heads, cos, sin)   one causal prefill attention on the fused projection
    patch_attention(model)                     rebinds ``forward`` of every attention module of an
                                               inf.py / HF model (attributes wqkv, wo, n_heads, head_dim)
    score_windows(...)                         inf.py:866-937 with the fused forward and the
                                               cross-entropy row kernel

Only the case the kernel covers is taken over -- causal attention over the whole sequence, no
attention mask, no KV cache, head_dim 64, fp16/bf16 on a B200; anything else (single-token decode
steps with a cache, padded-mask batches, CPU tensors) goes to the module's own forward, which is the
caller's code, not a path of this library.
"""
import types

import torch

import flash_attn_v100_cuda as _fa
import ulm_ops


def causal_attention(qkv, n_heads, cos=None, sin=None, softmax_scale=None):
    """qkv [n, L, 3*n_heads*64] 16-bit contiguous -> (attention output [n, L, n_heads*64], k, v) with k
    rotated, both as (n, n_heads, L, 64) views.  ``cos``/``sin``: the model's [1, L, >=64] or [L, >=64]
    fp32 RoPE tables (None: no rotation).  No autograd graph is built and nothing is saved: Q is rotated
    inside the kernel and its rotated copy is never written."""
    B, S, _ = qkv.shape
    q, k, v = (t.view(B, S, n_heads, 64).transpose(1, 2) for t in qkv.detach().chunk(3, dim=-1))
    scale = 64 ** -0.5 if softmax_scale is None else float(softmax_scale)
    if cos is not None:
        cos2d = cos.reshape(-1, cos.shape[-1])[:S, :64]
        sin2d = sin.reshape(-1, sin.shape[-1])[:S, :64]
        if not _fa.rope_can_use(q, k, cos2d, sin2d):
            raise ValueError('causal_attention needs fp32 RoPE tables of at least 64 columns on the same device')
        _, k = _fa._rope_launch(None, k, cos2d, sin2d, backward=False)
        o, _, _ = _fa.attn_forward(q, k, v, 0.0, True, scale, 0, cos=cos2d, sin=sin2d, want_q_rot=False)
    else:
        o, _, _ = _fa.attn_forward(q, k, v, 0.0, True, scale, 0)
    return o.transpose(1, 2).reshape(B, S, n_heads * 64), k, v


def _eligible(module, x, mask, past, is_causal):
    return (mask is None and past is None and is_causal and x.is_cuda and not torch.is_grad_enabled()
            and getattr(module, 'head_dim', None) == 64)


def _inf_forward(self, x, mask=None, cos=None, sin=None):
    """Replacement for inf.MultiHeadAttention.forward (inf.py:119-135)."""
    if not _eligible(self, x, mask, None, True):
        return self._ulm_original_forward(x, mask=mask, cos=cos, sin=sin)
    qkv = self.wqkv(x)
    if qkv.dtype not in (torch.float16, torch.bfloat16):
        return self._ulm_original_forward(x, mask=mask, cos=cos, sin=sin)
    out, _, _ = causal_attention(qkv.contiguous(), self.n_heads, cos, sin)
    return self.wo(out)


def _hf_forward(self, x, cos, sin, attention_mask=None, past_key_value=None, use_cache=False, is_causal=True):
    """Replacement for UniversalLMAttention.forward (hf_template/modeling_universal_lm.py:117-156):
    the prefill step; returns (output, (k, v) or None) like the original."""
    if not _eligible(self, x, attention_mask, past_key_value, is_causal):
        return self._ulm_original_forward(x, cos, sin, attention_mask=attention_mask, past_key_value=past_key_value,
                                          use_cache=use_cache, is_causal=is_causal)
    qkv = self.wqkv(x)
    if qkv.dtype not in (torch.float16, torch.bfloat16):
        return self._ulm_original_forward(x, cos, sin, attention_mask=attention_mask, past_key_value=past_key_value,
                                          use_cache=use_cache, is_causal=is_causal)
    out, k, v = causal_attention(qkv.contiguous(), self.n_heads, cos, sin)
    return self.wo(out), ((k, v) if use_cache else None)


def patch_attention(model, style='auto'):
    """Rebind ``forward`` of every attention module of ``model`` -- any submodule with ``wqkv``, ``wo``,
    ``n_heads`` and ``head_dim`` -- to the kernel-backed version.  ``style``: 'inf' for the reference's
    inference model (forward(x, mask, cos, sin)), 'hf' for its Hugging Face module (forward(x, cos, sin,
    attention_mask, past_key_value, use_cache, is_causal)), 'auto' picks 'hf' for modules that carry a
    ``layer_idx``.  Returns the number of modules patched; ``unpatch_attention`` undoes it."""
    n = 0
    for m in model.modules():
        if all(hasattr(m, a) for a in ('wqkv', 'wo', 'n_heads', 'head_dim')) and not hasattr(m, '_ulm_original_forward'):
            kind = style if style != 'auto' else ('hf' if hasattr(m, 'layer_idx') else 'inf')
            m._ulm_original_forward = m.forward
            m.forward = types.MethodType(_hf_forward if kind == 'hf' else _inf_forward, m)
            n += 1
    return n


def unpatch_attention(model):
    for m in model.modules():
        if hasattr(m, '_ulm_original_forward'):
            m.forward = m._ulm_original_forward
            del m._ulm_original_forward


def score_windows(model, windows, pad_id, device, batch_size, chunk_rows, amp_dtype=torch.float16):
    """inf.py:866-937: per-window (loss sum, token count, correct top-1 count), windows sorted by length
    into right-padded batches, ``input = w[:-1]``, ``label = w[1:]``; ``model`` provides
    ``forward_hidden`` and ``fc_out`` (ulm_model.DecoderOnlyTransformer or the reference's model after
    `patch_attention`).  The per-position losses come from the cross-entropy row kernel over 16-bit
    logit chunks of ``chunk_rows`` rows."""
    n = len(windows)
    losses, tokens, correct = [0.0] * n, [0] * n, [0] * n
    order = sorted(range(n), key=lambda i: len(windows[i]))
    for start in range(0, n, batch_size):
        idxs = order[start:start + batch_size]
        group = [windows[i] for i in idxs]
        t = max(len(w) for w in group) - 1
        if t < 1:
            continue
        input_ids = torch.full((len(group), t), pad_id, dtype=torch.long)
        labels = torch.full((len(group), t), -100, dtype=torch.long)
        for j, w in enumerate(group):
            length = len(w) - 1
            input_ids[j, :length] = torch.as_tensor(w[:-1], dtype=torch.long)
            labels[j, :length] = torch.as_tensor(w[1:], dtype=torch.long)
        input_ids = input_ids.to(device, non_blocking=True)
        labels = labels.to(device, non_blocking=True)
        with torch.no_grad():
            with torch.autocast('cuda', dtype=amp_dtype):
                hidden = model.forward_hidden(input_ids)
            flat_h = hidden.reshape(-1, hidden.shape[-1])
            flat_y = labels.reshape(-1)
            w16 = model.fc_out.weight.to(amp_dtype)
            loss_rows = torch.zeros(flat_y.numel(), dtype=torch.float32, device=device)
            hit_rows = torch.zeros(flat_y.numel(), dtype=torch.bool, device=device)
            for s in range(0, flat_y.numel(), chunk_rows):
                y = flat_y[s:s + chunk_rows].contiguous()
                hc = flat_h[s:s + chunk_rows].to(amp_dtype)
                if hc.shape[1] % 64 == 0 and w16.shape[0] % 64 == 0 and hc.is_contiguous() and w16.is_contiguous():
                    # logits and the per-position loss from one kernel (lm-head GEMM with the statistics in its epilogue)
                    _, per_pos, logits = ulm_ops.lm_head_lse(hc, w16, y, -100, keep_logits=True)
                else:
                    logits = hc @ w16.t()
                    _, per_pos = ulm_ops.ce_rows_forward(logits, y, -100)  # 0 where the label is ignored
                loss_rows[s:s + chunk_rows] = per_pos
                hit_rows[s:s + chunk_rows] = (logits.argmax(dim=-1) == y)
            keep = (flat_y != -100).view(len(group), t)
            l_sum = (loss_rows.view(len(group), t) * keep).sum(dim=1).tolist()
            n_tok = keep.sum(dim=1).tolist()
            n_hit = (hit_rows.view(len(group), t) & keep).sum(dim=1).tolist()
        for local, orig in enumerate(idxs):
            losses[orig] += float(l_sum[local])
            tokens[orig] += int(n_tok[local])
            correct[orig] += int(n_hit[local])
    return losses, tokens, correct
