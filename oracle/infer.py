"""Oracle restatement of the reference's forward-only consumers of attention: the inference
model's attention module (inf.py:109-135), the Hugging Face attention module
(hf_template/modeling_universal_lm.py:106-156, prefill and cached decode) and the perplexity
scorer (inf.py:866-937).  Plain PyTorch (F.scaled_dot_product_attention, F.cross_entropy).

Test infrastructure: see the package docstring.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


def _rope(q, k, cos, sin, head_dim):
    """inf.py:97-106: tables [1, L, >=head_dim] truncated to head_dim, eager rotation in fp32."""
    cos2d = cos.reshape(-1, cos.shape[-1])[:, :head_dim]
    sin2d = sin.reshape(-1, sin.shape[-1])[:, :head_dim]
    return ops.apply_rope(q, k, cos2d, sin2d)


class InfAttention(nn.Module):  # inf.py:109-135
    def __init__(self, d_model, n_heads):
        super().__init__()
        self.d_model, self.n_heads, self.head_dim = d_model, n_heads, d_model // n_heads
        self.wqkv = nn.Linear(d_model, 3 * d_model, bias=False)
        self.wo = nn.Linear(d_model, d_model, bias=False)

    def forward(self, x, mask=None, cos=None, sin=None):
        b, t, _ = x.shape
        q, k, v = (u.view(b, t, self.n_heads, self.head_dim).transpose(1, 2) for u in self.wqkv(x).chunk(3, dim=-1))
        if cos is not None and sin is not None:
            q, k = _rope(q, k, cos, sin, self.head_dim)
        a = F.scaled_dot_product_attention(q.to(v.dtype), k.to(v.dtype), v, attn_mask=mask, dropout_p=0.0, is_causal=True)
        return self.wo(a.transpose(1, 2).contiguous().view(b, t, self.d_model))


class HFAttention(nn.Module):  # hf_template/modeling_universal_lm.py:106-156 (tuple cache form)
    def __init__(self, d_model, n_heads, layer_idx=0):
        super().__init__()
        self.layer_idx = layer_idx
        self.d_model, self.n_heads, self.head_dim = d_model, n_heads, d_model // n_heads
        self.wqkv = nn.Linear(d_model, 3 * d_model, bias=False)
        self.wo = nn.Linear(d_model, d_model, bias=False)

    def forward(self, x, cos, sin, attention_mask=None, past_key_value=None, use_cache=False, is_causal=True):
        b, t, _ = x.shape
        q, k, v = (u.view(b, t, self.n_heads, self.head_dim).transpose(1, 2) for u in self.wqkv(x).chunk(3, dim=-1))
        q, k = _rope(q, k, cos, sin, self.head_dim)
        q, k = q.to(v.dtype), k.to(v.dtype)
        if past_key_value is not None:
            k = torch.cat([past_key_value[0], k], dim=2)
            v = torch.cat([past_key_value[1], v], dim=2)
        present = (k, v) if use_cache else None
        if attention_mask is None:
            a = F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=is_causal)
        else:
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask, dropout_p=0.0)
        return self.wo(a.transpose(1, 2).contiguous().view(b, t, self.d_model)), present


def score_windows(model, windows, pad_id, device, batch_size, chunk_rows, amp_dtype=torch.float16):
    """inf.py:866-937 on a model with ``hidden(ids)`` and ``fc_out`` (oracle.model.OracleLM):
    per-window (loss sum, token count, correct top-1 count)."""
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
        input_ids, labels = input_ids.to(device), labels.to(device)
        with torch.no_grad():
            with torch.autocast(device_type=device.type, dtype=amp_dtype):
                hidden = model.hidden(input_ids)
            flat_h = hidden.reshape(-1, hidden.shape[-1])
            flat_y = labels.reshape(-1)
            for s in range(0, flat_y.numel(), chunk_rows):
                y = flat_y[s:s + chunk_rows]
                if int((y != -100).sum()) == 0:
                    continue
                with torch.autocast(device_type=device.type, dtype=amp_dtype):
                    logits = model.fc_out(flat_h[s:s + chunk_rows])
                    per_pos = F.cross_entropy(logits, y, ignore_index=-100, reduction='none')
                pred = logits.argmax(dim=-1)
                for local, orig in enumerate(idxs):
                    lo, hi = max(s, local * t), min(s + chunk_rows, (local + 1) * t)
                    if hi <= lo:
                        continue
                    a, b = lo - s, hi - s
                    yb = y[a:b]
                    keep = yb != -100
                    nb = int(keep.sum())
                    if nb == 0:
                        continue
                    losses[orig] += float(per_pos[a:b][keep].sum())
                    tokens[orig] += nb
                    correct[orig] += int((pred[a:b][keep] == yb[keep]).sum())
    return losses, tokens, correct
