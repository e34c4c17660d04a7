"""The reference's decoder-only model (train.py:1862-2082) with the hot-path ops
served by the sm_100a library: fused RoPE, FlashAttention forward/backward,
RMSNorm and the chunked cross-entropy.  Class, method and parameter names
follow train.py so that its checkpoints' ``model_state_dict`` load unchanged.

The linear layers stay on cuBLAS through torch (plain library GEMMs).  There is
no SDPA or eager fallback in here: a shape the kernels do not take (head_dim
other than 64, CPU tensors) raises.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

import flash_attn_v100_cuda as _fa
import ulm_ops
from ulm_ops import FusedRMSNorm, linear, swiglu


@dataclass
class ModelConfig:  # train.py:725-737
    vocab_size: int = 32000
    d_model: int = 768
    n_heads: int = 12
    n_layers: int = 10
    d_ff: int = 2048
    max_seq_len: int = 4096
    dropout: float = 0.0
    use_rope: bool = True
    tie_weights: bool = True
    use_gradient_checkpointing: bool = False


# compute_loss pads the flattened token dimension to a multiple of this (see DecoderOnlyTransformer._forward_flat)
TOKEN_QUANTUM = 1024


def rope_tables(d_model: int, seq_len: int, base: float = 10000.0):
    """fp32 cos/sin tables [seq_len, d_model] as train.py:1878-1891 builds them:
    inv_freq spans the MODEL width (base ** -(2i/d_model), i < d_model/2) and is
    tiled twice; heads later read only the first head_dim columns, so all 64
    columns of a head carry different angles."""
    inv_freq = 1.0 / (base ** (torch.arange(0, d_model, 2).float() / d_model))
    t = torch.arange(seq_len, dtype=inv_freq.dtype)
    freqs = torch.einsum('i,j->ij', t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


class RotaryPositionalEmbedding(nn.Module):  # train.py:1877-1896
    """Buffers ``inv_freq`` [d_model/2], ``cos_cached`` and ``sin_cached`` [1, max_len, d_model] are
    persistent like the reference's, so its checkpoints load with ``strict=True`` and the reference
    loads checkpoints written from this model."""

    def __init__(self, d_model: int, max_len: int = 4096):
        super().__init__()
        self.d_model = d_model
        self.max_len = max_len
        self.register_buffer('inv_freq', 1.0 / (10000.0 ** (torch.arange(0, d_model, 2).float() / d_model)))
        self._build(max_len)

    def _build(self, n):
        # tables are computed on the CPU in fp32 (bit-equal to the reference's CPU construction) and moved
        cos, sin = rope_tables(self.d_model, n)
        dev = self.inv_freq.device
        self.register_buffer('cos_cached', cos.unsqueeze(0).to(dev))
        self.register_buffer('sin_cached', sin.unsqueeze(0).to(dev))

    def forward(self, seq_len):
        if seq_len > self.cos_cached.shape[1]:
            self._build(seq_len)
        return self.cos_cached[:, :seq_len], self.sin_cached[:, :seq_len]


def _tables_2d(cos, sin, hd):
    """The first head_dim columns of the [1, L, d_model] tables as [L, head_dim] views (train.py:1904-1911)."""
    cos2d = cos[..., :hd].reshape(-1, hd) if cos.shape[-1] == hd else cos[0, :, :hd]
    sin2d = sin[..., :hd].reshape(-1, hd) if sin.shape[-1] == hd else sin[0, :, :hd]
    return cos2d, sin2d


def apply_rotary_pos_emb(q, k, cos, sin):
    """train.py:1902-1918, fused branch only."""
    cos2d, sin2d = _tables_2d(cos, sin, q.shape[-1])
    if not _fa.rope_can_use(q, k, cos2d, sin2d):
        raise ValueError('fused RoPE needs 16-bit (B,H,S,64) CUDA views and fp32 (S,64) tables')
    return _fa.rope(q, k, cos2d, sin2d)


class MultiHeadAttention(nn.Module):  # train.py:1920-1964
    def __init__(self, config: ModelConfig):
        super().__init__()
        self.d_model, self.n_heads = config.d_model, config.n_heads
        self.head_dim = config.d_model // config.n_heads
        self.wqkv = nn.Linear(config.d_model, 3 * config.d_model, bias=False)
        self.wo = nn.Linear(config.d_model, config.d_model, bias=False)
        self.dropout = config.dropout

    def forward(self, x, cos=None, sin=None, shape=None):
        """``x``: [n, L, d], or -- with ``shape=(n, L)`` -- the flattened tokens [T', d] with T' >= n*L (rows
        beyond n*L are padding that only the projections see)."""
        flat = shape is not None
        n, L = shape if flat else x.shape[:2]
        T = n * L
        x2d = x if flat else x.reshape(T, x.shape[-1])
        qkv = linear(x2d, self.wqkv.weight)
        if qkv.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError('attention runs in fp16/bf16: call the model under torch.autocast')
        # train.py:1935-1964 between the two projections as one op on the fused tensor: chunk, RoPE, causal
        # attention, heads merged; q, k, v are views, the output needs no transpose copy and the backward
        # writes dq, dk, dv into the slices of one gradient tensor (no concatenation)
        p_drop = self.dropout if self.training else 0.0
        cos2d = sin2d = None
        if cos is not None:
            cos2d, sin2d = _tables_2d(cos, sin, self.head_dim)
        # on the flattened tensor: the op reads the first n*L rows as [n, L, 3d] and returns [T', d] with zero
        # padding rows, its backward a [T', 3d] gradient with zero padding rows (no pad or slice copies)
        a2d = _fa.qkv_rope_flash_attn(qkv, self.n_heads, cos2d, sin2d, dropout_p=p_drop, causal=True, flat_shape=(n, L))
        out = linear(a2d, self.wo.weight)
        return out if flat else out.view(n, L, out.shape[-1])


class FeedForward(nn.Module):  # train.py:1966-1975
    def __init__(self, d_model: int, d_ff: int, dropout: float):
        super().__init__()
        self.w1 = nn.Linear(d_model, d_ff, bias=False)
        self.w3 = nn.Linear(d_model, d_ff, bias=False)
        self.w2 = nn.Linear(d_ff, d_model, bias=False)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x):
        return linear(self.dropout(swiglu(linear(x, self.w1.weight), linear(x, self.w3.weight))), self.w2.weight)


class DecoderOnlyBlock(nn.Module):  # train.py:1977-1994
    """The reference's block computes x = x + attn(norm1(x)); x = x + dropout(ff(norm2(x))).  Here every
    residual add is fused with the norm that FOLLOWS it (one pass over the residual stream instead of
    two), so a block receives the residual stream together with the branch output that has not been
    added yet (`pending`: the previous block's feed-forward output, None for the first block) and hands
    its own feed-forward output on in the same way; the model's final norm absorbs the last one.  Same
    values, same parameter names."""

    def __init__(self, config: ModelConfig):
        super().__init__()
        self.self_attn = MultiHeadAttention(config)
        self.ff = FeedForward(config.d_model, config.d_ff, config.dropout)
        self.norm1 = FusedRMSNorm(config.d_model)
        self.norm2 = FusedRMSNorm(config.d_model)
        self.dropout = nn.Dropout(config.dropout)

    def forward(self, x, pending=None, cos=None, sin=None, shape=None):
        if pending is None:
            h = self.norm1(x)
        else:
            x, h = self.norm1.add_forward(x, pending)                 # train.py:1993 of the previous block + 1988
        x, h = self.norm2.add_forward(x, self.self_attn(h, cos=cos, sin=sin, shape=shape))   # train.py:1989 + 1991
        return x, self.dropout(self.ff(h))                            # added by whoever normalises next


class DecoderOnlyTransformer(nn.Module):  # train.py:1996-2082
    def __init__(self, config: ModelConfig):
        super().__init__()
        if config.d_model // config.n_heads != 64:
            raise ValueError('the sm_100a attention and RoPE kernels are built for head_dim 64')
        self.config = config
        self.embedding = nn.Embedding(config.vocab_size, config.d_model)
        self.use_gradient_checkpointing = config.use_gradient_checkpointing
        if config.use_rope:
            self.rope = RotaryPositionalEmbedding(config.d_model, config.max_seq_len)
        self.layers = nn.ModuleList([DecoderOnlyBlock(config) for _ in range(config.n_layers)])
        self.norm = FusedRMSNorm(config.d_model)
        self.fc_out = nn.Linear(config.d_model, config.vocab_size, bias=False)
        if config.tie_weights:
            self.fc_out.weight = self.embedding.weight
        for m in self.modules():  # train.py:2015-2022
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def _forward_flat(self, ids, quantum=0):
        """Hidden states of the flattened tokens, [T', d] with T' = n*L rounded up to a multiple of ``quantum``
        (0: no padding).  Everything outside the attention works on rows, so the layers run on the 2-D tensor;
        the padding rows carry an arbitrary token, are seen by projections, norms and gates only, and reach
        no loss term.  Why pad: a library GEMM costs its launcher 0.65-1.4 ms the first time it sees a row
        count (10 us afterwards); a micro-batch's token count is almost always new, a multiple of 1024 soon is
        not."""
        n, L = ids.shape
        T = n * L
        Tp = T if quantum <= 1 else -(-T // quantum) * quantum
        flat_ids = ids.reshape(-1)
        if Tp > T:
            flat_ids = torch.cat([flat_ids, flat_ids.new_zeros(Tp - T)])
        x = self.embedding(flat_ids)
        cos = sin = None
        if self.config.use_rope:
            cos, sin = self.rope(L)
        pending = None
        for layer in self.layers:
            if self.use_gradient_checkpointing and self.training:
                x, pending = torch.utils.checkpoint.checkpoint(layer, x, pending, cos, sin, (n, L), use_reentrant=False)
            else:
                x, pending = layer(x, pending, cos=cos, sin=sin, shape=(n, L))
        x = self.norm(x) if pending is None else self.norm.add_forward(x, pending)[1]
        return x, T

    def forward_hidden(self, x):
        n, L = x.shape
        h, T = self._forward_flat(x, 0)
        return h.view(n, L, h.shape[-1])

    def forward(self, x):
        return self.fc_out(self.forward_hidden(x))

    def compute_loss(self, input_ids, labels=None, ignore_index=0, chunk_rows: int = 2048,
                     denominator=None):
        """Shifted CE, mean over targets != ignore_index, chunked over rows
        (train.py:2059-2082).  ``denominator`` replaces the local count of valid
        targets: the data-parallel step passes the micro-batch's global count."""
        labels = input_ids if labels is None else labels
        n, L = input_ids.shape
        hidden, T = self._forward_flat(input_ids, TOKEN_QUANTUM)
        # position i predicts label i+1; a row's last position and the padding rows predict nothing
        target = labels.new_full((hidden.shape[0],), ignore_index)
        target[:T].view(n, L)[:, :-1] = labels[:, 1:]
        return ulm_ops.chunked_cross_entropy(hidden, self.fc_out.weight, target, ignore_index=ignore_index,
                                             chunk_rows=chunk_rows, denominator=denominator)
