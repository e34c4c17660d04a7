"""Seeded inputs shared by the golden-vector generator and the tests, so both
sides see identical tensors without storing them."""
import numpy as np
import torch

TINY_MODEL = dict(vocab_size=4096, d_model=128, n_heads=4, n_layers=2, d_ff=344, max_seq_len=256)

# head_dim 64 (the CUDA kernels' shape) toy used for the state_dict layout check
TINY64_MODEL = dict(vocab_size=4096, d_model=128, n_heads=2, n_layers=2, d_ff=344, max_seq_len=256)

# dropout keep-mask blocks: (seed, batch*head index, p, first row, rows, first col, cols)
DROPOUT_CASES = [
    (1, 0, 0.1, 0, 200, 0, 200),
    (0xDEADBEEF, 95, 0.5, 0, 64, 0, 64),
    (2654435761, 11, 0.1, 4000, 96, 4000, 96),          # the last rows/cols of a 4096-long sequence
    (123456789, 7, 0.25, 1000, 33, 17, 129),
    (42, 3, 0.9, 0, 128, 64, 128),
    (7, 0, 0.0, 0, 16, 0, 16),                           # p = 0 keeps everything
]

# name -> (documents, length seed, samples_per_step, target_tokens, sampler seed)
SAMPLER_CASES = {
    'c3_small': (5000, 7, 64, 32768, 42),
    'c5_small': (6000, 11, 256, 32768, 42),
    'ref_budget': (3000, 13, 64, 12288, 1234),
}


def log_uniform_lengths(n, seed, lo=64, hi=4094):
    """Body lengths floor(exp(U(ln lo, ln hi))) -- the synthetic corpus shape."""
    rng = np.random.default_rng(seed)
    return np.floor(np.exp(rng.uniform(np.log(lo), np.log(hi), size=n))).astype(np.int64)


def collate_rows():
    rng = np.random.default_rng(5)
    return [rng.integers(3, 4096, size=n).astype(np.uint16) for n in (5, 1, 17, 0, 33, 8)]


def _randn(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32)


def rope_qk():
    return _randn((2, 3, 70, 64), 101), _randn((2, 3, 70, 64), 102)


def rope_grads():
    return _randn((2, 3, 70, 64), 103), _randn((2, 3, 70, 64), 104)


def attn_small():
    return tuple(_randn((1, 2, 150, 64), 200 + i) for i in range(4))


def rms_small():
    x = _randn((37, 128), 301)
    w = 1.0 + 0.02 * _randn((128,), 302)
    return x, w, _randn((37, 128), 303)


def ce_small():
    h = _randn((150, 64), 401)
    W = 0.02 * _randn((500, 64), 402)
    g = torch.Generator().manual_seed(403)
    t = torch.randint(1, 500, (150,), generator=g)
    t[torch.rand(150, generator=g) < 0.05] = 0
    return h, W, t


def tiny_batch(seed=0, n=8, lo=32, hi=256):
    """Config-1 batch: n rows, total length (with BOS/EOS) uniform in [lo, hi]."""
    rng = np.random.default_rng(seed)
    return [rng.integers(3, 4096, size=int(L) - 2).astype(np.uint16)
            for L in rng.integers(lo, hi + 1, size=n)]


def seeded_weights(seed=0, cfg=TINY_MODEL):
    """name -> tensor in the *reference's* parameter naming, N(0, 0.02) matrices
    and 1 + N(0, 0.02) norm gains, drawn in a fixed order from one generator."""
    g = torch.Generator().manual_seed(1000 + seed)
    d, ff, V = cfg['d_model'], cfg['d_ff'], cfg['vocab_size']
    out = {'embedding.weight': 0.02 * torch.randn(V, d, generator=g)}
    for i in range(cfg['n_layers']):
        p = f'layers.{i}.'
        out[p + 'self_attn.wqkv.weight'] = 0.02 * torch.randn(3 * d, d, generator=g)
        out[p + 'self_attn.wo.weight'] = 0.02 * torch.randn(d, d, generator=g)
        out[p + 'ff.w1.weight'] = 0.02 * torch.randn(ff, d, generator=g)
        out[p + 'ff.w3.weight'] = 0.02 * torch.randn(ff, d, generator=g)
        out[p + 'ff.w2.weight'] = 0.02 * torch.randn(d, ff, generator=g)
        out[p + 'norm1.weight'] = 1.0 + 0.02 * torch.randn(d, generator=g)
        out[p + 'norm2.weight'] = 1.0 + 0.02 * torch.randn(d, generator=g)
    out['norm.weight'] = 1.0 + 0.02 * torch.randn(d, generator=g)
    return out


def load_seeded_weights_into_reference(model, seed=0):
    sd = seeded_weights(seed, dict(vocab_size=model.config.vocab_size, d_model=model.config.d_model,
                                   d_ff=model.config.d_ff, n_layers=model.config.n_layers))
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(sd[n])


def load_seeded_weights_into_oracle(model, seed=0):
    """Same tensors, mapped onto oracle.model.OracleLM's parameter names."""
    c = model.cfg
    sd = seeded_weights(seed, dict(vocab_size=c.vocab_size, d_model=c.d_model, d_ff=c.d_ff,
                                   n_layers=c.n_layers))
    with torch.no_grad():
        model.embedding.weight.copy_(sd['embedding.weight'])
        for i in range(c.n_layers):
            p = f'layers.{i}.'
            model.wqkv[i].weight.copy_(sd[p + 'self_attn.wqkv.weight'])
            model.wo[i].weight.copy_(sd[p + 'self_attn.wo.weight'])
            model.w1[i].weight.copy_(sd[p + 'ff.w1.weight'])
            model.w3[i].weight.copy_(sd[p + 'ff.w3.weight'])
            model.w2[i].weight.copy_(sd[p + 'ff.w2.weight'])
            model.norm1[i].copy_(sd[p + 'norm1.weight'])
            model.norm2[i].copy_(sd[p + 'norm2.weight'])
        model.norm_f.copy_(sd['norm.weight'])
