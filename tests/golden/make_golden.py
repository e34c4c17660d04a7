"""Regenerates tests/golden/*.npz|json by importing the reference itself.

Run in the build container only (needs the reference checkout):

    ULM_REFERENCE_DIR=/path/to/Universal-LM-Trainer python tests/golden/make_golden.py

The reference ships no golden vectors of its own for the hot path, so these
files -- outputs of the reference's PyTorch path on seeded inputs -- are what
pins the CPU oracle (and through it the CUDA kernels).  Versions used: see
``meta`` in golden.json.
"""
import hashlib
import json
import os
import sys

import numpy as np

REF = os.environ.get('ULM_REFERENCE_DIR')
if not REF or not os.path.isfile(os.path.join(REF, 'train.py')):
    raise SystemExit('set ULM_REFERENCE_DIR to a checkout of sunyi9161/Universal-LM-Trainer')
os.environ['FA_V100_DISABLE'] = '1'
os.environ['UNIVERSAL_LM_COMPILE'] = '0'
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402
import train as ref  # noqa: E402  (the reference's train.py)

from tests.golden import inputs  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    torch.set_num_threads(1)  # reduction order of the fixtures must not depend on the host
    G = {}   # json-able
    A = {}   # arrays

    # ---- buckets (train.py:2587, 1060) ----
    G['boundaries'] = {str(m): ref.build_bucket_boundaries(m) for m in (4096, 256, 128, 50, 49, 30)}
    fb = ref.FastBucket(ref.build_bucket_boundaries(4096))
    probe = [0, 1, 49, 50, 51, 99, 100, 101, 2048, 4049, 4050, 4051, 4094, 4096, 5000]
    G['bucket_of'] = {str(n): fb.get_bucket(n) for n in probe}

    # ---- micro-batch sizes (train.py:1770) ----
    G['pick_bs'] = {}
    for name, (tt, mmb, spp) in {'c3': (32768, 64, 64), 'c5': (32768, 64, 256),
                                 'ref100m': (12288, 64, 64)}.items():
        G['pick_bs'][name] = [ref.TokenBudgetBatchSampler._pick_bs(b, tt, mmb, spp)
                              for b in ref.build_bucket_boundaries(4096)]

    # ---- sampler stream (train.py:1812) ----
    class DS:  # the three attributes the sampler reads
        pass
    for name, (n_docs, seed_len, spp, tt, seed) in inputs.SAMPLER_CASES.items():
        lens = inputs.log_uniform_lengths(n_docs, seed_len)
        bounds = ref.build_bucket_boundaries(4096)
        fbk = ref.FastBucket(bounds)
        counts = np.zeros(len(bounds), dtype=np.int64)
        for L in lens:
            counts[bounds.index(fbk.get_bucket(int(L)))] += 1
        ds = DS()
        ds.boundaries, ds.counts = bounds, counts
        ds.starts = np.concatenate(([0], np.cumsum(counts)[:-1])).astype(np.int64)
        ds.total = int(counts.sum())
        smp = ref.TokenBudgetBatchSampler(ds, samples_per_step=spp, target_tokens=tt,
                                          max_micro_batch=64, seed=seed)
        rec = {}
        for epoch in (0, 1):
            smp.set_epoch(epoch)
            mbs = list(iter(smp))
            flat = np.array([i for mb in mbs for i in mb], dtype=np.int64)
            sizes = np.array([len(mb) for mb in mbs], dtype=np.int64)
            rec[str(epoch)] = dict(ids_sha=sha(flat), sizes_sha=sha(sizes), n_mb=len(mbs),
                                   first_mb=mbs[0], last_mb=mbs[-1], sizes_head=sizes[:32].tolist())
        # resume fast-forward (train.py:1793): skip the first 3 optimiser steps
        smp.set_epoch(0, skip_samples=3 * spp)
        tail = [i for mb in iter(smp) for i in mb]
        rec['resume3_sha'] = sha(np.array(tail, dtype=np.int64))
        rec['counts_sha'] = sha(counts)
        G.setdefault('sampler', {})[name] = rec

    # ---- collate (train.py:1691) ----
    rows = inputs.collate_rows()
    A['collate_bos_eos'] = ref.collate_pad(rows, eos_id=3, bos_id=2, max_len=256).numpy()
    A['collate_eos_only'] = ref.collate_pad(rows, eos_id=3, bos_id=None, max_len=256).numpy()
    A['collate_plain'] = ref.collate_pad(rows, max_len=256).numpy()
    try:
        ref.collate_pad(rows, eos_id=3, bos_id=2, max_len=34)
        G['collate_overflow_raises'] = False
    except RuntimeError:
        G['collate_overflow_raises'] = True

    # ---- RoPE tables and the eager rotation (train.py:1877-1918) ----
    for d_model, S, hd in ((768, 4096, 64), (1024, 4096, 64), (128, 256, 32)):
        rope = ref.RotaryPositionalEmbedding(d_model, S)
        cos, sin = rope(S)
        c = cos[0, :, :hd].contiguous().numpy()
        s = sin[0, :, :hd].contiguous().numpy()
        G.setdefault('rope_tables', {})[f'{d_model}_{S}_{hd}'] = dict(cos_sha=sha(c), sin_sha=sha(s))
        if d_model == 768:
            A['rope768_cos_rows'] = c[[0, 1, 2, 63, 1000, 4095]]
            A['rope768_sin_rows'] = s[[0, 1, 2, 63, 1000, 4095]]
    q, k = inputs.rope_qk()
    rope = ref.RotaryPositionalEmbedding(768, 4096)
    cos, sin = rope(q.shape[2])
    for name, dt in (('f16', torch.float16), ('bf16', torch.bfloat16)):
        qe, ke = ref.apply_rotary_pos_emb(q.to(dt), k.to(dt), cos, sin)
        assert qe.dtype == torch.float32
        A[f'rope_q_{name}'] = qe.to(dt).view(torch.int16).numpy()
        A[f'rope_k_{name}'] = ke.to(dt).view(torch.int16).numpy()
        # autograd adjoint of the eager path in fp32 (the fused bwd rounds once from this)
        q0 = q.to(dt).float().requires_grad_(True)
        k0 = k.to(dt).float().requires_grad_(True)
        qe, ke = ref.apply_rotary_pos_emb(q0, k0, cos, sin)
        gq, gk = inputs.rope_grads()
        (qe * gq.to(dt).float()).sum().backward(retain_graph=True)
        (ke * gk.to(dt).float()).sum().backward()
        A[f'rope_dq_{name}'] = q0.grad.numpy()
        A[f'rope_dk_{name}'] = k0.grad.numpy()

    # ---- attention: the reference's SDPA call (train.py:1956) in fp32 ----
    q, k, v, do = inputs.attn_small()
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    o = F.scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=True)
    o.backward(do)
    A['attn_o'], A['attn_dq'], A['attn_dk'], A['attn_dv'] = (
        o.detach().numpy(), q.grad.numpy(), k.grad.numpy(), v.grad.numpy())

    # ---- RMSNorm (train.py:1862) ----
    x, w, dy = inputs.rms_small()
    m = ref.FusedRMSNorm(x.shape[-1])
    with torch.no_grad():
        m.weight.copy_(w)
    x.requires_grad_(True)
    y = m(x)
    y.backward(dy)
    A['rms_y'], A['rms_dx'], A['rms_dw'] = y.detach().numpy(), x.grad.numpy(), m.weight.grad.numpy()

    # ---- tiny model: one loss + grads (train.py:2059) ----
    cfg = ref.ModelConfig(**inputs.TINY_MODEL, dropout=0.0, use_rope=True, tie_weights=True,
                          use_fp16=False, use_compile=False, use_gradient_checkpointing=False)
    model = ref.DecoderOnlyTransformer(cfg)
    inputs.load_seeded_weights_into_reference(model)
    ids = torch.from_numpy(ref.collate_pad(inputs.tiny_batch(), eos_id=3, bos_id=2, max_len=256).numpy())
    loss = model.compute_loss(ids, ignore_index=0, chunk_rows=256)
    loss.backward()
    G['tiny_loss'] = float(loss)
    G['tiny_ids_sha'] = sha(ids.numpy())
    G['tiny_grad_norms'] = {n: float(p.grad.norm()) for n, p in model.named_parameters()}
    A['tiny_emb_grad_rows'] = model.embedding.weight.grad[:8].numpy()

    # chunked CE on its own (body of compute_loss after forward_hidden)
    h, W, t = inputs.ce_small()
    h.requires_grad_(True), W.requires_grad_(True)
    n_tok = (t != 0).sum().clamp(min=1)
    total = None
    for i in range(0, h.shape[0], 64):
        part = F.cross_entropy(F.linear(h[i:i + 64], W), t[i:i + 64], ignore_index=0, reduction='sum')
        total = part if total is None else total + part
    loss = total / n_tok
    loss.backward()
    G['ce_loss'] = float(loss)
    A['ce_dh'], A['ce_dw'] = h.grad.numpy(), W.grad.numpy()

    # ---- state_dict layout of the reference model (train.py:1996-2031, 1877-1891) ----
    # head_dim-64 toy (the shape the CUDA model accepts): names and shapes of every entry, and the
    # bits of the RoPE buffers, so the product model can be checked for strict two-way loadability
    cfg64 = ref.ModelConfig(**inputs.TINY64_MODEL, dropout=0.0, use_rope=True, tie_weights=True,
                            use_fp16=False, use_compile=False, use_gradient_checkpointing=False)
    sd = ref.DecoderOnlyTransformer(cfg64).state_dict()
    G['state_dict_tiny64'] = {k: [list(v.shape), str(v.dtype)] for k, v in sd.items()}
    G['state_dict_tiny64_rope_sha'] = {k: sha(sd[k].numpy()) for k in ('rope.inv_freq', 'rope.cos_cached', 'rope.sin_cached')}

    # ---- dropout keep mask (csrc/flash_attn_v100/fa_common.cuh:21-38) from the reference's own source ----
    # compiled for the host by oracle/ref_build.py; blocks are stored bit-packed
    from oracle import ref_build
    ref_build.build_ref(REF)
    hlib = ref_build.load_ref()
    G['hash_u32'] = {str(x): int(hlib.ref_hash_u32(x)) for x in (0, 1, 2, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFF, 0x9E3779B1, 123456789)}
    G['dropout_keep_cases'] = []
    for i, (seed, bh, p_drop, row0, nrows, col0, ncols) in enumerate(inputs.DROPOUT_CASES):
        blk = ref_build.ref_keep_block(hlib, seed, bh, p_drop, row0, nrows, col0, ncols)
        A[f'dropout_keep_{i}'] = np.packbits(blk, axis=None)
        G['dropout_keep_cases'].append(dict(seed=seed, bh=bh, p=p_drop, row0=row0, nrows=nrows, col0=col0, ncols=ncols,
                                            kept=int(blk.sum())))

    G['meta'] = dict(torch=torch.__version__, numpy=np.__version__,
                     note='generated by importing the reference train.py on CPU, 1 thread')
    with open(os.path.join(HERE, 'golden.json'), 'w') as f:
        json.dump(G, f, indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, 'golden.npz'), **A)
    print('wrote golden.json, golden.npz:', {k: v.shape for k, v in A.items()})


if __name__ == '__main__':
    main()
