"""Drop-in for the reference's ``flash_attn_v100_cuda`` module on B200.

Same names, arguments and error behaviour as flash_attn_v100_cuda.py of
sunyi9161/Universal-LM-Trainer (the module train.py:82 imports and calls at
train.py:90,94,100,1912,1913,1950), backed by the sm_100a library
``libulm_b200.so`` through ctypes instead of a torch C++ extension:

    is_available()  build_error()  can_use(q,k,v)
    rope_can_use(q,k,cos2d,sin2d)  rope(q,k,cos2d,sin2d)
    flash_attn_v100(q,k,v,dropout_p=0.0,causal=True,softmax_scale=None)

Differences a caller can see: bf16 is accepted beside fp16; the attention
output has shape (B,H,S,64) like the reference's but is laid out (B,S,H,64) in
memory, so train.py:1963's ``transpose(1,2).contiguous()`` is a no-op; dO may be
strided.  There is no SDPA or CPU path in here: if the library cannot be loaded
the Functions raise, and train.py's own ``if`` decides what to do.

One addition: ``rope_flash_attn(q, k, v, cos2d, sin2d, ...)`` does what
``flash_attn_v100(*rope(q, k, cos2d, sin2d), v, ...)`` does (train.py:1913 +
1950) with the rotation of Q inside the attention forward and the adjoint
rotation of dQ and dK inside the backward's epilogues; only K still goes through
the stand-alone RoPE kernel.  Results are bit-identical to the two-call form.
"""
import ctypes as C
import itertools

import torch

import _native as N

_SEED_COUNTER = itertools.count(1)
_STATUS = {}            # device index -> uint32[1] tensor the kernels OR their timeout bits into
_16BIT = (torch.float16, torch.bfloat16)


_last_seed = 0          # seed of the most recent forward (tests rebuild the dropout mask from it)


def _next_seed():
    # flash_attn_v100_cuda.py:29-33: the mask is a pure function of the seed, so
    # backward only needs the integer back.
    global _last_seed
    _last_seed = (int(torch.cuda.initial_seed()) * 2654435761 + next(_SEED_COUNTER)) & 0xFFFFFFFF
    return _last_seed


def is_available():
    return N.available()


def build_error():
    return N.build_error()


def _dt(t):
    return N.ULM_F16 if t.dtype == torch.float16 else N.ULM_BF16


def _stream(t=None):
    """torch's current stream on the tensor's device (or the current device)."""
    return N.current_stream(t.device.index if t is not None and t.device.index is not None else torch.cuda.current_device())


def _status(dev):
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    s = _STATUS.get(index)
    if s is None:
        s = _STATUS[index] = torch.zeros(1, dtype=torch.int32, device=torch.device('cuda', index))
    return s


def check_status(device=None):
    """Raise if any kernel on ``device`` gave up on a barrier wait since the last
    call (synchronises; meant for step boundaries and tests)."""
    dev = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    s = _STATUS.get(index)
    if s is None:
        return
    bits = int(s.item())
    if bits:
        s.zero_()
        raise RuntimeError(f'attention kernel reported a barrier timeout (status bits {bits:#x})')


def _fa_ready(t):
    """flash_attn_v100_cuda.py:97-102, with bf16 admitted: (B,H,S,64), innermost
    contiguous, 32-byte aligned base and strides."""
    return (t.is_cuda and t.dtype in _16BIT and t.dim() == 4
            and t.size(3) == 64 and t.stride(3) == 1
            and t.data_ptr() % 32 == 0
            and all((s * 2) % 32 == 0 for s in t.stride()[:3])
            and all(s > 0 or n == 1 for s, n in zip(t.stride()[:3], t.shape[:3]))
            and (t.size(2) == 1 or t.stride(2) >= 64))


def can_use(q, k, v):
    return (_fa_ready(q) and _fa_ready(k) and _fa_ready(v)
            and q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype)


def _empty_bshd(B, H, S, like):
    """(B,H,S,64) tensor stored as (B,S,H,64)."""
    return torch.empty((B, S, H, 64), dtype=like.dtype, device=like.device).transpose(1, 2)


def _strides3(t):
    return t.stride(0), t.stride(1), t.stride(2)


def attn_forward(q, k, v, dropout_p, causal, softmax_scale, seed, cos=None, sin=None, want_q_rot=True, o_out=None):
    """The reference's ``fa_fwd`` (flash_attn_v100.cu:337-364): returns (o, lse, q_rot).
    With ``cos``/``sin`` (fp32 [S,64] views) q is taken unrotated and rotated inside the
    kernel; q_rot is the rotated copy the backward needs (None without tables).  ``o_out``: a
    preallocated (B,H,S,64) view to write the output into."""
    lib = N.lib()
    B, H, S, _ = q.shape
    o = o_out if o_out is not None else _empty_bshd(B, H, S, q)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    q_rot = None
    cos_p = sin_p = qr_p = None
    cos_s = sin_s = 0
    qr_s = (0, 0, 0)
    if cos is not None:
        cos_p, sin_p, cos_s, sin_s = cos.data_ptr(), sin.data_ptr(), cos.stride(0), sin.stride(0)
        if want_q_rot:
            q_rot = _empty_bshd(B, H, S, q)
            qr_p, qr_s = q_rot.data_ptr(), _strides3(q_rot)
    # positional construction: field by field assignment costs 4x as much host time per launch
    a = N.AttnFwdArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                      *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(o),
                      B, H, S, _dt(q), int(bool(causal)), float(softmax_scale), float(dropout_p), int(seed),
                      _status(q.device).data_ptr(), _stream(), cos_p, sin_p, cos_s, sin_s, qr_p, *qr_s)
    N.check(lib.ulm_attn_fwd(C.byref(a)), 'flash_attn_v100 forward')
    return o, lse, q_rot


class _FlashAttnV100Cuda(torch.autograd.Function):
    """flash_attn_v100_cuda.py:69-94."""

    @staticmethod
    def forward(ctx, q, k, v, dropout_p, causal, softmax_scale):
        seed = _next_seed()
        o, lse, _ = attn_forward(q, k, v, dropout_p, causal, softmax_scale, seed)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.dropout_p, ctx.causal = float(dropout_p), bool(causal)
        ctx.softmax_scale, ctx.seed = float(softmax_scale), seed
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attn_backward(q, k, v, o, lse, do, ctx.dropout_p, ctx.causal,
                                   ctx.softmax_scale, ctx.seed)
        return dq, dk, dv, None, None, None


def attn_backward(q, k, v, o, lse, do, dropout_p, causal, softmax_scale, seed, mode=7,
                  delta=None, cos=None, sin=None, out=None):
    """The reference's ``fa_bwd`` (flash_attn_v100_bwd.cu:433-506): returns
    (dq, dk, dv); ``mode`` selects delta / dQ / dK,dV passes like its bitmask.
    With ``cos``/``sin`` q and k are the rotated tensors and dq, dk come back as the
    gradients of the unrotated ones (adjoint rotation in the kernels' epilogues)."""
    lib = N.lib()
    B, H, S, _ = q.shape
    if not _fa_ready(do):
        do = do.contiguous()
    if not _fa_ready(o):
        o = o.contiguous()
    if out is None:
        buf = torch.empty((3, B, S, H, 64), dtype=q.dtype, device=q.device)
        dq, dk, dv = (buf[i].transpose(1, 2) for i in range(3))
    else:
        dq, dk, dv = out                                   # caller's (B,H,S,64) views, any 8-element-aligned strides
    if delta is None:
        delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    cos_p = sin_p = None
    cos_s = sin_s = 0
    if cos is not None:
        cos_p, sin_p, cos_s, sin_s = cos.data_ptr(), sin.data_ptr(), cos.stride(0), sin.stride(0)
    a = N.AttnBwdArgs(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                      dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                      *_strides3(q), *_strides3(k), *_strides3(v), *_strides3(o), *_strides3(do),
                      *_strides3(dq), *_strides3(dk), *_strides3(dv),
                      B, H, S, _dt(q), int(bool(causal)), int(mode), float(softmax_scale), float(dropout_p), int(seed),
                      _status(q.device).data_ptr(), _stream(), cos_p, sin_p, cos_s, sin_s)
    N.check(lib.ulm_attn_bwd(C.byref(a)), 'flash_attn_v100 backward')
    return dq, dk, dv


def _rope_out_like(x):
    """Dense output in the input's memory order (fast_ops.cu:142-150): fused-qkv
    views come back as (B,S,H,64)-ordered tensors, not 3x-sized copies."""
    B, H, S, D = x.shape
    dense = sum((n - 1) * s for n, s in zip(x.shape, x.stride())) + 1 == x.numel()
    if dense:
        return torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    if x.stride(1) == D and x.stride(2) >= H * D:
        return torch.empty((B, S, H, D), dtype=x.dtype, device=x.device).transpose(1, 2)
    return torch.empty((B, H, S, D), dtype=x.dtype, device=x.device)


def _rope_launch(q, k, cos, sin, backward, shape_like=None, out=None):
    """q may be None: only k is rotated then (and None comes back in q's place).  ``out`` = (qo, ko)
    preallocated (B,H,S,64) views to write into."""
    lib = N.lib()
    ref_q, ref_k = shape_like if shape_like is not None else (q, k)
    ko = out[1] if out is not None else _rope_out_like(ref_k)
    a = N.RopeArgs()
    a.k, a.ko = k.data_ptr(), ko.data_ptr()
    a.k_sb, a.k_sh, a.k_ss = _strides3(k)
    a.ko_sb, a.ko_sh, a.ko_ss = _strides3(ko)
    qo = None
    if q is not None:
        qo = out[0] if out is not None else _rope_out_like(ref_q)
        a.q, a.qo = q.data_ptr(), qo.data_ptr()
        a.q_sb, a.q_sh, a.q_ss = _strides3(q)
        a.qo_sb, a.qo_sh, a.qo_ss = _strides3(qo)
    a.cos_tab, a.sin_tab = cos.data_ptr(), sin.data_ptr()
    a.cos_stride, a.sin_stride = cos.stride(0), sin.stride(0)
    a.B, a.H, a.S = k.shape[0], k.shape[1], k.shape[2]
    a.dtype, a.backward = _dt(k), int(backward)
    a.stream = _stream()
    N.check(lib.ulm_rope(C.byref(a)), 'rope')
    return qo, ko


class _RopeV100Cuda(torch.autograd.Function):
    """flash_attn_v100_cuda.py:111-138: fused RoPE, one kernel each way."""

    @staticmethod
    def forward(ctx, q, k, cos, sin):
        qo, ko = _rope_launch(q, k, cos, sin, backward=False)
        ctx.save_for_backward(q, k, cos, sin)
        return qo, ko

    @staticmethod
    def backward(ctx, dqo, dko):
        q, k, cos, sin = ctx.saved_tensors
        # A branch whose output went unused arrives as None: run the kernel on
        # zeros for it but hand None back (flash_attn_v100_cuda.py:124-138).
        q_unused, k_unused = dqo is None, dko is None
        if q_unused and k_unused:
            return None, None, None, None
        dqo = torch.zeros_like(q) if q_unused else (dqo if _rope_grad_ready(dqo) else dqo.contiguous())
        dko = torch.zeros_like(k) if k_unused else (dko if _rope_grad_ready(dko) else dko.contiguous())
        dq, dk = _rope_launch(dqo, dko, cos, sin, backward=True, shape_like=(q, k))
        return (None if q_unused else dq), (None if k_unused else dk), None, None


def _rope_grad_ready(t):
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3]))


def rope_can_use(q, k, cos, sin):
    """flash_attn_v100_cuda.py:141-147 (plus the 16-byte table alignment the
    vector loads here need)."""
    return (_fa_ready(q) and _fa_ready(k)
            and q.shape == k.shape and q.dtype == k.dtype
            and cos.dtype == torch.float32 and sin.dtype == torch.float32
            and cos.device == q.device and sin.device == q.device
            and cos.shape == (q.size(2), 64) and sin.shape == cos.shape
            and cos.stride(1) == 1 and sin.stride(1) == 1
            and cos.stride(0) % 4 == 0 and sin.stride(0) % 4 == 0
            and cos.data_ptr() % 16 == 0 and sin.data_ptr() % 16 == 0)


def rope(q, k, cos2d, sin2d):
    """q,k: (B,H,S,64) 16-bit views of any stride; cos2d/sin2d: fp32 (S,64), rows may be padded."""
    return _RopeV100Cuda.apply(q, k, cos2d, sin2d)


def flash_attn_v100(q, k, v, dropout_p: float = 0.0, causal: bool = True, softmax_scale=None):
    """flash_attn_v100_cuda.py:155-166."""
    if not (q.is_cuda and q.dtype in _16BIT and q.size(3) == 64):
        raise ValueError('flash_attn_v100 needs CUDA fp16/bf16 inputs with head_dim 64')
    if not _fa_ready(q) or not _fa_ready(k) or not _fa_ready(v):
        q, k, v = (t if _fa_ready(t) else t.contiguous() for t in (q, k, v))
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    return _FlashAttnV100Cuda.apply(q, k, v, float(dropout_p), bool(causal), float(softmax_scale))


# Where the RoPE work of rope_flash_attn / qkv_rope_flash_attn runs.  All three give the same bits.
#   'none'  stand-alone RoPE kernel on q and k, plain attention kernels, stand-alone RoPE adjoint kernel
#   'fwd'   Q rotated inside the attention forward (K through the stand-alone kernel), backward as 'none'
#   'all'   as 'fwd', and the adjoint applied in the dQ / dK epilogues of the backward kernels
# Measured at B=8, H=12, S=4096 on B200 the forward fusion costs what it saves (the rotation sits on each
# CTA's start-up path) and the backward fusion costs more than the launch it removes (the epilogue of a
# persistent in-order pipeline is on its critical path), so 'none' is the default; profiles/ has the numbers.
ROPE_FUSION = 'none'


def _rope_attn_forward(q, k, v, cos, sin, dropout_p, causal, softmax_scale, seed, fuse, o_out=None):
    """-> (o, lse, q_rot, k_rot)"""
    if fuse == 'none':
        q_rot, k_rot = _rope_launch(q, k, cos, sin, backward=False)
        o, lse, _ = attn_forward(q_rot, k_rot, v, dropout_p, causal, softmax_scale, seed, o_out=o_out)
    else:
        _, k_rot = _rope_launch(None, k, cos, sin, backward=False)
        o, lse, q_rot = attn_forward(q, k_rot, v, dropout_p, causal, softmax_scale, seed, cos=cos, sin=sin, o_out=o_out)
    return o, lse, q_rot, k_rot


def _rope_attn_backward(q_rot, k_rot, v, o, lse, do, cos, sin, dropout_p, causal, softmax_scale, seed, fuse, out=None):
    """-> (dq, dk, dv) of the UNROTATED q, k and of v; ``out`` = three preallocated (B,H,S,64) views."""
    if fuse == 'all':
        return attn_backward(q_rot, k_rot, v, o, lse, do, dropout_p, causal, softmax_scale, seed, cos=cos, sin=sin, out=out)
    if out is None:
        dqr, dkr, dv = attn_backward(q_rot, k_rot, v, o, lse, do, dropout_p, causal, softmax_scale, seed)
        dq, dk = _rope_launch(dqr, dkr, cos, sin, backward=True)
        return dq, dk, dv
    B, H, S, _ = q_rot.shape
    tmp = torch.empty((2, B, S, H, 64), dtype=q_rot.dtype, device=q_rot.device)
    dqr, dkr = tmp[0].transpose(1, 2), tmp[1].transpose(1, 2)
    attn_backward(q_rot, k_rot, v, o, lse, do, dropout_p, causal, softmax_scale, seed, out=(dqr, dkr, out[2]))
    _rope_launch(dqr, dkr, cos, sin, backward=True, out=(out[0], out[1]))
    return out


class _RopeFlashAttn(torch.autograd.Function):
    """RoPE + attention as one differentiable op: what ``_RopeV100Cuda`` followed by
    ``_FlashAttnV100Cuda`` compute (flash_attn_v100_cuda.py:111-138, 69-94).  Saves the rotated
    q and k (the backward recomputes the scores from them), not the unrotated ones."""

    @staticmethod
    def forward(ctx, q, k, v, cos, sin, dropout_p, causal, softmax_scale, fuse):
        seed = _next_seed()
        o, lse, q_rot, k_rot = _rope_attn_forward(q, k, v, cos, sin, dropout_p, causal, softmax_scale, seed, fuse)
        ctx.save_for_backward(q_rot, k_rot, v, o, lse, cos, sin)
        ctx.args = (float(dropout_p), bool(causal), float(softmax_scale), seed, fuse)
        return o

    @staticmethod
    def backward(ctx, do):
        q_rot, k_rot, v, o, lse, cos, sin = ctx.saved_tensors
        dq, dk, dv = _rope_attn_backward(q_rot, k_rot, v, o, lse, do, cos, sin, *ctx.args)
        return dq, dk, dv, None, None, None, None, None, None


def rope_flash_attn(q, k, v, cos2d, sin2d, dropout_p: float = 0.0, causal: bool = True, softmax_scale=None, fuse=None):
    """``flash_attn_v100(*rope(q, k, cos2d, sin2d), v, ...)`` as one op (see the module docstring);
    ``fuse`` picks where the RoPE work runs (default: ROPE_FUSION).  Inputs must satisfy
    ``rope_can_use`` and ``can_use``; there is no other path."""
    if not (rope_can_use(q, k, cos2d, sin2d) and can_use(q, k, v)):
        raise ValueError('rope_flash_attn needs 16-bit (B,H,S,64) CUDA views and fp32 (S,64) tables')
    fuse = ROPE_FUSION if fuse is None else fuse
    if fuse not in ('none', 'fwd', 'all'):
        raise ValueError("fuse must be 'none', 'fwd' or 'all'")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    return _RopeFlashAttn.apply(q, k, v, cos2d, sin2d, float(dropout_p), bool(causal), float(softmax_scale), fuse)


class _QkvRopeFlashAttn(torch.autograd.Function):
    """The attention block between the two projections of train.py:1934-1964 as one op on the FUSED
    projection output: qkv [n, L, 3*H*64] -> chunk into q, k, v (train.py:1935-1939), RoPE on q and k,
    causal attention, heads merged back to [n, L, H*64] (train.py:1963).  Nothing is copied that the
    reference copies around the kernels: q, k, v are strided views of qkv, the output comes out of the
    kernel in (n, L, H, 64) order, and the backward kernels write dq, dk, dv straight into the three
    slices of one [n, L, 3*H*64] gradient tensor (autograd would otherwise concatenate them)."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, n_heads, dropout_p, causal, softmax_scale, fuse, flat_shape=None):
        # flat_shape = (B, S): qkv is the flattened [T', 3*H*64] projection with T' >= B*S; the rows beyond B*S
        # are padding -- the output gets zero rows there and so does the gradient, without any copy
        if flat_shape is not None:
            B, S = flat_shape
            rows = qkv.shape[0]
            qkv3 = qkv[:B * S].view(B, S, qkv.shape[-1])
        else:
            B, S, _ = qkv.shape
            rows = None
            qkv3 = qkv
        q, k, v = (t.view(B, S, n_heads, 64).transpose(1, 2) for t in qkv3.chunk(3, dim=-1))
        seed = _next_seed()
        o_out = out2d = None
        if rows is not None:
            out2d = torch.empty((rows, n_heads * 64), dtype=qkv.dtype, device=qkv.device)
            out2d[B * S:].zero_()
            o_out = out2d[:B * S].view(B, S, n_heads, 64).transpose(1, 2)
        if cos is not None:
            o, lse, q, k = _rope_attn_forward(q, k, v, cos, sin, dropout_p, causal, softmax_scale, seed, fuse, o_out=o_out)
        else:
            o, lse, _ = attn_forward(q, k, v, dropout_p, causal, softmax_scale, seed, o_out=o_out)
        ctx.save_for_backward(q, k, v, o, lse, cos, sin)
        ctx.args = (float(dropout_p), bool(causal), float(softmax_scale), seed, fuse)
        ctx.rows = rows
        if rows is not None:
            return out2d
        return o.transpose(1, 2).reshape(B, S, n_heads * 64)          # a view: o is stored (B,S,H,64)

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, o, lse, cos, sin = ctx.saved_tensors
        B, H, S, _ = q.shape
        rows = ctx.rows
        if not d_out.is_contiguous():
            d_out = d_out.contiguous()
        do = (d_out if rows is None else d_out[:B * S]).view(B, S, H, 64).transpose(1, 2)
        if rows is None:
            d_qkv = torch.empty((B, S, 3, H, 64), dtype=q.dtype, device=q.device)
            d3 = d_qkv
        else:
            d_qkv = torch.empty((rows, 3, H, 64), dtype=q.dtype, device=q.device)
            d_qkv[B * S:].zero_()
            d3 = d_qkv[:B * S].view(B, S, 3, H, 64)
        out = tuple(d3[:, :, i].transpose(1, 2) for i in range(3))
        if cos is not None:
            _rope_attn_backward(q, k, v, o, lse, do, cos, sin, *ctx.args, out=out)
        else:
            attn_backward(q, k, v, o, lse, do, *ctx.args[:4], out=out)
        d_flat = d_qkv.view(B, S, 3 * H * 64) if rows is None else d_qkv.view(rows, 3 * H * 64)
        return d_flat, None, None, None, None, None, None, None, None


def qkv_rope_flash_attn(qkv, n_heads, cos2d=None, sin2d=None, dropout_p: float = 0.0, causal: bool = True,
                        softmax_scale=None, fuse=None, flat_shape=None):
    """qkv [n, L, 3*n_heads*64] (the fused projection, 16-bit, contiguous) -> attention output
    [n, L, n_heads*64]; RoPE with the fp32 (L,64) tables when they are given.  With ``flat_shape=(n, L)``
    qkv is the flattened [T', 3*n_heads*64] tensor with T' >= n*L (padding rows at the end) and the output is
    [T', n_heads*64] with zero padding rows: no copy either way."""
    if flat_shape is not None:
        n_, L_ = flat_shape
        if not (qkv.dim() == 2 and qkv.shape[0] >= n_ * L_):
            raise ValueError('flat_shape=(n, L) needs a 2-D qkv with at least n*L rows')
        probe = qkv[:n_ * L_].view(n_, L_, qkv.shape[-1])
    else:
        probe = qkv
    if not (qkv.is_cuda and qkv.dtype in _16BIT and probe.dim() == 3 and qkv.is_contiguous()
            and qkv.shape[-1] == 3 * n_heads * 64 and qkv.data_ptr() % 32 == 0):
        raise ValueError('qkv_rope_flash_attn needs a contiguous CUDA fp16/bf16 [n, L, 3*n_heads*64] tensor')
    if (cos2d is None) != (sin2d is None):
        raise ValueError('cos2d and sin2d must be given together')
    if cos2d is not None:
        L = probe.shape[1]
        ok = (cos2d.dtype == torch.float32 and sin2d.dtype == torch.float32 and cos2d.device == qkv.device
              and sin2d.device == qkv.device and cos2d.shape == (L, 64) and sin2d.shape == (L, 64)
              and cos2d.stride(1) == 1 and sin2d.stride(1) == 1 and cos2d.stride(0) % 4 == 0 and sin2d.stride(0) % 4 == 0
              and cos2d.data_ptr() % 16 == 0 and sin2d.data_ptr() % 16 == 0)
        if not ok:
            raise ValueError('RoPE tables must be fp32 (L,64) views on the same device, 16-byte aligned rows')
    fuse = ROPE_FUSION if fuse is None else fuse
    if fuse not in ('none', 'fwd', 'all'):
        raise ValueError("fuse must be 'none', 'fwd' or 'all'")
    if softmax_scale is None:
        softmax_scale = 64 ** -0.5
    if probe.shape[0] == 0 or probe.shape[1] == 0:
        shape = (qkv.shape[0], n_heads * 64) if flat_shape is not None else (qkv.shape[0], qkv.shape[1], n_heads * 64)
        return qkv.new_zeros(shape) + 0 * qkv.sum()
    return _QkvRopeFlashAttn.apply(qkv, cos2d, sin2d, int(n_heads), float(dropout_p), bool(causal), float(softmax_scale), fuse,
                                   None if flat_shape is None else (int(flat_shape[0]), int(flat_shape[1])))


def selftest_wait_timeout(limit_ns=2_000_000, device=None):
    """Launch the library's wait self-test: one bounded barrier wait of ``limit_ns`` on a
    barrier nothing arrives at.  The kernel returns by itself and leaves the timeout bit
    in the device's status word, where ``check_status`` finds it."""
    dev = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    N.check(N.lib().ulm_selftest_wait_timeout(int(limit_ns), _status(dev).data_ptr(), _stream()), 'selftest_wait_timeout')


def tensor_map_cache_stats():
    """(hits, misses) of the library's cache of encoded TMA tensor maps."""
    h, m = C.c_uint64(0), C.c_uint64(0)
    N.lib().ulm_tensor_map_cache_stats(C.byref(h), C.byref(m))
    return int(h.value), int(m.value)
