"""RMSNorm, the SwiGLU gate and chunked cross-entropy on the sm_100a library, as autograd ops.

The reference has no custom kernels for these: ``FusedRMSNorm`` calls
F.rms_norm (train.py:1862-1875) and ``compute_loss`` loops fc_out +
F.cross_entropy over row chunks (train.py:2059-2082).  The classes and functions
below keep those names and argument meanings.
"""
import contextlib
import ctypes as C

import torch
import torch.nn as nn

import _native as N

_DT = {torch.float16: N.ULM_F16, torch.bfloat16: N.ULM_BF16, torch.float32: N.ULM_F32}


def _stream(t=None):
    """torch's current stream on the tensor's device (or the current device)."""
    return N.current_stream(t.device.index if t is not None and t.device.index is not None else torch.cuda.current_device())


def _rows(x):
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    if x2.stride(1) != 1 or x2.data_ptr() % 16 or (x2.stride(0) * x2.element_size()) % 16:
        x2 = x2.contiguous()
    return x2


_KIND = {torch.float16: N.ULM_Y_F16, torch.bfloat16: N.ULM_Y_BF16}


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, out_dtype):
        lib = N.lib()
        x2 = _rows(x)
        rows, d = x2.shape
        y = torch.empty((rows, d), dtype=out_dtype, device=x.device)
        rstd = torch.empty((rows,), dtype=torch.float32, device=x.device)
        w = weight if weight.dtype in (x.dtype, torch.float32) else weight.float()
        w = w.contiguous()
        kind = N.ULM_Y_SAME if out_dtype == x.dtype else _KIND[out_dtype]
        a = N.RmsFwdArgs(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(),
                         x2.stride(0), y.stride(0), rows, d, _DT[x.dtype], _DT[w.dtype],
                         float(eps), _stream(), kind, 0)
        N.check(lib.ulm_rmsnorm_fwd(C.byref(a)), 'rms_norm forward')
        ctx.save_for_backward(x2, w, rstd)
        ctx.eps, ctx.shape, ctx.wdtype, ctx.ydtype, ctx.kind = float(eps), x.shape, weight.dtype, out_dtype, kind
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        lib = N.lib()
        x2, w, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = _rows(dy if dy.dtype == ctx.ydtype else dy.to(ctx.ydtype))
        dx = torch.empty_like(x2)
        dw = torch.empty((d,), dtype=torch.float32, device=x2.device)
        parts = int(lib.ulm_rmsnorm_bwd_partial_rows(rows))
        partial = torch.empty((parts, d), dtype=torch.float32, device=x2.device)
        a = N.RmsBwdArgs(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                         dw.data_ptr(), partial.data_ptr(), x2.stride(0), dy2.stride(0), dx.stride(0),
                         rows, d, _DT[x2.dtype], _DT[w.dtype], ctx.eps, _stream(), ctx.kind, 0)
        N.check(lib.ulm_rmsnorm_bwd(C.byref(a)), 'rms_norm backward')
        return dx.view(ctx.shape), dw.to(ctx.wdtype), None, None


def rms_norm(x, weight, eps: float = 1e-6, out_dtype=None):
    """``weight * x * rsqrt(mean(x^2, -1) + eps)``; fp32 reduction.  The output has x's dtype,
    except that an fp32 x under CUDA autocast gives the autocast dtype directly: F.rms_norm
    (train.py:1872) would return fp32 there and the Linear that follows would round it to 16 bits,
    so rounding the fp32 result once in the kernel yields the same values and saves the cast pass
    (and, in the backward, the cast of the 16-bit gradient back to fp32).  ``out_dtype`` overrides."""
    if not x.is_cuda or x.dtype not in _DT:
        raise ValueError('rms_norm needs a CUDA fp16/bf16/fp32 tensor')
    if out_dtype is None:
        out_dtype = x.dtype
        if x.dtype == torch.float32 and torch.is_autocast_enabled('cuda'):
            out_dtype = torch.get_autocast_dtype('cuda')
    if out_dtype != x.dtype and not (x.dtype == torch.float32 and out_dtype in _KIND):
        raise ValueError('rms_norm: a different output dtype needs an fp32 input and a 16-bit output')
    return _RMSNorm.apply(x, weight, eps, out_dtype)


class _AddRMSNorm(torch.autograd.Function):
    """x_new = x + branch, y = rms_norm(x_new) in one pass each way (see add_rms_norm)."""

    @staticmethod
    def forward(ctx, x, branch, weight, eps):
        lib = N.lib()
        x2, b2 = _rows(x), _rows(branch)
        rows, d = x2.shape
        x_new = torch.empty((rows, d), dtype=torch.float32, device=x.device)
        y = torch.empty((rows, d), dtype=branch.dtype, device=x.device)
        rstd = torch.empty((rows,), dtype=torch.float32, device=x.device)
        w = weight.float().contiguous()
        kind = _KIND[branch.dtype]
        a = N.RmsFwdArgs(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), x2.stride(0), y.stride(0), rows, d,
                         N.ULM_F32, N.ULM_F32, float(eps), _stream(), kind, 0,
                         b2.data_ptr(), x_new.data_ptr(), b2.stride(0), x_new.stride(0))
        N.check(lib.ulm_rmsnorm_fwd(C.byref(a)), 'add_rms_norm forward')
        ctx.save_for_backward(x_new, w, rstd)
        ctx.eps, ctx.shape, ctx.wdtype, ctx.kind, ctx.bdtype = float(eps), x.shape, weight.dtype, kind, branch.dtype
        return x_new.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, g_x, g_y):
        lib = N.lib()
        x_new, w, rstd = ctx.saved_tensors
        rows, d = x_new.shape
        if g_y is None:                                   # the normalised output went unused
            g = g_x if g_x is not None else torch.zeros(ctx.shape, dtype=torch.float32, device=x_new.device)
            return g, g.to(ctx.bdtype), None, None
        dy2 = _rows(g_y if g_y.dtype == ctx.bdtype else g_y.to(ctx.bdtype))
        ga = _rows(g_x.float()) if g_x is not None else None
        dx = torch.empty_like(x_new)
        d_branch = torch.empty((rows, d), dtype=ctx.bdtype, device=x_new.device)
        dw = torch.empty((d,), dtype=torch.float32, device=x_new.device)
        partial = torch.empty((int(lib.ulm_rmsnorm_bwd_partial_rows(rows)), d), dtype=torch.float32, device=x_new.device)
        a = N.RmsBwdArgs(x_new.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                         partial.data_ptr(), x_new.stride(0), dy2.stride(0), dx.stride(0), rows, d, N.ULM_F32, N.ULM_F32,
                         ctx.eps, _stream(), ctx.kind, 0,
                         ga.data_ptr() if ga is not None else None, d_branch.data_ptr(),
                         ga.stride(0) if ga is not None else 0, d_branch.stride(0))
        N.check(lib.ulm_rmsnorm_bwd(C.byref(a)), 'add_rms_norm backward')
        return dx.view(ctx.shape), d_branch.view(ctx.shape), dw.to(ctx.wdtype), None


def add_rms_norm(x, branch, weight, eps: float = 1e-6):
    """The residual add in front of a norm fused with that norm: ``x_new = x + branch`` (train.py:1989,
    1993) and ``y = rms_norm(x_new)`` (the next norm: train.py:1991, 1988 of the following block, or 2054)
    in one pass over memory; returns ``(x_new, y)``.  x is the fp32 residual stream, branch the 16-bit
    output of the attention or feed-forward projection under autocast; x_new is fp32 and y has branch's
    dtype -- the values the unfused sequence (add in fp32, F.rms_norm in fp32, autocast's cast in front
    of the next Linear) produces.  The backward adds the gradient arriving at x_new to rms_norm's and
    writes the sum once, as the fp32 gradient of x and, rounded, as the 16-bit gradient of branch."""
    if not (x.is_cuda and x.dtype == torch.float32 and branch.dtype in _KIND and branch.shape == x.shape):
        raise ValueError('add_rms_norm needs an fp32 CUDA x and a 16-bit branch of the same shape')
    if x.shape[-1] > 1024 or x.shape[-1] % 4:
        raise ValueError('add_rms_norm takes rows of at most 1024 elements, a multiple of 4')
    return _AddRMSNorm.apply(x, branch, weight, eps)


class FusedRMSNorm(nn.Module):
    """train.py:1862-1875."""

    def __init__(self, d_model: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d_model))
        self.eps = eps

    def forward(self, x):
        return rms_norm(x, self.weight, self.eps)

    def add_forward(self, x, branch):
        """(x + branch, norm(x + branch)); the fused kernel when the tensors have the training layout
        (fp32 residual stream, 16-bit branch, d <= 1024), the two separate ops otherwise."""
        if (x.is_cuda and x.dtype == torch.float32 and branch.dtype in _KIND and x.shape[-1] <= 1024
                and x.shape[-1] % 4 == 0 and torch.is_autocast_enabled('cuda')
                and torch.get_autocast_dtype('cuda') == branch.dtype):
            return add_rms_norm(x, branch, self.weight, self.eps)
        x = x + branch
        return x, rms_norm(x, self.weight, self.eps)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        lib = N.lib()
        a, b = a.contiguous(), b.contiguous()
        y = torch.empty_like(a)
        args = N.SwigluArgs(a.data_ptr(), b.data_ptr(), y.data_ptr(), None, None, None, a.numel(),
                            _DT[a.dtype], 0, _stream())
        N.check(lib.ulm_swiglu_fwd(C.byref(args)), 'swiglu forward')
        ctx.save_for_backward(a, b)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = N.lib()
        a, b = ctx.saved_tensors
        dy = dy.to(a.dtype).contiguous()
        da, db = torch.empty_like(a), torch.empty_like(b)
        args = N.SwigluArgs(a.data_ptr(), b.data_ptr(), None, dy.data_ptr(), da.data_ptr(), db.data_ptr(),
                            a.numel(), _DT[a.dtype], 0, _stream())
        N.check(lib.ulm_swiglu_bwd(C.byref(args)), 'swiglu backward')
        return da, db


def swiglu(a, b):
    """``F.silu(a) * b`` (the gate of train.py:1966-1975's feed-forward) in one kernel each way."""
    if not a.is_cuda or a.dtype not in _DT or b.dtype != a.dtype or b.shape != a.shape:
        raise ValueError('swiglu needs two CUDA tensors of one shape and one of fp16/bf16/fp32')
    return _SwiGLU.apply(a, b)


# ---------------------------------------------------------------------------
# Bias-free linear layers with the weight gradient accumulated where it lives
# ---------------------------------------------------------------------------
_WGRAD_IN_PLACE = False


@contextlib.contextmanager
def wgrad_in_place(enabled=True):
    """While active, `linear` and `chunked_cross_entropy` add their weight gradients straight into an
    existing fp32 ``weight.grad`` with one GEMM (16-bit operands, fp32 accumulation and output, beta = 1)
    instead of returning a 16-bit product that autograd casts and adds in two more passes per parameter
    and micro-batch.  The caller owns the gradient buffers (they must exist, be zeroed per step, and no
    post-accumulate hook may be waiting for these parameters): `ulm_dp.DataParallelStep` does."""
    global _WGRAD_IN_PLACE
    prev, _WGRAD_IN_PLACE = _WGRAD_IN_PLACE, bool(enabled)
    try:
        yield
    finally:
        _WGRAD_IN_PLACE = prev


def _weight_grad(weight, dy2d, x2d):
    """dW = dy^T x for autograd, or None after adding it into ``weight.grad`` in place."""
    g = weight.grad
    if (_WGRAD_IN_PLACE and g is not None and g.dtype == torch.float32 and g.is_contiguous() and dy2d.is_cuda
            and dy2d.dtype in (torch.float16, torch.bfloat16)):
        torch.addmm(g, dy2d.t(), x2d, out_dtype=torch.float32, out=g)
        return None
    return (dy2d.t() @ x2d).to(weight.dtype)


_CAST_SCOPE = None      # identity of the active weight-cast scope, or None: no caching


@contextlib.contextmanager
def weight_cast_scope():
    """While active, `linear` keeps the 16-bit copy it makes of a weight and reuses it: the caller promises
    that the weights do not change inside the scope (one optimiser step's forward/backward calls).  Nothing
    is reused across scopes or outside one -- a parameter's version counter cannot be relied on for that
    (fused optimisers update parameters without bumping it)."""
    global _CAST_SCOPE
    prev, _CAST_SCOPE = _CAST_SCOPE, object()
    try:
        yield
    finally:
        _CAST_SCOPE = prev


def _cast_cached(weight, dtype):
    """The weight in the compute dtype (the parameter itself if it already has it)."""
    if weight.dtype == dtype:
        return weight
    scope = _CAST_SCOPE
    if scope is None:
        return weight.detach().to(dtype)
    c = getattr(weight, '_ulm_cast', None)
    if c is None or c[0] is not scope or c[1].dtype != dtype or c[1].device != weight.device:
        c = (scope, weight.detach().to(dtype))
        weight._ulm_cast = c
    return c[1]


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        cd = x.dtype
        if x.is_cuda and torch.is_autocast_enabled():
            cd = torch.get_autocast_dtype('cuda')
        xc = x if x.dtype == cd else x.to(cd)
        ctx.save_for_backward(xc, weight)
        ctx.cd, ctx.x_dtype = cd, x.dtype
        return torch.nn.functional.linear(xc, _cast_cached(weight, cd))

    @staticmethod
    def backward(ctx, dy):
        xc, weight = ctx.saved_tensors
        dy2d = dy.reshape(-1, dy.shape[-1])
        if dy2d.dtype != ctx.cd:
            dy2d = dy2d.to(ctx.cd)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = (dy2d @ _cast_cached(weight, ctx.cd)).view(xc.shape).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(weight, dy2d, xc.reshape(-1, xc.shape[-1]))
        return dx, dw


def linear(x, weight):
    """``x @ weight.T`` for the model's bias-free projections (train.py:1925-1926, 1969-1971) in the autocast
    dtype; see `wgrad_in_place` for what it does differently from ``nn.Linear`` in the backward."""
    return _Linear.apply(x, weight)


def ce_rows_forward(logits, target, ignore_index):
    """One logits tile [rows, V] -> (lse[rows], loss[rows]) in fp32."""
    lib = N.lib()
    rows, V = logits.shape
    lse = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    loss = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    a = N.CeFwdArgs(logits.data_ptr(), target.data_ptr(), lse.data_ptr(), loss.data_ptr(),
                    logits.stride(0), rows, V, _DT[logits.dtype], int(ignore_index), _stream())
    N.check(lib.ulm_ce_fwd(C.byref(a)), 'cross-entropy forward')
    return lse, loss


def lm_head_lse(hidden, weight, target=None, ignore_index=0, keep_logits=True):
    """The lm-head GEMM with the loss statistics taken in its epilogue (one tcgen05 kernel + a per-row
    finishing kernel): hidden [rows, d] and weight [V, d], both fp16 or both bf16 ->
    (lse [rows] fp32, loss [rows] fp32 or None, logits [rows, V] in the operands' dtype or None).
    With ``keep_logits`` the rounded logits are stored (the backward turns them into their gradient) and the
    per-row loss lse - z[target] is returned; without, only lse."""
    lib = N.lib()
    if hidden.dtype not in (torch.float16, torch.bfloat16) or weight.dtype != hidden.dtype:
        raise ValueError('lm_head_lse takes fp16 or bf16 operands of one dtype')
    if hidden.dim() != 2 or weight.dim() != 2 or hidden.shape[1] != weight.shape[1] or hidden.stride(1) != 1 or weight.stride(1) != 1:
        raise ValueError('lm_head_lse takes hidden [rows, d] and weight [V, d] with contiguous rows')
    rows, d = hidden.shape
    V = weight.shape[0]
    dev = hidden.device
    lse = torch.empty((rows,), dtype=torch.float32, device=dev)
    logits = torch.empty((rows, V), dtype=hidden.dtype, device=dev) if keep_logits else None
    loss = torch.empty((rows,), dtype=torch.float32, device=dev) if keep_logits and target is not None else None
    parts = int(lib.ulm_lmhead_lse_parts(V))
    part = torch.empty((2, max(rows, 1) * parts), dtype=torch.float32, device=dev)
    import flash_attn_v100_cuda as fa
    a = N.LmHeadLseArgs(hidden.data_ptr(), weight.data_ptr(), logits.data_ptr() if logits is not None else None,
                        target.data_ptr() if loss is not None else None, lse.data_ptr(),
                        loss.data_ptr() if loss is not None else None, part[0].data_ptr(), part[1].data_ptr(),
                        hidden.stride(0), weight.stride(0), logits.stride(0) if logits is not None else 0,
                        rows, V, d, _DT[hidden.dtype], 0, int(ignore_index), fa._status(dev).data_ptr(), _stream(hidden))
    N.check(lib.ulm_lmhead_lse(C.byref(a)), 'lm-head GEMM + LSE')
    return lse, loss, logits


def ce_rows_backward_(logits, target, lse, gscale_dev, ignore_index, gscale=1.0):
    """In place: logits <- (softmax - onehot) * gscale * gscale_dev[0] (0 on ignored rows)."""
    lib = N.lib()
    rows, V = logits.shape
    a = N.CeBwdArgs(logits.data_ptr(), target.data_ptr(), lse.data_ptr(),
                    gscale_dev.data_ptr() if gscale_dev is not None else None, float(gscale),
                    logits.stride(0), rows, V, _DT[logits.dtype], int(ignore_index), _stream())
    N.check(lib.ulm_ce_bwd(C.byref(a)), 'cross-entropy backward')
    return logits


# Largest [rows, V] 16-bit logits buffer the cross-entropy keeps between forward and backward.  Up to this size
# (2.1 GB for the 32768-row token budget at V = 32000: small change on a 180 GB part) the backward turns the
# kept logits into their gradient in place and runs ONE GEMM each for dH and dW over all rows; beyond it the
# loss falls back to the reference's chunk-by-chunk form, recomputing each chunk's logits in the backward.
KEEP_LOGITS_BYTES = 8 << 30

# The kept form takes its logits and their log-sum-exp from ONE kernel (`lm_head_lse`: tcgen05 GEMM with the
# statistics in its epilogue) where the shapes allow (d and V multiples of 64), instead of a library GEMM
# followed by a pass over the logits.  Measured at 32768 x 32000 x 768 in bf16 on B200: 1.44 ms against
# 1.25 + 0.45 ms, identical logits bits.
FUSED_LM_HEAD = True


class _ChunkedCE(torch.autograd.Function):
    """Loss of train.py:2069-2082.  The reference loops fc_out + F.cross_entropy over row chunks so that
    no fp32 [rows, V] tensor is ever alive (autograd still keeps each chunk's fp32 log-softmax).  Here only
    16-bit logits ever exist.  Two forms, same values:
      kept     logits of all rows are produced by one lm-head GEMM into one 16-bit buffer and kept; the
               backward rewrites them in place as (softmax - onehot) * g and runs one GEMM for dH and one
               for dW (5 launches per micro-batch in all, no recomputation);
      chunked  one [chunk_rows, V] tile at a time; the forward keeps one fp32 lse per row and the backward
               recomputes each tile with the lm-head GEMM (buffers beyond KEEP_LOGITS_BYTES)."""

    @staticmethod
    def forward(ctx, hidden, weight, target, ignore_index, chunk_rows, compute_dtype, denominator):
        rows = hidden.shape[0]
        wc = _cast_cached(weight, compute_dtype)
        if denominator is None:
            n_tokens = (target != ignore_index).sum().clamp(min=1).float()
        elif torch.is_tensor(denominator):
            n_tokens = denominator.to(device=hidden.device, dtype=torch.float32)
        else:
            # a host number stays a host number: turning it into a device tensor is a pageable host-to-device
            # copy, which makes the launching thread wait for the GPU (measured: 4.6 ms per micro-batch)
            n_tokens = float(denominator)
        keep = rows * weight.shape[0] * 2 <= KEEP_LOGITS_BYTES
        if keep:
            hc = hidden.to(compute_dtype)
            if (FUSED_LM_HEAD and hc.is_cuda and compute_dtype in (torch.float16, torch.bfloat16) and hc.shape[1] % 64 == 0
                    and wc.shape[0] % 64 == 0 and hc.is_contiguous() and wc.is_contiguous()):
                lse_all, loss, logits = lm_head_lse(hc, wc, target, ignore_index, keep_logits=True)
            else:
                logits = hc @ wc.t()
                lse_all, loss = ce_rows_forward(logits, target, ignore_index)
            total = loss.sum()
        else:
            logits = None
            lse_all = torch.empty((rows,), dtype=torch.float32, device=hidden.device)
            total = torch.zeros((), dtype=torch.float32, device=hidden.device)
            for i in range(0, rows, chunk_rows):
                tile = hidden[i:i + chunk_rows].to(compute_dtype) @ wc.t()
                lse, loss = ce_rows_forward(tile, target[i:i + chunk_rows], ignore_index)
                lse_all[i:i + chunk_rows] = lse
                total = total + loss.sum()
        tensors = [hidden, weight, target, lse_all] + ([logits] if keep else []) + ([n_tokens] if torch.is_tensor(n_tokens) else [])
        ctx.save_for_backward(*tensors)
        ctx.keep, ctx.n_tokens, ctx.consumed = keep, (None if torch.is_tensor(n_tokens) else n_tokens), False
        ctx.ignore_index, ctx.chunk_rows, ctx.compute_dtype = ignore_index, chunk_rows, compute_dtype
        return total / n_tokens

    @staticmethod
    def backward(ctx, gout):
        saved = list(ctx.saved_tensors)
        hidden, weight, target, lse_all = saved[:4]
        logits = saved[4] if ctx.keep else None
        n_tokens = ctx.n_tokens if ctx.n_tokens is not None else saved[-1]
        cd = ctx.compute_dtype
        wc = _cast_cached(weight, cd)
        g = (gout.float() / n_tokens).reshape(1)
        if ctx.keep:
            if ctx.consumed:
                raise RuntimeError('chunked_cross_entropy: the kept logits were turned into their gradient in place by the '
                                   'first backward; a second backward through the same graph is not supported')
            ctx.consumed = True
            hc = hidden.to(cd)
            dl = ce_rows_backward_(logits, target, lse_all, g, ctx.ignore_index)       # in place over the kept logits
            dh = (dl @ wc).to(hidden.dtype)
            return dh, _weight_grad(weight, dl, hc), None, None, None, None, None      # fp32 in place, or rounded to 16 bits once
        dh = torch.empty_like(hidden)
        dw = None
        for i in range(0, hidden.shape[0], ctx.chunk_rows):
            hc = hidden[i:i + ctx.chunk_rows].to(cd)
            dl = ce_rows_backward_(hc @ wc.t(), target[i:i + ctx.chunk_rows],
                                   lse_all[i:i + ctx.chunk_rows], g, ctx.ignore_index)
            dh[i:i + ctx.chunk_rows] = dl @ wc
            part = _weight_grad(weight, dl, hc)            # None: already added into weight.grad
            if part is not None:
                dw = part.float() if dw is None else dw.add_(part)
        return dh, (None if dw is None else dw.to(weight.dtype)), None, None, None, None, None


def chunked_cross_entropy(hidden, weight, target, ignore_index=0, chunk_rows=2048,
                          compute_dtype=None, denominator=None):
    """hidden [rows, d], weight [V, d] (the tied lm head), target int64 [rows]
    -> CE summed over targets != ignore_index and divided by their count
    (train.py:2069-2082), or by ``denominator`` when one is given."""
    if compute_dtype is None:
        compute_dtype = torch.get_autocast_dtype('cuda') if torch.is_autocast_enabled() else (
            hidden.dtype if hidden.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16)
    if hidden.shape[0] == 0:
        return torch.zeros((), device=hidden.device, requires_grad=True)
    return _ChunkedCE.apply(hidden, weight, target.contiguous(), int(ignore_index),
                            int(chunk_rows), compute_dtype, denominator)


_SUMSQ_SCRATCH = {}     # device index -> fp32 scratch for the per-CTA partial sums


def grad_unscale_sumsq_(flat_grad, inv_scale, out2):
    """flat fp32 grads *= inv_scale[0]; out2[0] += sum(g^2); out2[1] = 1 on inf/nan.
    The sum is formed in a fixed order (per-CTA partials, then one CTA), so it is
    bit-identical from call to call on the same values."""
    lib = N.lib()
    scratch = _SUMSQ_SCRATCH.get(flat_grad.device.index)
    if scratch is None:
        scratch = _SUMSQ_SCRATCH[flat_grad.device.index] = torch.empty(
            int(lib.ulm_grad_sumsq_partial_count()), dtype=torch.float32, device=flat_grad.device)
    N.check(lib.ulm_grad_unscale_sumsq(flat_grad.data_ptr(), flat_grad.numel(),
                                       inv_scale.data_ptr() if inv_scale is not None else None,
                                       out2.data_ptr(), scratch.data_ptr(), _stream()), 'grad_unscale_sumsq')
    return out2
