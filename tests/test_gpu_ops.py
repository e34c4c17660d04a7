"""GPU parity tests: every kernel is called through the C-ABI (ctypes wrappers)
and compared with the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

from oracle import ops

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]


@pytest.fixture(scope='module')
def fa():
    import flash_attn_v100_cuda as m
    assert torch.cuda.is_available(), 'these tests need a GPU'
    assert m.is_available(), m.build_error()
    return m


def randn(shape, seed, dtype=torch.float32, device='cuda'):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype).to(device)


def relerr(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp(min=1e-30))


# ---------------------------------------------------------------- RoPE ----
def qkv_views(B, H, S, dtype, seed, fused):
    """q, k, v as (B,H,S,64) views: dense, or slices of one fused [B,S,3*H*64] buffer
    like train.py:1934-1939 produces."""
    if fused:
        buf = randn((B, S, 3 * H * 64), seed, dtype)
        return tuple(t.view(B, S, H, 64).transpose(1, 2) for t in buf.chunk(3, dim=-1))
    return tuple(randn((B, H, S, 64), seed + i, dtype) for i in range(3))


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('fused', [False, True])
@pytest.mark.parametrize('B,H,S', [(1, 1, 1), (2, 3, 70), (1, 12, 257), (2, 12, 1024)])
def test_rope_bit_exact(fa, dtype, fused, B, H, S):
    q, k, _ = qkv_views(B, H, S, dtype, 11, fused)
    cos, sin = ops.rope_tables(768, 4096)
    cos2d, sin2d = cos.cuda()[:S, :64], sin.cuda()[:S, :64]       # row stride 768, like the model's table
    assert fa.rope_can_use(q, k, cos2d, sin2d)
    qo, ko = fa.rope(q, k, cos2d, sin2d)
    eq, ek = ops.apply_rope(q.cpu(), k.cpu(), cos[:S, :64], sin[:S, :64], out_dtype=dtype)
    assert torch.equal(qo.cpu(), eq) and torch.equal(ko.cpu(), ek)
    if fused:   # output is dense in the input's (B,S,H,D) order, not a 3x-sized copy
        assert qo.stride() == (S * H * 64, 64, H * 64, 1)
    gq, gk = randn((B, H, S, 64), 21, dtype), randn((B, H, S, 64), 22, dtype)
    q.requires_grad_(True), k.requires_grad_(True)
    qo, ko = fa.rope(q, k, cos2d, sin2d)
    torch.autograd.backward([qo, ko], [gq, gk])
    dq, dk = ops.rope_backward(gq.cpu(), gk.cpu(), cos[:S, :64], sin[:S, :64], out_dtype=dtype)
    assert torch.equal(q.grad.cpu(), dq) and torch.equal(k.grad.cpu(), dk)


def test_rope_unused_branch_gets_none(fa):
    q, k, _ = qkv_views(1, 2, 33, torch.float16, 5, False)
    cos, sin = ops.rope_tables_head(768, 33, 64)
    q.requires_grad_(True), k.requires_grad_(True)
    qo, ko = fa.rope(q, k, cos.cuda(), sin.cuda())
    qo.sum().backward()
    # autograd materialises the unused output's gradient as zeros before the Function sees
    # it (as it does for the reference's Function), so k's gradient is None or exactly zero
    assert q.grad is not None and (k.grad is None or not k.grad.any())


# ------------------------------------------------------------- RMSNorm ----
@pytest.mark.parametrize('dtype,wdtype', [(torch.bfloat16, torch.float32), (torch.float16, torch.float16),
                                           (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize('rows,d', [(1, 128), (37, 768), (300, 1024), (5, 64)])
def test_rmsnorm(dtype, wdtype, rows, d):
    import ulm_ops
    x = randn((rows, d), 1, dtype)
    w = (1 + 0.02 * randn((d,), 2)).to(wdtype)
    dy = randn((rows, d), 3, dtype)
    x.requires_grad_(True), w.requires_grad_(True)
    y = ulm_ops.rms_norm(x, w, 1e-6)
    y.backward(dy)
    ey = ops.rms_norm(x.detach().cpu(), w.detach().cpu())
    edx, edw = ops.rms_norm_backward(x.detach().cpu(), w.detach().cpu(), dy.cpu())
    tol = 1e-5 if dtype == torch.float32 else (2e-3 if dtype == torch.float16 else 1e-2)
    torch.testing.assert_close(y.detach().cpu().float(), ey.float(), rtol=tol, atol=tol)
    torch.testing.assert_close(x.grad.cpu().float(), edx.float(), rtol=tol, atol=tol)
    assert relerr(w.grad.float(), edw) < (1e-5 if wdtype == torch.float32 else 5e-3)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('rows,d', [(37, 768), (300, 1024), (3, 132)])
def test_rmsnorm_fp32_in_autocast_dtype_out(dtype, rows, d):
    """fp32 residual stream under autocast: the kernel rounds its fp32 result once to the
    autocast dtype, which is what the reference gets from F.rms_norm (fp32 out) followed by
    autocast's cast in front of the next Linear; the 16-bit gradient comes back to an fp32 dx."""
    import ulm_ops
    x = randn((rows, d), 11, torch.float32).requires_grad_(True)
    w = (1 + 0.02 * randn((d,), 12)).requires_grad_(True)
    dy = randn((rows, d), 13, dtype)
    with torch.autocast('cuda', dtype=dtype):
        y = ulm_ops.rms_norm(x, w, 1e-6)
    assert y.dtype == dtype and ulm_ops.rms_norm(x, w, 1e-6).dtype == torch.float32
    y.backward(dy)
    assert x.grad.dtype == torch.float32 and w.grad.dtype == torch.float32
    ey = ops.rms_norm(x.detach().cpu(), w.detach().cpu()).to(dtype)          # fp32 result, rounded once
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    torch.testing.assert_close(y.detach().cpu().float(), ey.float(), rtol=ulp, atol=1e-6)
    assert float((y.detach().cpu() != ey).float().mean()) < 0.01             # at most rare last-bit ties
    edx, edw = ops.rms_norm_backward(x.detach().cpu(), w.detach().cpu(), dy.cpu().float())
    torch.testing.assert_close(x.grad.cpu(), edx.float(), rtol=1e-4, atol=1e-5)
    assert relerr(w.grad, edw) < 1e-5
    with pytest.raises(ValueError):
        ulm_ops.rms_norm(x.detach().half(), w.detach(), 1e-6, out_dtype=torch.bfloat16)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('rows,d', [(37, 768), (301, 1024), (3, 132), (4096, 768), (1, 64)])
def test_add_rmsnorm_matches_the_unfused_sequence(dtype, rows, d):
    """x_new = x + branch; y = norm(x_new) in one kernel against the reference's sequence run eagerly on
    the same GPU (fp32 add, F.rms_norm in fp32, cast to the autocast dtype): x_new bit-equal, y within a
    16-bit ulp; the backward -- rms_norm's gradient plus the gradient arriving at x_new, written as the
    fp32 gradient of x and the 16-bit gradient of branch -- against autograd through that sequence."""
    import torch.nn.functional as F
    import ulm_ops
    x = randn((rows, d), 51, torch.float32).requires_grad_(True)
    br = randn((rows, d), 52, dtype).requires_grad_(True)
    w = (1 + 0.02 * randn((d,), 53)).requires_grad_(True)
    g_x, g_y = randn((rows, d), 54, torch.float32), randn((rows, d), 55, dtype)
    x_new, y = ulm_ops.add_rms_norm(x, br, w, 1e-6)
    assert x_new.dtype == torch.float32 and y.dtype == dtype
    torch.autograd.backward([x_new, y], [g_x, g_y])
    x1, b1, w1 = (t.detach().clone().requires_grad_(True) for t in (x, br, w))
    xn1 = x1 + b1
    y1 = F.rms_norm(xn1, (d,), w1, 1e-6).to(dtype)
    torch.autograd.backward([xn1, y1], [g_x, g_y])
    assert torch.equal(x_new, xn1)
    ulp = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    torch.testing.assert_close(y.float(), y1.float(), rtol=ulp, atol=1e-6)
    torch.testing.assert_close(x.grad, x1.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(br.grad.float(), b1.grad.float(), rtol=2 * ulp, atol=1e-6)
    assert relerr(w.grad, w1.grad) < 1e-4
    # against the CPU oracle as well
    ey = ops.rms_norm((x.detach() + br.detach().float()).cpu(), w.detach().cpu()).to(dtype)
    torch.testing.assert_close(y.cpu().float(), ey.float(), rtol=ulp, atol=1e-6)
    # x_new unused downstream (the model's final norm): no gradient arrives at it
    x2, b2, w2 = (t.detach().clone().requires_grad_(True) for t in (x, br, w))
    ulm_ops.add_rms_norm(x2, b2, w2, 1e-6)[1].backward(g_y)
    x3, b3, w3 = (t.detach().clone().requires_grad_(True) for t in (x, br, w))
    F.rms_norm(x3 + b3, (d,), w3, 1e-6).to(dtype).backward(g_y)
    torch.testing.assert_close(x2.grad, x3.grad, rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):
        ulm_ops.add_rms_norm(x.detach().half(), br.detach(), w.detach())


@pytest.mark.parametrize('dtype,d', [(torch.bfloat16, 256), (torch.bfloat16, 512), (torch.float32, 768), (torch.float32, 1024),
                                     (torch.float16, 1024), (torch.bfloat16, 1536), (torch.bfloat16, 2048), (torch.float32, 2048)])
def test_rmsnorm_every_register_tile_size(dtype, d):
    """One row width per register-tile size of the kernels (1, 2, 3, 4, 6, 8 vectors per lane) plus the
    two-pass kernel for wider rows; odd row counts exercise the several-rows-per-warp tails."""
    import ulm_ops
    for rows in (1, 7, 66):
        x = randn((rows, d), 61, dtype)
        w = (1 + 0.02 * randn((d,), 62))
        y = ulm_ops.rms_norm(x, w, 1e-6)
        tol = 1e-5 if dtype == torch.float32 else (2e-3 if dtype == torch.float16 else 1e-2)
        torch.testing.assert_close(y.cpu().float(), ops.rms_norm(x.cpu(), w.cpu()).float(), rtol=tol, atol=tol)
        if d <= 1024:
            xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
            dy = randn((rows, d), 63, dtype)
            ulm_ops.rms_norm(xg, wg, 1e-6).backward(dy)
            edx, edw = ops.rms_norm_backward(x.cpu(), w.cpu(), dy.cpu())
            torch.testing.assert_close(xg.grad.cpu().float(), edx.float(), rtol=tol, atol=tol)
            assert relerr(wg.grad, edw) < 1e-4


def test_rmsnorm_3d_and_wide_rows():
    import ulm_ops
    x = randn((2, 5, 4096), 4, torch.bfloat16)      # wider than the register tile: forward only
    w = torch.ones(4096, device='cuda')
    y = ulm_ops.rms_norm(x, w)
    torch.testing.assert_close(y.cpu().float(), ops.rms_norm(x.cpu(), w.cpu()).float(), rtol=1e-2, atol=1e-2)
    with pytest.raises(RuntimeError):
        xg = x.clone().requires_grad_(True)
        ulm_ops.rms_norm(xg, w).sum().backward()


# -------------------------------------------------------------- SwiGLU ----
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize('shape', [(3, 5, 2048), (1, 7, 13), (2, 1000, 344)])
def test_swiglu_matches_eager_path(dtype, shape):
    """Against the reference's own expression F.silu(a) * b run eagerly on the GPU in the same
    dtype (same intermediate roundings): 16-bit results may differ in the last bit only where
    exp() differs by an fp32 ulp; and against fp32 truth."""
    import torch.nn.functional as F
    import ulm_ops
    a = (2.5 * randn(shape, 31)).to(dtype).requires_grad_(True)
    b = randn(shape, 32).to(dtype).requires_grad_(True)
    dy = randn(shape, 33).to(dtype)
    y = ulm_ops.swiglu(a, b)
    y.backward(dy)
    a1, b1 = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    y1 = F.silu(a1) * b1
    y1.backward(dy)
    ulp = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7, torch.float32: 1e-5}[dtype]
    for got, ref in ((y, y1), (a.grad, a1.grad), (b.grad, b1.grad)):
        torch.testing.assert_close(got.detach().float(), ref.detach().float(), rtol=2 * ulp, atol=1e-6)
        if dtype != torch.float32:   # fp32 has no intermediate rounding to hide an ulp of exp()
            assert float((got.detach() != ref.detach()).float().mean()) < 0.02
    a2, b2 = a.detach().double().requires_grad_(True), b.detach().double().requires_grad_(True)
    y2 = F.silu(a2) * b2
    y2.backward(dy.double())
    tol = 4 * ulp
    assert relerr(y.detach(), y2.detach()) < tol and relerr(a.grad, a2.grad) < tol and relerr(b.grad, b2.grad) < tol


def test_swiglu_rejects_mismatched_inputs():
    import ulm_ops
    with pytest.raises(ValueError):
        ulm_ops.swiglu(randn((4, 8), 1, torch.float16), randn((4, 8), 2, torch.bfloat16))
    with pytest.raises(ValueError):
        ulm_ops.swiglu(randn((4, 8), 1, torch.float16), randn((4, 9), 2, torch.float16))


# ----------------------------------------------------- cross-entropy ----
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('rows,V', [(1, 8), (33, 1000), (64, 32000), (7, 4099)])
def test_ce_rows(dtype, rows, V):
    import ulm_ops
    Vs = ((V + 7) // 8) * 8                              # rows 16-byte aligned, V itself may be ragged
    buf = (3 * randn((rows, Vs), 7)).to(dtype)
    logits = buf[:, :V]
    g = torch.Generator().manual_seed(8)
    t = torch.randint(0, V, (rows,), generator=g)
    t[torch.rand(rows, generator=g) < 0.2] = 0
    tc = t.cuda()
    lse, loss = ulm_ops.ce_rows_forward(logits, tc, 0)
    elsum = ops.ce_rows(logits.cpu(), t, 0)
    torch.testing.assert_close(lse.cpu(), elsum[0], rtol=1e-5, atol=1e-5)
    assert abs(float(loss.sum()) - float(elsum[1])) <= 1e-4 * max(1.0, abs(float(elsum[1])))
    gs = torch.tensor([0.37], device='cuda')
    work = buf.clone()
    ulm_ops.ce_rows_backward_(work[:, :V], tc, lse, gs, 0, gscale=2.0)
    want = (elsum[2] * 0.74).to(dtype).float()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    torch.testing.assert_close(work[:, :V].cpu().float(), want, rtol=tol, atol=tol * 1e-2)


@pytest.mark.parametrize('form', ['kept', 'chunked'])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_chunked_ce_matches_reference_loss(dtype, form, monkeypatch):
    import ulm_ops
    if form == 'chunked':
        monkeypatch.setattr(ulm_ops, 'KEEP_LOGITS_BYTES', 0)
    rows, d, V, R = 1000, 128, 4096, 256
    h = randn((rows, d), 31)
    W = 0.02 * randn((V, d), 32)
    g = torch.Generator().manual_seed(33)
    t = torch.randint(1, V, (rows,), generator=g)
    t[torch.rand(rows, generator=g) < 0.05] = 0
    h.requires_grad_(True), W.requires_grad_(True)
    loss = ulm_ops.chunked_cross_entropy(h, W, t.cuda(), ignore_index=0, chunk_rows=R, compute_dtype=dtype)
    loss.backward()
    hc, Wc = h.detach().cpu().requires_grad_(True), W.detach().cpu().requires_grad_(True)
    ref = ops.chunked_ce(hc, Wc, t, ignore_index=0, chunk_rows=R, logits_dtype=dtype)
    ref.backward()
    assert abs(float(loss) - float(ref)) <= 1e-4      # fp32 loss tolerance
    assert relerr(h.grad, hc.grad) < 2e-2 and relerr(W.grad, Wc.grad) < 2e-2


# ------------------------------------------------------------ attention ----
def attn_case(fa, B, H, S, dtype, fused, causal=True, dropout_p=0.0, seed=100):
    q, k, v = qkv_views(B, H, S, dtype, seed, fused)
    do = randn((B, H, S, 64), seed + 9, dtype)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    assert fa.can_use(q, k, v)
    o = fa._FlashAttnV100Cuda.apply(q, k, v, dropout_p, causal, 0.125)
    seed_used = fa._last_seed
    o.backward(do)
    fa.check_status()
    return q, k, v, do, o, seed_used


# Relative (Frobenius) distance between two correctly rounded bf16 results of the same fp32 values is
# about sqrt(2) * 2^-9 / sqrt(3) = 1.6e-3 from the output rounding alone; the bf16 P / dS operands of any
# flash-style kernel add as much again.  test_bf16_reference_against_itself measures the reference's own
# bf16 SDPA run on two devices (CPU and GPU) against each other: that distance is the floor for
# "same dtype" agreement in bf16, and BF16_SAME is set just above what it shows.
BF16_SAME = 6e-3      # largest distance test_bf16_reference_against_itself shows at the shapes check_attn sees: 3.6e-3


def check_attn(name, got, same_dtype_ref, truth, dtype):
    """Tolerances, all norm-wise (Frobenius) relative errors.

    fp16: within 2e-3 of the same-dtype oracle (the reference's SDPA call) and of
    the fp32 truth, and max-abs within 2e-3 of the largest magnitude.
    bf16: 2e-3 against fp32 truth is below the rounding floor of the format for
    the gradients (see BF16_SAME above and test_bf16_reference_against_itself), so
    the bar is: no worse than twice the reference's own bf16 SDPA error against
    the same truth, at most 5e-3 against truth, within BF16_SAME of the reference's
    bf16 SDPA result, and max-abs within two bf16 ulps (2^-7) of the largest
    magnitude.  A result that is exactly zero in exact arithmetic (S=1 gradients)
    is checked absolutely."""
    tn = float(truth.double().norm())
    if tn < 1e-6:
        assert float(got.double().abs().max()) < 1e-3, name
        return
    e_same = relerr(got, same_dtype_ref)
    e_truth, e_ref = relerr(got, truth), relerr(same_dtype_ref, truth)
    mx = float(truth.abs().max())
    amax = float((got.float().cpu() - truth.float().cpu()).abs().max())
    if dtype == torch.float16:
        assert e_same <= 2e-3 and e_truth <= 2e-3, f'{name}: {e_same:.2e} vs oracle, {e_truth:.2e} vs truth'
        assert amax <= 2e-3 * mx, f'{name}: max abs {amax:.3e} of {mx:.3e}'
    else:
        assert e_truth <= 5e-3, f'{name}: {e_truth:.2e} vs truth'
        assert e_same <= BF16_SAME, f'{name}: {e_same:.2e} vs the reference bf16 SDPA'
        assert amax <= 2 ** -7 * mx, f'{name}: max abs {amax:.3e} of {mx:.3e}'
    assert e_truth <= 2 * e_ref + 2e-4, f'{name}: err vs truth {e_truth:.2e}, oracle {e_ref:.2e}'


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('B,H,S,fused', [(1, 1, 1, False), (1, 2, 63, False), (2, 2, 64, True), (1, 3, 65, False),
                                         (1, 2, 127, True), (2, 1, 128, False), (1, 2, 129, False),
                                         (1, 2, 200, True), (1, 1, 257, False), (1, 2, 1000, True)])
def test_attention_causal_parity(fa, dtype, B, H, S, fused):
    q, k, v, do, o, _ = attn_case(fa, B, H, S, dtype, fused)
    qc, kc, vc, doc = (t.detach().cpu() for t in (q, k, v, do))
    # same-dtype oracle: the reference's SDPA call; truth: explicit fp32 softmax
    q1, k1, v1 = (t.clone().requires_grad_(True) for t in (qc, kc, vc))
    o1 = ops.sdpa_causal(q1, k1, v1, scale=0.125)
    o1.backward(doc)
    q2, k2, v2 = (t.float().requires_grad_(True) for t in (qc, kc, vc))
    o2, lse2 = ops.attention_explicit(q2, k2, v2, scale=0.125)
    o2.backward(doc.float())
    check_attn('o', o.detach(), o1.detach(), o2.detach(), dtype)
    check_attn('dq', q.grad, q1.grad, q2.grad, dtype)
    check_attn('dk', k.grad, k1.grad, k2.grad, dtype)
    check_attn('dv', v.grad, v1.grad, v2.grad, dtype)


@pytest.mark.parametrize('B,H,S', [(1, 2, 200), (1, 2, 1000), (1, 12, 4096)])
def test_bf16_reference_against_itself(fa, B, H, S):
    """The reference's attention call (F.scaled_dot_product_attention, is_causal) in bf16 on the CPU
    against the same call in bf16 on this GPU, same inputs: two correct bf16 implementations of one
    formula.  Their distance is what "within 2e-3 of the bf16 oracle" would have to beat; it does not
    (the gradients sit at 2-4e-3), which is why the bf16 rows of check_attn use BF16_SAME and the
    error-vs-fp32-truth comparison instead.  Our kernels must be at least as close to the CPU oracle as
    the GPU library is.  Measured on B200 (norm-wise relative distances): library GPU vs CPU 0.8-2.1e-3
    for o and dq, 3.5e-3 for dk and dv at S <= 1000 and 6.4e-3 at S = 4096 (the CPU kernel itself is 6.4e-3
    from fp32 truth there); every GPU result, the library's and ours, is 1.9-2.5e-3 from fp32 truth."""
    import torch.nn.functional as F
    dtype = torch.bfloat16
    q, k, v = qkv_views(B, H, S, dtype, 100, False)
    do = randn((B, H, S, 64), 109, dtype)

    def run(dev, fn):
        qq, kk, vv = (t.detach().to(dev).clone().requires_grad_(True) for t in (q, k, v))
        o = fn(qq, kk, vv)
        o.backward(do.to(dev))
        return [t.detach().cpu() for t in (o, qq.grad, kk.grad, vv.grad)]
    sdpa = lambda a, b, c: F.scaled_dot_product_attention(a, b, c, is_causal=True, scale=0.125)   # noqa: E731
    cpu = run('cpu', sdpa)
    gpu = run('cuda', sdpa)
    ours = run('cuda', lambda a, b, c: fa.flash_attn_v100(a, b, c, softmax_scale=0.125))
    fa.check_status()
    q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o2 = F.scaled_dot_product_attention(q2, k2, v2, is_causal=True, scale=0.125)
    o2.backward(do.float())
    truth = [t.detach().cpu() for t in (o2, q2.grad, k2.grad, v2.grad)]
    report = {}
    for name, c, g, u, t in zip(('o', 'dq', 'dk', 'dv'), cpu, gpu, ours, truth):
        lib_same, our_same = relerr(g, c), relerr(u, c)
        report[name] = dict(lib_gpu_vs_cpu=lib_same, ours_vs_cpu=our_same, cpu_vs_truth=relerr(c, t),
                            lib_gpu_vs_truth=relerr(g, t), ours_vs_truth=relerr(u, t))
    print(f'bf16 reference against itself, B={B} H={H} S={S}:',
          {n: {k_: f'{v_:.2e}' for k_, v_ in r.items()} for n, r in report.items()})
    for name, r in report.items():
        # as accurate as the library kernel on the same GPU, and no farther from the CPU reference than the
        # larger of (library GPU vs CPU) and (CPU vs truth) -- the two are independent roundings of one value
        assert r['ours_vs_truth'] <= 1.05 * r['lib_gpu_vs_truth'] + 1e-4, (name, r)
        assert r['ours_vs_cpu'] <= 1.1 * max(r['lib_gpu_vs_cpu'], r['cpu_vs_truth']) + 2e-4, (name, r)


# ------------------------------------------------- RoPE fused into attention ----
@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('B,H,S,fused_qkv,p', [(1, 1, 1, False, 0.0), (2, 3, 63, True, 0.0), (1, 2, 129, False, 0.0),
                                               (2, 2, 200, True, 0.1), (1, 3, 1000, True, 0.0), (3, 12, 384, True, 0.0),
                                               (1, 12, 4096, True, 0.0)])
def test_fused_rope_attention_is_bit_identical_to_the_two_calls(fa, monkeypatch, dtype, B, H, S, fused_qkv, p):
    """rope() followed by flash_attn_v100() -- the reference's two calls -- against rope_flash_attn with
    the RoPE work in each of its three placements ('none': stand-alone kernels inside one op; 'fwd': Q
    rotated inside the forward kernel; 'all': also dQ/dK un-rotated in the backward epilogues) and against
    qkv_rope_flash_attn on the fused projection tensor: every output bit equal -- o, and the gradients
    of the UNROTATED q, k and of v."""
    monkeypatch.setattr(fa, '_next_seed', lambda: 0x1234ABCD)      # every run draws the same dropout mask
    q, k, v = qkv_views(B, H, S, dtype, 700, fused_qkv)
    do = randn((B, H, S, 64), 709, dtype)
    cos, sin = ops.rope_tables(768, 4096)
    c2, s2 = cos.cuda()[:S, :64], sin.cuda()[:S, :64]
    outs = []
    modes = ['two calls', 'none', 'fwd', 'all'] + (['qkv'] if fused_qkv else [])
    for mode in modes:
        if fused_qkv:      # views of one buffer, like the model's projection: one gradient tensor for all three
            buf = torch.cat([t.detach().transpose(1, 2).reshape(B, S, H * 64) for t in (q, k, v)], dim=-1).requires_grad_(True)
            qq, kk, vv = (t.view(B, S, H, 64).transpose(1, 2) for t in buf.chunk(3, dim=-1))
            leaves = [buf]
        else:
            qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            leaves = [qq, kk, vv]
        if mode == 'two calls':
            qr, kr = fa.rope(qq, kk, c2, s2)
            o = fa._FlashAttnV100Cuda.apply(qr, kr, vv, p, True, 0.125)
        elif mode == 'qkv':
            o = fa.qkv_rope_flash_attn(buf, H, c2, s2, dropout_p=p, softmax_scale=0.125)
            assert o.shape == (B, S, H * 64)
            o = o.view(B, S, H, 64).transpose(1, 2)
        else:
            o = fa.rope_flash_attn(qq, kk, vv, c2, s2, dropout_p=p, softmax_scale=0.125, fuse=mode)
        o.backward(do)
        outs.append((o.detach(), [t.grad for t in leaves]))
    fa.check_status()
    for mode, (o, grads) in zip(modes[1:], outs[1:]):
        assert torch.equal(outs[0][0], o), mode
        for a, b in zip(outs[0][1], grads):
            assert torch.equal(a, b), mode
    assert float(outs[0][1][0].abs().max()) > 0 or S == 1


def test_qkv_attention_without_rope_and_argument_checks(fa):
    B, H, S = 2, 3, 100
    buf = randn((B, S, 3 * H * 64), 730, torch.float16).requires_grad_(True)
    do = randn((B, S, H * 64), 731, torch.float16)
    o = fa.qkv_rope_flash_attn(buf, H)
    o.backward(do)
    b2 = buf.detach().clone().requires_grad_(True)
    q, k, v = (t.view(B, S, H, 64).transpose(1, 2) for t in b2.chunk(3, dim=-1))
    o2 = fa.flash_attn_v100(q, k, v).transpose(1, 2).reshape(B, S, H * 64)
    o2.backward(do)
    fa.check_status()
    assert torch.equal(o, o2) and torch.equal(buf.grad, b2.grad)
    with pytest.raises(ValueError):
        fa.qkv_rope_flash_attn(buf.detach()[:, :, :-64], H)                       # not 3*H*64 wide
    with pytest.raises(ValueError):
        fa.qkv_rope_flash_attn(buf.detach(), H, torch.zeros(S, 64, device='cuda'), None)
    with pytest.raises(ValueError):
        fa.rope_flash_attn(q, k, v, torch.zeros(S, 64, device='cuda'), torch.zeros(S, 64, device='cuda'), fuse='sometimes')


def test_rope_k_only_and_fused_forward_without_q_rot(fa):
    """C ABI details of the fused path: ulm_rope with q = qo = NULL rotates K alone; a forward with
    tables but no q_rot output (inference) gives the same o."""
    B, H, S = 2, 3, 150
    q, k, v = qkv_views(B, H, S, torch.float16, 720, True)
    cos, sin = ops.rope_tables(768, S)
    c2, s2 = cos.cuda()[:, :64], sin.cuda()[:, :64]
    qr, kr = fa.rope(q, k, c2, s2)
    _, k_only = fa._rope_launch(None, k, c2, s2, backward=False)
    assert torch.equal(k_only, kr)
    o_ref, lse_ref, _ = fa.attn_forward(qr, kr, v, 0.0, True, 0.125, 0)
    o1, lse1, q_rot = fa.attn_forward(q, kr, v, 0.0, True, 0.125, 0, cos=c2, sin=s2)
    o2, lse2, none = fa.attn_forward(q, kr, v, 0.0, True, 0.125, 0, cos=c2, sin=s2, want_q_rot=False)
    fa.check_status()
    assert none is None and torch.equal(q_rot, qr)
    assert torch.equal(o1, o_ref) and torch.equal(o2, o_ref) and torch.equal(lse1, lse_ref) and torch.equal(lse2, lse_ref)


# ------------------------------------------------ failure detection, host side ----
def test_expired_wait_is_reported_and_the_context_survives(fa):
    """The attention kernels bound every barrier wait; on expiry they set a status bit and return.
    The library's self-test runs that same wait routine with a 2 ms limit on a barrier nothing
    arrives at: the kernel must come back by itself, the status word must carry the timeout bit,
    check_status() must raise, and the GPU must go on working afterwards."""
    fa.check_status()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    fa.selftest_wait_timeout(limit_ns=2_000_000)
    t1.record()
    torch.cuda.synchronize()
    assert 1.0 <= t0.elapsed_time(t1) < 200.0            # it waited about the limit, then returned
    with pytest.raises(RuntimeError, match='barrier timeout'):
        fa.check_status()
    fa.check_status()                                     # the word was cleared by the raise
    q, k, v = qkv_views(1, 2, 100, torch.float16, 5, False)
    o = fa.flash_attn_v100(q, k, v)
    eo, _ = ops.attention_explicit(q.cpu().float(), k.cpu().float(), v.cpu().float(), 0.125)
    fa.check_status()
    assert relerr(o, eo) < 2e-3


def test_dp_step_raises_when_a_kernel_timed_out(fa):
    """The data-parallel step reads the status word at its step boundary: a step during which a wait
    expired must raise instead of stepping the optimiser on partly written gradients."""
    import ulm_dp
    import ulm_train
    model, preset = ulm_train.build('tiny64', torch.device('cuda'), seed=0)
    opt = ulm_train.make_optimizer(model)
    steps = ulm_train.step_batches('tiny64', 16, 1, target_tokens=2048, max_micro_batch=16, n_docs=16, data_seed=3)
    runner = ulm_dp.DataParallelStep(model, opt, samples_per_step=16, autocast_dtype=torch.bfloat16,
                                     ce_chunk_rows=512, device=torch.device('cuda'))
    runner.step(steps[0])
    fa.selftest_wait_timeout(limit_ns=1_000_000)
    with pytest.raises(RuntimeError, match='barrier timeout'):
        runner.step(steps[0])
    runner.step(steps[0])                                 # and recovers on the next one


def test_tensor_maps_are_cached(fa):
    q, k, v = qkv_views(1, 2, 300, torch.float16, 15, False)
    fa.flash_attn_v100(q, k, v)
    h0, m0 = fa.tensor_map_cache_stats()
    for _ in range(3):
        fa.flash_attn_v100(q, k, v)
    h1, m1 = fa.tensor_map_cache_stats()
    fa.check_status()
    assert m1 == m0 and h1 == h0 + 9                      # q, k, v maps of three forwards, all from the cache


def test_attention_lse_and_noncausal(fa):
    import ctypes as C
    import _native as N
    B, H, S = 1, 2, 200
    for causal in (True, False):
        q, k, v = qkv_views(B, H, S, torch.float16, 77, False)
        o = fa._FlashAttnV100Cuda.apply(q, k, v, 0.0, causal, 0.125)
        fa.check_status()
        eo, elsum = ops.attention_explicit(q.cpu().float(), k.cpu().float(), v.cpu().float(), 0.125, causal=causal)
        assert relerr(o, eo) < 2e-3
    # LSE straight from the C ABI
    q, k, v = qkv_views(B, H, S, torch.bfloat16, 78, False)
    o = torch.empty_like(q)
    lse = torch.empty((B, H, S), dtype=torch.float32, device='cuda')
    a = N.AttnFwdArgs()
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    for n, t in (('q', q), ('k', k), ('v', v), ('o', o)):
        setattr(a, n + '_sb', t.stride(0)), setattr(a, n + '_sh', t.stride(1)), setattr(a, n + '_ss', t.stride(2))
    a.B, a.H, a.S, a.dtype, a.causal, a.softmax_scale = B, H, S, N.ULM_BF16, 1, 0.125
    a.stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert N.lib().ulm_attn_fwd(C.byref(a)) == 0
    _, elsum = ops.attention_explicit(q.cpu().float(), k.cpu().float(), v.cpu().float(), 0.125)
    torch.testing.assert_close(lse.cpu(), elsum, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize('dtype', DTYPES)
def test_attention_dropout_matches_hash_oracle(fa, dtype):
    B, H, S, p = 1, 2, 200, 0.1
    q, k, v, do, o, seed = attn_case(fa, B, H, S, dtype, False, dropout_p=p, seed=300)
    qc, kc, vc = (t.detach().cpu().float() for t in (q, k, v))
    eo, elsum = ops.attention_explicit(qc, kc, vc, 0.125, dropout_p=p, seed=seed)
    assert relerr(o.detach(), eo) < 4e-3
    dq, dk, dv, _ = ops.attention_bwd_explicit(qc, kc, vc, eo, elsum, do.cpu().float(), 0.125, dropout_p=p, seed=seed)
    assert relerr(q.grad, dq) < 6e-3 and relerr(k.grad, dk) < 6e-3 and relerr(v.grad, dv) < 6e-3


@pytest.mark.parametrize('dtype', DTYPES)
def test_rope_then_attention_config2_shape_small_batch(fa, dtype):
    """Config 2's pipeline (RoPE with the 768-wide table, then causal attention,
    grads w.r.t. the pre-RoPE q,k) at S=4096 on one batch element, against the
    oracle run on the GPU in the same dtype and in fp32."""
    B, H, S = 1, 12, 4096
    q, k, v = qkv_views(B, H, S, dtype, 500, True)
    do = randn((B, H, S, 64), 509, dtype)
    cos, sin = ops.rope_tables(768, S)
    cos2d, sin2d = cos.cuda()[:, :64], sin.cuda()[:, :64]
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    qr, kr = fa.rope(q, k, cos2d, sin2d)
    o = fa.flash_attn_v100(qr, kr, v, causal=True)
    o.backward(do)
    fa.check_status()
    ref = ops.rope_attention_grads(q.detach(), k.detach(), v.detach(), do, cos2d, sin2d, dtype, use_sdpa=True)
    tru = ops.rope_attention_grads(q.detach().float(), k.detach().float(), v.detach().float(), do.float(),
                                   cos2d, sin2d, torch.float32, use_sdpa=True)
    check_attn('o', o.detach(), ref['o'], tru['o'], dtype)
    check_attn('dq', q.grad, ref['dq'], tru['dq'], dtype)
    check_attn('dk', k.grad, ref['dk'], tru['dk'], dtype)
    check_attn('dv', v.grad, ref['dv'], tru['dv'], dtype)


def test_attention_full_config2_properties(fa):
    """B=8,H=12,S=4096: size-independent properties instead of a dense oracle --
    rows of softmax sum to one (V = ones gives O = 1), the first query only sees
    itself, and batch elements are independent (batch 0 equals a B=1 run)."""
    B, H, S = 8, 12, 4096
    q, k, v = qkv_views(B, H, S, torch.bfloat16, 900, False)
    o = fa.flash_attn_v100(q, k, v)
    o1 = fa.flash_attn_v100(q[:1], k[:1], v[:1])
    fa.check_status()
    assert torch.equal(o[:1], o1)
    assert torch.equal(o[:, :, 0], v[:, :, 0])
    ones = torch.ones_like(v)
    torch.testing.assert_close(fa.flash_attn_v100(q, k, ones).float(), ones.float(), rtol=0, atol=8e-3)


def test_grad_unscale_sumsq_is_deterministic():
    """Data-parallel ranks derive the clip factor from this number and never re-synchronise their
    weights, so identical gradients must give identical bits: per-CTA partials added in a fixed order."""
    import ulm_ops
    g0 = randn((9_000_001,), 43)
    outs = []
    for _ in range(4):
        g = g0.clone()
        out = torch.zeros(2, device='cuda')
        ulm_ops.grad_unscale_sumsq_(g, None, out)
        outs.append(out.clone())
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    want = float(g0.double().pow(2).sum())
    assert abs(float(outs[0][0]) - want) <= 1e-5 * want


def test_grad_unscale_sumsq():
    import ulm_ops
    g = randn((100003,), 41)
    inv = torch.tensor([1 / 1024.0], device='cuda')
    out = torch.zeros(2, device='cuda')
    want = (g * inv).double().pow(2).sum()
    ulm_ops.grad_unscale_sumsq_(g, inv, out)
    assert abs(float(out[0]) - float(want)) <= 1e-4 * float(want) and float(out[1]) == 0.0
    torch.testing.assert_close(g, randn((100003,), 41) / 1024.0)
    g[77] = float('inf')
    out.zero_()
    ulm_ops.grad_unscale_sumsq_(g, None, out)
    assert float(out[1]) == 1.0


# ---------------------------------------------------------- edge cases ----
def test_attention_edge_inputs(fa):
    # empty batch: nothing to launch, shapes preserved
    q = torch.empty((0, 2, 16, 64), dtype=torch.float16, device='cuda')
    assert tuple(fa.flash_attn_v100(q, q, q).shape) == (0, 2, 16, 64)
    # inputs the kernel cannot take as they are (odd strides) are made contiguous by the wrapper
    base = randn((1, 2, 50, 72), 61, torch.float16)
    qv, kv, vv = base[..., :64], base[..., 4:68], base[..., 8:72]
    assert not fa.can_use(qv, kv, vv)
    o = fa.flash_attn_v100(qv, kv, vv)
    eo, _ = ops.attention_explicit(qv.cpu().float(), kv.cpu().float(), vv.cpu().float(), 0.125)
    assert relerr(o, eo) < 2e-3
    # wrong dtype / head_dim / device are refused the way the reference refuses them
    with pytest.raises(ValueError):
        fa.flash_attn_v100(qv.float(), kv.float(), vv.float())
    with pytest.raises(ValueError):
        fa.flash_attn_v100(base[..., :32], base[..., :32], base[..., :32])
    # tables that are not [S, 64] fp32 make the fused RoPE ineligible
    cos, sin = ops.rope_tables_head(768, 50, 64)
    assert not fa.rope_can_use(qv.contiguous(), kv.contiguous(), cos.cuda().half(), sin.cuda().half())
    assert not fa.rope_can_use(qv.contiguous(), kv.contiguous(), cos.cuda()[:49], sin.cuda()[:49])
    fa.check_status()


def test_attention_backward_is_deterministic(fa):
    q, k, v = qkv_views(2, 3, 777, torch.bfloat16, 71, True)
    do = randn((2, 3, 777, 64), 72, torch.bfloat16)
    outs = []
    for _ in range(2):
        qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        o = fa.flash_attn_v100(qq, kk, vv)
        o.backward(do)
        outs.append((o.detach(), qq.grad, kk.grad, vv.grad))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_long_sequence_8192(fa):
    q, k, v = qkv_views(1, 2, 8192, torch.float16, 81, False)
    do = randn((1, 2, 8192, 64), 82, torch.float16)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    o = fa.flash_attn_v100(q, k, v)
    o.backward(do)
    fa.check_status()
    q1, k1, v1 = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    o1 = ops.sdpa_causal(q1, k1, v1, scale=0.125)
    o1.backward(do)
    assert relerr(o.detach(), o1.detach()) < 2e-3
    assert relerr(q.grad, q1.grad) < 2e-3 and relerr(k.grad, k1.grad) < 2e-3 and relerr(v.grad, v1.grad) < 2e-3


@pytest.mark.parametrize('B,H,S', [(40, 12, 1), (40, 12, 64), (40, 12, 128), (48, 12, 200), (25, 24, 300)])
def test_many_short_work_items_per_cta(fa, B, H, S):
    """More than three work items per persistent backward CTA, each of one to a few
    tiles (the shapes a token-budget batch of short documents produces): no barrier
    may run out, and the gradients match the reference's SDPA on the same GPU."""
    dtype = torch.float16
    q, k, v = (randn((B, S, H, 64), 600 + i, dtype).transpose(1, 2).requires_grad_(True) for i in range(3))
    do = randn((B, H, S, 64), 609, dtype)
    o = fa.flash_attn_v100(q, k, v)
    o.backward(do)
    fa.check_status()
    q1, k1, v1 = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    o1 = ops.sdpa_causal(q1, k1, v1, scale=0.125)
    o1.backward(do)
    assert relerr(o.detach(), o1.detach()) < 2e-3
    if S > 1:   # S = 1: every gradient but dv is exactly zero
        assert relerr(q.grad, q1.grad) < 2e-3 and relerr(k.grad, k1.grad) < 2e-3
    assert relerr(v.grad, v1.grad) < 2e-3


def test_dropout_with_several_work_items_per_cta(fa):
    """Dropout variants of the persistent backward kernels with more than one work item
    per CTA (20 x 12 heads x two 128-row tiles = 480 items on 148 CTAs), against the
    hash-mask oracle on a slice of the batch."""
    B, H, S, p = 20, 12, 200, 0.1
    q, k, v, do, o, seed = attn_case(fa, B, H, S, torch.float16, False, dropout_p=p, seed=310)
    # batch element 0 (the mask depends on the batch*head index, which the oracle counts from 0): its
    # heads' two row tiles are first items of some CTAs and second items of others
    qc, kc, vc = (t.detach()[:1].cpu().float() for t in (q, k, v))
    eo, elsum = ops.attention_explicit(qc, kc, vc, 0.125, dropout_p=p, seed=seed)
    assert relerr(o.detach()[:1], eo) < 4e-3
    dq, dk, dv, _ = ops.attention_bwd_explicit(qc, kc, vc, eo, elsum, do[:1].cpu().float(), 0.125, dropout_p=p, seed=seed)
    assert relerr(q.grad[:1], dq) < 6e-3 and relerr(k.grad[:1], dk) < 6e-3 and relerr(v.grad[:1], dv) < 6e-3


def test_backward_is_deterministic_with_several_work_items_per_cta(fa):
    q, k, v = qkv_views(4, 12, 1024, torch.bfloat16, 91, True)        # 384 work items on 148 persistent CTAs
    do = randn((4, 12, 1024, 64), 92, torch.bfloat16)
    outs = []
    for _ in range(2):
        qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        o = fa.flash_attn_v100(qq, kk, vv)
        o.backward(do)
        outs.append((o.detach(), qq.grad, kk.grad, vv.grad))
    fa.check_status()
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.gpu
def test_weight_gradients_accumulated_in_place_match_autograd():
    """`ulm_ops.wgrad_in_place`: the GEMMs add dW into the existing fp32 .grad (fp32 accumulation and output);
    the result must agree with autograd's route (16-bit product, cast, add) to the 16-bit rounding of that
    route, sit closer to an fp32 computation, and leave nothing for autograd to accumulate."""
    import ulm_model
    import ulm_ops
    torch.manual_seed(5)
    cfg = ulm_model.ModelConfig(vocab_size=512, d_model=256, n_heads=4, n_layers=2, d_ff=512, max_seq_len=256, dropout=0.0)
    dev = torch.device('cuda')
    m = ulm_model.DecoderOnlyTransformer(cfg).to(dev)
    ids = [torch.randint(1, 512, (3, 200), device=dev), torch.randint(1, 512, (2, 131), device=dev)]

    def grads(in_place, dtype):
        for p in m.parameters():
            p.grad = torch.zeros_like(p)
        with torch.autocast('cuda', dtype=dtype), ulm_ops.wgrad_in_place(in_place):
            for x in ids:
                m.compute_loss(x, ignore_index=0, chunk_rows=128).backward()
        return {n: p.grad.clone() for n, p in m.named_parameters()}

    for dtype in (torch.bfloat16, torch.float16):
        a, b = grads(False, dtype), grads(True, dtype)
        for n in a:
            assert b[n].dtype == torch.float32
            rel = float((a[n] - b[n]).norm() / a[n].norm())
            assert rel <= (8e-3 if dtype == torch.bfloat16 else 2e-3), (n, rel)
        # linear layers outside the context behave like nn.Linear
        x = torch.randn(7, 256, device=dev, requires_grad=True)
        w = m.layers[0].self_attn.wo.weight
        w.grad = None
        with torch.autocast('cuda', dtype=dtype):
            y1 = ulm_ops.linear(x, w)
            y2 = torch.nn.functional.linear(x, w)
        assert torch.equal(y1, y2)
        g1 = torch.autograd.grad(y1.float().sum(), (x, w))
        g2 = torch.autograd.grad(y2.float().sum(), (x, w))
        assert torch.equal(g1[0], g2[0]) and torch.allclose(g1[1], g2[1], rtol=1e-2, atol=1e-3)


@pytest.mark.gpu
def test_cached_weight_casts_do_not_outlive_a_step():
    """The 16-bit weight copies `linear` keeps inside `weight_cast_scope` must be remade after the optimiser
    changed the weights (a fused optimiser does not bump the parameters' version counters): training with
    the data-parallel step follows the same losses as the same steps without any caching."""
    import ulm_dp
    import ulm_model
    import ulm_ops
    cfg = ulm_model.ModelConfig(vocab_size=512, d_model=256, n_heads=4, n_layers=2, d_ff=512, max_seq_len=256, dropout=0.0)
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(3)
    steps = [[torch.randint(1, 512, (4, 160), generator=g), torch.randint(1, 512, (4, 96), generator=g)]] * 6   # one batch, six times

    def run(cached):
        torch.manual_seed(11)
        m = ulm_model.DecoderOnlyTransformer(cfg).to(dev)
        opt = torch.optim.AdamW(m.parameters(), lr=3e-3, fused=True)
        runner = ulm_dp.DataParallelStep(m, opt, samples_per_step=8, autocast_dtype=torch.bfloat16, device=dev, ce_chunk_rows=128)
        losses = []
        for st in steps:
            if cached:
                losses.append(float(runner.step(st)[0]))
            else:
                orig = ulm_ops.weight_cast_scope
                ulm_ops.weight_cast_scope = contextlib.nullcontext
                try:
                    losses.append(float(runner.step(st)[0]))
                finally:
                    ulm_ops.weight_cast_scope = orig
        return losses

    import contextlib
    a, b = run(True), run(False)
    assert a[0] > a[-1] + 0.05, a                        # it trains
    assert max(abs(x - y) for x, y in zip(a, b)) <= 2e-3, (a, b)


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_lm_head_lse_matches_gemm_then_logsumexp(dtype):
    """`ulm_lmhead_lse` (train.py:2075-2079's fc_out + cross_entropy forward as one tensor-core kernel): the
    stored logits are the 16-bit-rounded product, lse and the per-row loss agree with an fp32 log-sum-exp over
    those logits to 1e-5; ragged row counts, a ragged last column tile, ignored targets, statistics-only mode."""
    import ulm_ops
    import flash_attn_v100_cuda as fa
    dev = torch.device('cuda')
    torch.manual_seed(2)
    for rows, V, d, keep in [(1, 64, 64, True), (127, 320, 128, True), (129, 256, 64, True), (300, 6464, 768, True),
                             (515, 1000, 192, False), (2048, 32000, 768, True), (64, 32000, 768, False),
                             (40000, 32000, 64, True)]:       # more than 2^40 bytes of rows x V x 64-column blocks: the unused outer stride
        h = torch.randn(rows, d, device=dev).to(dtype)
        w = (torch.randn(V, d, device=dev) * (2.0 * d ** -0.5)).to(dtype)
        t = torch.randint(0, V, (rows,), device=dev)
        t[::5] = 0
        lse, loss, z = ulm_ops.lm_head_lse(h, w, t, 0, keep_logits=keep)
        zr = (h.float() @ w.float().t()).to(dtype)             # fp32 product, one rounding: the kernel's contract
        lser = torch.logsumexp(zr.float(), dim=1)
        tol = 2e-2 if dtype == torch.bfloat16 else 3e-3                     # one-ulp differences of the rounded logits
        assert float((lse - lser).abs().max()) <= tol
        if keep:
            # the library GEMM in the same dtype (what the unfused path stores): same bits up to rare one-ulp flips
            zl = h @ w.t()
            assert float((z != zl).float().mean()) <= 1e-3
            assert float((z.float() - zr.float()).abs().max()) <= float(zr.float().abs().max()) * 2 ** (-7 if dtype == torch.bfloat16 else -10)
            lse_own = torch.logsumexp(z.float(), dim=1)           # against its own stored logits: exact arithmetic contract
            assert float((lse - lse_own).abs().max()) <= 1e-5
            want = torch.where(t == 0, torch.zeros_like(lse_own), lse_own - z.float().gather(1, t[:, None])[:, 0])
            assert float((loss - want).abs().max()) <= 1e-5
            assert float(loss[t == 0].abs().max()) == 0.0
        else:
            assert loss is None and z is None
    fa.check_status()
    # and through the loss: fused and unfused kept forms give the same value and gradients
    h = torch.randn(700, 256, device=dev, requires_grad=True)
    w = (torch.randn(1024, 256, device=dev) * 0.1).requires_grad_(True)
    t = torch.randint(0, 1024, (700,), device=dev)
    outs = []
    for fused in (True, False):
        ulm_ops.FUSED_LM_HEAD = fused
        try:
            loss = ulm_ops.chunked_cross_entropy(h, w, t, ignore_index=0, chunk_rows=256, compute_dtype=dtype)
            gh, gw = torch.autograd.grad(loss, (h, w))
        finally:
            ulm_ops.FUSED_LM_HEAD = True
        outs.append((float(loss), gh, gw))
    assert abs(outs[0][0] - outs[1][0]) <= 1e-5
    assert torch.allclose(outs[0][1], outs[1][1], rtol=0, atol=2e-6 + 1e-3 * float(outs[1][1].abs().max()))
    assert torch.allclose(outs[0][2], outs[1][2], rtol=0, atol=2e-6 + 1e-3 * float(outs[1][2].abs().max()))


@pytest.mark.gpu
def test_first_cuda_call_of_a_thread_may_be_ours():
    """A thread whose first CUDA work is one of this library's entry points (an autograd worker running our
    backward as its first node, its outputs served from cached allocator blocks) has no context bound yet;
    the entry point must bind the tensors' device itself before it encodes tensor maps."""
    import threading
    import flash_attn_v100_cuda as fa
    dev = torch.device('cuda')
    torch.manual_seed(0)
    q, k, v, do = (torch.randn(1, 2, 256, 64, device=dev).to(torch.bfloat16) for _ in range(4))
    o, lse, _ = fa.attn_forward(q, k, v, 0.0, True, 0.125, 0)
    want = fa.attn_backward(q, k, v, o, lse, do, 0.0, True, 0.125, 0)      # also leaves cached blocks of the right sizes
    torch.cuda.synchronize()
    want = [t.clone() for t in want]
    got, err = [], []

    def work():
        try:
            got.extend(fa.attn_backward(q, k, v, o, lse, do, 0.0, True, 0.125, 0))
            torch.cuda.synchronize()
        except Exception as e:  # noqa: BLE001 - reported by the assertion below
            err.append(e)
    th = threading.Thread(target=work)
    th.start()
    th.join()
    assert not err, err
    for a, b in zip(got, want):
        assert torch.equal(a, b)


@pytest.mark.gpu
def test_lm_head_lse_random_shapes():
    """Tile-edge sweep of `ulm_lmhead_lse`: 40 random (rows, V, d) with V and d multiples of 64 -- row blocks and
    column tiles that do not divide, one-tile and many-group cases -- against the library GEMM + fp32 log-sum-exp."""
    import random
    import ulm_ops
    import flash_attn_v100_cuda as fa
    rng = random.Random(1234)
    dev = torch.device('cuda')
    torch.manual_seed(7)
    for i in range(40):
        rows = rng.choice([1, 2, 63, 127, 128, 129, 255, 257, 300, 511, 640, 1000])
        V = 64 * rng.choice([1, 2, 3, 4, 5, 8, 9, 25, 26, 51, 100, 101, 104, 125, 129])
        d = 64 * rng.choice([1, 2, 3, 12])
        dtype = torch.bfloat16 if i % 2 else torch.float16
        h = torch.randn(rows, d, device=dev).to(dtype)
        w = (torch.randn(V, d, device=dev) * (2.0 * d ** -0.5)).to(dtype)
        t = torch.randint(0, V, (rows,), device=dev)
        lse, loss, z = ulm_ops.lm_head_lse(h, w, t, 0, keep_logits=True)
        zl = h @ w.t()
        assert float((z != zl).float().mean()) <= 2e-3, (rows, V, d, dtype)
        lse_own = torch.logsumexp(z.float(), dim=1)
        assert float((lse - lse_own).abs().max()) <= 1e-5, (rows, V, d, dtype)
        want = torch.where(t == 0, torch.zeros_like(lse_own), lse_own - z.float().gather(1, t[:, None])[:, 0])
        assert float((loss - want).abs().max()) <= 1e-5, (rows, V, d, dtype)
        lse2, _, _ = ulm_ops.lm_head_lse(h, w, None, 0, keep_logits=False)
        assert torch.equal(lse2, lse), (rows, V, d, dtype)
    fa.check_status()
