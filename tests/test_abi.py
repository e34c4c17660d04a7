"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every
symbol the header declares, and rejects bad arguments before touching CUDA."""
import ctypes as C
import os
import re

import pytest

import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_reports_version():
    assert N.available(), N.build_error()
    assert N.lib().ulm_abi_version() == N.ABI_VERSION == 4


def test_every_declared_symbol_is_exported():
    text = open(os.path.join(ROOT, 'include', 'ulm_b200.h')).read()
    declared = set(re.findall(r'\b(ulm_[a-z0-9_]+)\s*\(', text))
    assert declared, 'no declarations found'
    lib = C.CDLL(os.path.join(ROOT, 'universal-lm-trainer_b200', 'libulm_b200.so'))
    for name in sorted(declared):
        assert hasattr(lib, name), f'{name} declared in ulm_b200.h but not exported'
    assert declared == set(N.EXPORTS), declared ^ set(N.EXPORTS)


def test_struct_sizes_match_the_header():
    # field counts x widths, as laid out by the C compiler for the header's structs
    assert C.sizeof(N.RopeArgs) == 6 * 8 + 14 * 8 + 5 * 4 + 4 + 8
    assert C.sizeof(N.AttnFwdArgs) == 5 * 8 + 12 * 8 + 5 * 4 + 3 * 4 + 8 + 8 + 4 * 8 + 4 * 8
    assert C.sizeof(N.AttnBwdArgs) == 10 * 8 + 24 * 8 + 6 * 4 + 3 * 4 + 4 + 8 + 8 + 4 * 8
    assert C.sizeof(N.RmsFwdArgs) == 4 * 8 + 2 * 8 + 8 + 4 * 4 + 8 + 2 * 4 + 4 * 8
    assert C.sizeof(N.RmsBwdArgs) == 7 * 8 + 3 * 8 + 8 + 4 * 4 + 8 + 2 * 4 + 4 * 8
    assert C.sizeof(N.CeFwdArgs) == 4 * 8 + 8 + 8 + 2 * 4 + 8 + 8
    assert C.sizeof(N.LmHeadLseArgs) == 8 * 8 + 3 * 8 + 8 + 4 * 4 + 8 + 2 * 8


def test_bad_arguments_are_refused_with_a_message():
    lib = N.lib()
    a = N.RopeArgs()
    a.B, a.H, a.S, a.dtype = 1, 1, 1, 7
    assert lib.ulm_rope(C.byref(a)) == -1
    assert b'dtype' in lib.ulm_last_error()
    with pytest.raises(ValueError):
        N.check(lib.ulm_rope(C.byref(a)), 'rope')
    f = N.AttnFwdArgs()
    f.B, f.H, f.S, f.dtype = 1, 1, 16, N.ULM_F16
    assert lib.ulm_attn_fwd(C.byref(f)) == -1          # null tensors
    assert b'null' in lib.ulm_last_error()
    f.S = 0
    assert lib.ulm_attn_fwd(C.byref(f)) == 0           # empty problem: nothing to do
    r = N.RmsFwdArgs()
    r.rows, r.d, r.x_dtype, r.w_dtype = 4, 12, N.ULM_BF16, N.ULM_F32
    assert lib.ulm_rmsnorm_fwd(C.byref(r)) == -1       # d not a multiple of 8
    assert lib.ulm_rmsnorm_bwd_partial_rows(10) >= 1
    assert lib.ulm_rmsnorm_bwd_partial_rows(10 ** 9) == 296
    assert lib.ulm_grad_sumsq_partial_count() == 592
    assert lib.ulm_grad_unscale_sumsq(None, 8, None, None, None, None) == -1      # null pointers
    assert lib.ulm_selftest_wait_timeout(0, None, None) == -1                      # limit out of range
    assert b'limit_ns' in lib.ulm_last_error()
    f.S, f.cos_tab = 16, 64                                                       # tables must come as a pair
    f.q = f.k = f.v = f.o = f.lse = 256
    f.softmax_scale = 0.125
    assert lib.ulm_attn_fwd(C.byref(f)) == -1
    assert b'together' in lib.ulm_last_error()
    h, m = C.c_uint64(7), C.c_uint64(7)
    lib.ulm_tensor_map_cache_stats(C.byref(h), C.byref(m))
    assert h.value == 0 and m.value == 0                                          # nothing encoded without a GPU


def test_wrapper_module_surface():
    import flash_attn_v100
    import flash_attn_v100_cuda as m
    for name in ('is_available', 'build_error', 'can_use', 'rope_can_use', 'rope', 'flash_attn_v100',
                 '_FlashAttnV100Cuda', '_RopeV100Cuda', 'rope_flash_attn', 'check_status'):
        assert hasattr(m, name)
    assert flash_attn_v100.flash_attn_v100 is m.flash_attn_v100
    assert m.is_available() and m.build_error() is None
    import torch
    q = torch.zeros(1, 2, 8, 64, dtype=torch.float16)
    assert not m.can_use(q, q, q)                      # CPU tensors are never eligible
    with pytest.raises(ValueError):
        m.flash_attn_v100(q, q, q)
