"""Loader for libulm_b200.so -- the C-ABI CUDA library behind every op here.

Mirrors what flash_attn_v100_cuda.py:36-66 of the reference does with
torch.utils.cpp_extension.load: build lazily on first use, cache the result
next to the sources, never raise at import time, and report a failed build
through ``build_error()``.  The library is plain ``nvcc -shared`` output with
``extern "C"`` entry points (include/ulm_b200.h); it does not link against
torch.  There is no fallback: every op raises if the library is unavailable.
"""
from __future__ import annotations

import concurrent.futures
import ctypes as C
import os
import subprocess
import tempfile
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, 'csrc')
_LIB_PATH = os.path.join(_HERE, 'libulm_b200.so')
_SOURCES = ['attn_bwd.cu', 'attn_fwd.cu', 'lmhead.cu', 'lib.cu', 'tc_host.cu', 'rope.cu', 'rmsnorm.cu', 'ce.cu', 'swiglu.cu',
            'grad_post.cu', 'selftest.cu']          # slowest first: they are compiled in parallel
_HEADERS = ['common.cuh', 'tc.cuh', 'rope_math.cuh', os.path.join('..', '..', 'include', 'ulm_b200.h')]

_lock = threading.Lock()
_lib = None
_error = None

ULM_F16, ULM_BF16, ULM_F32 = 0, 1, 2
ULM_Y_SAME, ULM_Y_F16, ULM_Y_BF16 = 0, 1, 2
ABI_VERSION = 4
i64, i32, u32, f32, vp = C.c_int64, C.c_int32, C.c_uint32, C.c_float, C.c_void_p


class RopeArgs(C.Structure):
    _fields_ = ([(n, vp) for n in ('q', 'k', 'qo', 'ko', 'cos_tab', 'sin_tab')] +
                [(n, i64) for n in ('q_sb', 'q_sh', 'q_ss', 'k_sb', 'k_sh', 'k_ss',
                                    'qo_sb', 'qo_sh', 'qo_ss', 'ko_sb', 'ko_sh', 'ko_ss',
                                    'cos_stride', 'sin_stride')] +
                [(n, i32) for n in ('B', 'H', 'S', 'dtype', 'backward')] + [('stream', vp)])


class AttnFwdArgs(C.Structure):
    _fields_ = ([(n, vp) for n in ('q', 'k', 'v', 'o', 'lse')] +
                [(n, i64) for n in ('q_sb', 'q_sh', 'q_ss', 'k_sb', 'k_sh', 'k_ss',
                                    'v_sb', 'v_sh', 'v_ss', 'o_sb', 'o_sh', 'o_ss')] +
                [(n, i32) for n in ('B', 'H', 'S', 'dtype', 'causal')] +
                [('softmax_scale', f32), ('dropout_p', f32), ('seed', u32),
                 ('status_dev', vp), ('stream', vp),
                 ('cos_tab', vp), ('sin_tab', vp), ('cos_stride', i64), ('sin_stride', i64),
                 ('q_rot', vp), ('qr_sb', i64), ('qr_sh', i64), ('qr_ss', i64)])


class AttnBwdArgs(C.Structure):
    _fields_ = ([(n, vp) for n in ('q', 'k', 'v', 'o', 'd_o', 'lse', 'delta', 'dq', 'dk', 'dv')] +
                [(f'{t}_{s}', i64) for t in ('q', 'k', 'v', 'o', 'do', 'dq', 'dk', 'dv')
                 for s in ('sb', 'sh', 'ss')] +
                [(n, i32) for n in ('B', 'H', 'S', 'dtype', 'causal', 'mode')] +
                [('softmax_scale', f32), ('dropout_p', f32), ('seed', u32),
                 ('status_dev', vp), ('stream', vp),
                 ('cos_tab', vp), ('sin_tab', vp), ('cos_stride', i64), ('sin_stride', i64)])


class RmsFwdArgs(C.Structure):
    _fields_ = [('x', vp), ('w', vp), ('y', vp), ('rstd', vp), ('x_stride', i64), ('y_stride', i64),
                ('rows', i64), ('d', i32), ('x_dtype', i32), ('w_dtype', i32), ('eps', f32),
                ('stream', vp), ('y_kind', i32), ('reserved', i32),
                ('branch', vp), ('x_out', vp), ('branch_stride', i64), ('xout_stride', i64)]


class RmsBwdArgs(C.Structure):
    _fields_ = [('x', vp), ('w', vp), ('dy', vp), ('rstd', vp), ('dx', vp), ('dw', vp),
                ('partial', vp), ('x_stride', i64), ('dy_stride', i64), ('dx_stride', i64),
                ('rows', i64), ('d', i32), ('x_dtype', i32), ('w_dtype', i32), ('eps', f32),
                ('stream', vp), ('dy_kind', i32), ('reserved', i32),
                ('g_add', vp), ('d_branch', vp), ('gadd_stride', i64), ('dbranch_stride', i64)]


class SwigluArgs(C.Structure):
    _fields_ = [('a', vp), ('b', vp), ('y', vp), ('dy', vp), ('da', vp), ('db', vp), ('n', i64),
                ('dtype', i32), ('reserved', i32), ('stream', vp)]


class CeFwdArgs(C.Structure):
    _fields_ = [('logits', vp), ('target', vp), ('lse', vp), ('loss', vp), ('row_stride', i64),
                ('rows', i64), ('V', i32), ('dtype', i32), ('ignore_index', i64), ('stream', vp)]


class CeBwdArgs(C.Structure):
    _fields_ = [('logits', vp), ('target', vp), ('lse', vp), ('gscale_dev', vp), ('gscale', f32),
                ('row_stride', i64), ('rows', i64), ('V', i32), ('dtype', i32),
                ('ignore_index', i64), ('stream', vp)]


class LmHeadLseArgs(C.Structure):
    _fields_ = [('h', vp), ('w', vp), ('logits', vp), ('target', vp), ('lse', vp), ('loss', vp),
                ('part_m', vp), ('part_s', vp), ('h_stride', i64), ('w_stride', i64), ('z_stride', i64),
                ('rows', i64), ('V', i32), ('d', i32), ('dtype', i32), ('reserved', i32),
                ('ignore_index', i64), ('status_dev', vp), ('stream', vp)]


# every symbol include/ulm_b200.h declares: name -> (restype, argtypes)
EXPORTS = {
    'ulm_abi_version': (C.c_int, []),
    'ulm_last_error': (C.c_char_p, []),
    'ulm_device_ok': (C.c_int, [C.c_int]),
    'ulm_launch_count': (C.c_uint64, []),
    'ulm_rope': (C.c_int, [C.POINTER(RopeArgs)]),
    'ulm_attn_fwd': (C.c_int, [C.POINTER(AttnFwdArgs)]),
    'ulm_attn_bwd': (C.c_int, [C.POINTER(AttnBwdArgs)]),
    'ulm_rmsnorm_fwd': (C.c_int, [C.POINTER(RmsFwdArgs)]),
    'ulm_rmsnorm_bwd': (C.c_int, [C.POINTER(RmsBwdArgs)]),
    'ulm_rmsnorm_bwd_partial_rows': (C.c_int64, [C.c_int64]),
    'ulm_rmsnorm_bwd_static': (C.c_int, [C.POINTER(RmsBwdArgs)]),
    'ulm_ce_fwd': (C.c_int, [C.POINTER(CeFwdArgs)]),
    'ulm_lmhead_lse': (C.c_int, [C.POINTER(LmHeadLseArgs)]),
    'ulm_lmhead_lse_parts': (C.c_int64, [C.c_int32]),
    'ulm_ce_bwd': (C.c_int, [C.POINTER(CeBwdArgs)]),
    'ulm_swiglu_fwd': (C.c_int, [C.POINTER(SwigluArgs)]),
    'ulm_swiglu_bwd': (C.c_int, [C.POINTER(SwigluArgs)]),
    'ulm_grad_unscale_sumsq': (C.c_int, [vp, i64, vp, vp, vp, vp]),
    'ulm_grad_sumsq_partial_count': (C.c_int64, []),
    'ulm_tensor_map_cache_stats': (None, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    'ulm_selftest_wait_timeout': (C.c_int, [C.c_uint64, vp, vp]),
}


def _nvcc():
    return os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')


_ARCH = ['-gencode', 'arch=compute_100a,code=sm_100a']
_CFLAGS = ['-O3', '-lineinfo', '-std=c++17', '-Xcompiler', '-fPIC', '-I', os.path.join(_HERE, '..', 'include')]


def nvcc_commands(obj_dir, out_path=_LIB_PATH, extra=()):
    """One compile command per source (they run in parallel) and the link command."""
    objs = [os.path.join(obj_dir, s[:-3] + '.o') for s in _SOURCES]
    compile_cmds = [[_nvcc(), *extra, *_ARCH, *_CFLAGS, '-c', os.path.join(_CSRC, s), '-o', o]
                    for s, o in zip(_SOURCES, objs)]
    link = [_nvcc(), *_ARCH, '-shared', '-Xcompiler', '-fPIC', '-cudart', 'static', *objs, '-o', out_path]
    return compile_cmds, link


def _stale():
    if not os.path.exists(_LIB_PATH):
        return True
    t = os.path.getmtime(_LIB_PATH)
    deps = [os.path.join(_CSRC, s) for s in _SOURCES + _HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile csrc/*.cu for sm_100a into libulm_b200.so beside this file."""
    if not force and not _stale():
        return _LIB_PATH
    # Several ranks may find the library stale at once: each links into a file of its own
    # and the rename is atomic, so a reader never sees a half-written library.
    tmp_path = f'{_LIB_PATH}.{os.getpid()}.tmp'
    with tempfile.TemporaryDirectory(prefix='ulm_b200_build_') as obj_dir:
        compile_cmds, link = nvcc_commands(obj_dir, tmp_path)

        def run(cmd):
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode:
                print(' '.join(cmd))
                print(r.stdout, r.stderr)
            if r.returncode:
                raise RuntimeError(f'nvcc failed ({r.returncode}):\n{r.stderr[-4000:]}')
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(compile_cmds), os.cpu_count() or 1)) as ex:
            list(ex.map(run, compile_cmds))
        run(link)
    os.replace(tmp_path, _LIB_PATH)
    return _LIB_PATH


def _load():
    global _lib, _error
    with _lock:
        if _lib is not None or _error is not None:
            return
        try:
            # Sources are newer than the library only on a developer's machine; the
            # shipped .so is used as is when no compiler is around.
            if _stale() and os.path.exists(_nvcc()):
                build()
            lib = C.CDLL(_LIB_PATH)
            for name, (res, args) in EXPORTS.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            if lib.ulm_abi_version() != ABI_VERSION:
                raise RuntimeError(f'libulm_b200 ABI {lib.ulm_abi_version()} != {ABI_VERSION}')
            _lib = lib
        except Exception as e:  # noqa: BLE001 - reported through build_error()
            _error = e


def lib():
    """The loaded library, or raise: there is no other implementation to fall back to."""
    _load()
    if _lib is None:
        raise RuntimeError(f'libulm_b200.so is unavailable: {_error}')
    return _lib


def available() -> bool:
    _load()
    return _lib is not None


def build_error():
    _load()
    return _error


def check(rc: int, what: str):
    if rc == 0:
        return
    msg = lib().ulm_last_error().decode('utf-8', 'replace')
    if rc == -1:
        raise ValueError(f'{what}: {msg}')
    raise RuntimeError(f'{what}: {msg} (code {rc})')


try:
    from torch._C import _cuda_getCurrentRawStream as _raw_stream      # one C call; the public API builds a Stream object
except ImportError:  # pragma: no cover - older torch
    _raw_stream = None


def current_stream(device_index):
    """cudaStream_t of torch's current stream on ``device_index`` as a ctypes void pointer."""
    if _raw_stream is not None:
        return C.c_void_p(_raw_stream(device_index))
    import torch
    return C.c_void_p(torch.cuda.current_stream(device_index).cuda_stream)


def launch_count() -> int:
    return int(lib().ulm_launch_count())
