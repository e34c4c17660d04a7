"""Recipe that compiles the one piece of the reference's native code that runs on a
host: the dropout keep-mask hash of csrc/flash_attn_v100/fa_common.cuh:21-38.

Test infrastructure only.  ``build_ref(reference_dir)`` compiles
oracle/ref_dropout_hash.cpp -- which merely #includes the reference's header from where
it lies -- with g++ into oracle/_ref/libref_dropout_hash.so (git-ignored).  The
reference's attention and RoPE kernels themselves are sm_70 wmma code that is wrong on
any other architecture (fa_common.cuh:40-48) and are not built.

``load_ref()`` returns the ctypes library or None when it has not been built; tests use it,
where present, to check the numpy restatement in oracle/ops.py bit for bit, and
tests/golden/make_golden.py uses it to write the committed keep-mask fixture.
"""
import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_OUT_DIR = os.path.join(_HERE, '_ref')
_LIB = os.path.join(_OUT_DIR, 'libref_dropout_hash.so')


def build_ref(reference_dir, cuda_include='/usr/local/cuda/include'):
    hdr_dir = os.path.join(reference_dir, 'csrc', 'flash_attn_v100')
    if not os.path.isfile(os.path.join(hdr_dir, 'fa_common.cuh')):
        raise FileNotFoundError(f'{hdr_dir}/fa_common.cuh not found')
    os.makedirs(_OUT_DIR, exist_ok=True)
    cmd = ['g++', '-O2', '-shared', '-fPIC', '-Wno-attributes', '-I', cuda_include, '-I', hdr_dir,
           os.path.join(_HERE, 'ref_dropout_hash.cpp'), '-o', _LIB + '.tmp']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError('g++ failed:\n' + r.stderr[-2000:])
    os.replace(_LIB + '.tmp', _LIB)
    return _LIB


def load_ref():
    if not os.path.exists(_LIB):
        return None
    lib = C.CDLL(_LIB)
    lib.ref_hash_u32.restype, lib.ref_hash_u32.argtypes = C.c_uint32, [C.c_uint32]
    lib.ref_dropout_keep.restype = C.c_int
    lib.ref_dropout_keep.argtypes = [C.c_uint32, C.c_int, C.c_int, C.c_uint32, C.c_float]
    lib.ref_dropout_keep_block.restype = None
    lib.ref_dropout_keep_block.argtypes = [C.c_uint32, C.c_uint32, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_void_p]
    return lib


def ref_keep_block(lib, seed, bh, p, row0, nrows, col0, ncols):
    import numpy as np
    out = np.empty((nrows, ncols), dtype=np.uint8)
    lib.ref_dropout_keep_block(seed & 0xFFFFFFFF, bh, p, row0, nrows, col0, ncols, out.ctypes.data)
    return out.astype(bool)
