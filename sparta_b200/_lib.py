"""ctypes binding of ``libsparta_b200.so`` (declared in ``include/sparta_b200.h``).

There is no CPU or eager fallback: when the shared library is missing, ``lib()`` raises, and every
operator of this package goes through ``lib()``.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from typing import Optional

import torch

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'lib', 'libsparta_b200.so')

OK = 0
F32, F16, BF16 = 0, 1, 2
IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05 = 0, 1, 2
OP_SDD, OP_DSD, OP_DDS, OP_SOFTMAX, OP_ATTENTION = range(5)

DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


class BsmmArgs(ctypes.Structure):
    """Mirror of ``sparta_bsmm_args``."""
    _fields_ = [
        ('A', c_void_p), ('B', c_void_p), ('bias', c_void_p), ('C', c_void_p),
        ('ptr', c_void_p), ('idx', c_void_p), ('nnz', c_void_p),
        ('batch', c_int32), ('M', c_int32), ('K', c_int32), ('N', c_int32),
        ('BM', c_int32), ('BK', c_int32), ('BN', c_int32),
        ('trans_a', c_int32), ('trans_b', c_int32), ('compressed', c_int32), ('idx_is_64', c_int32),
        ('dtype', c_int32), ('impl', c_int32), ('n_index_sets', c_int32),
        ('ptr_stride', c_int64), ('idx_stride', c_int64), ('val_stride_blocks', c_int64),
        ('grid_blocks_hint', c_int64),
    ]


class TileEntry(ctypes.Structure):
    """Mirror of ``sparta_tile_entry``."""
    _fields_ = [
        ('op', c_int32), ('dtype', c_int32), ('impl', c_int32),
        ('block_m', c_int32), ('block_k', c_int32), ('block_n', c_int32),
        ('trans_a', c_int32), ('trans_b', c_int32), ('compressed', c_int32),
    ]


# name -> (restype, argtypes); the list is also what the symbol-export test walks
SIGNATURES = {
    'sparta_version': (c_int, []),
    'sparta_status_string': (c_char_p, [c_int]),
    'sparta_device_supported': (c_int, [c_int]),
    'sparta_bcs_build_workspace_bytes': (c_size_t, [c_int] * 5),
    'sparta_bcs_build': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_size_t, c_void_p]),
    'sparta_bcs_build_static': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                        c_void_p]),
    'sparta_bcs_gather': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_int64, c_int64, c_void_p]),
    'sparta_bcs_scatter': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_int, c_int, c_int64, c_int64, c_void_p]),
    'sparta_bcs_sum': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int64, c_void_p]),
    'sparta_bsmm_sdd': (c_int, [POINTER(BsmmArgs), c_void_p]),
    'sparta_bsmm_dsd': (c_int, [POINTER(BsmmArgs), c_void_p]),
    'sparta_bsmm_dds': (c_int, [POINTER(BsmmArgs), c_void_p]),
    'sparta_softmax_fwd': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_void_p]),
    'sparta_softmax_bwd': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int64,
                                   c_void_p]),
    'sparta_attn_fwd_workspace_bytes': (c_size_t, [c_int] * 5),
    'sparta_attn_fwd': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                c_void_p, c_void_p, c_size_t, c_void_p]),
    'sparta_attn_fwd_gather': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p, POINTER(c_void_p), c_int, c_void_p]),
    'sparta_last_status': (c_int, [POINTER(c_int32)]),
    'sparta_tile_table': (c_int, [c_int, c_int, POINTER(TileEntry), c_int]),
}

_LIB: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """Load the CUDA library once; raise (never fall back) when it has not been built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f'{LIB_PATH} is missing: build it with `python -m sparta_b200.csrc.build` '
                '(there is no CPU fallback for the sparse kernels)')
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = handle
    return _LIB


class SpartaError(RuntimeError):
    def __init__(self, status: int, where: str):
        text = lib().sparta_status_string(status).decode()
        super().__init__(f'{where}: status {status} ({text})')
        self.status = status


def check(status: int, where: str):
    if status != OK:
        raise SpartaError(status, where)


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def require_cuda(*tensors: torch.Tensor):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError('sparta_b200 operators run on CUDA tensors only (no CPU fallback)')


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f'unsupported dtype {t.dtype}: expected float32, float16 or bfloat16')


def tile_table(op: int, dtype: int = F32):
    """Prebuilt tile shapes for an operation, preferred entries first."""
    n = lib().sparta_tile_table(op, dtype, None, 0)
    buf = (TileEntry * max(n, 1))()
    lib().sparta_tile_table(op, dtype, buf, n)
    return [buf[i] for i in range(n)]


def last_status():
    """Status words of the tcgen05 kernels (synchronises the device); all zero when clean."""
    buf = (c_int32 * 4)()
    check(lib().sparta_last_status(buf), 'sparta_last_status')
    return list(buf)
