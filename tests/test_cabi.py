"""The C-ABI library loads, exports every function ``include/sparta_b200.h`` declares, and rejects
bad arguments on the host (no kernel is launched by any of these calls, so no GPU is needed)."""
import ctypes
import os
import re

from sparta_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'sparta_b200.h')


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(sparta_[a-z0-9_]+)\s*\(', text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared_functions()
    assert len(names) >= 15
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(handle, name), f'{name} is declared in the header but not exported'
        assert name in _lib.SIGNATURES, f'{name} has no ctypes signature'
    assert set(_lib.SIGNATURES) <= set(names)


def test_version_and_status_strings():
    L = _lib.lib()
    assert L.sparta_version() == 100
    assert L.sparta_status_string(0) == b'ok'
    for code in range(-7, 0):
        assert len(L.sparta_status_string(code)) > 5


def test_struct_layout_matches_header():
    assert ctypes.sizeof(_lib.BsmmArgs) == 7 * 8 + 14 * 4 + 4 * 8
    assert ctypes.sizeof(_lib.TileEntry) == 9 * 4


def test_host_side_argument_checks():
    L = _lib.lib()
    # null pointers
    assert L.sparta_bcs_build(None, 1, 64, 64, 32, 32, 1, 0, None, None, None, None, 4, None, None, None,
                              None, 0, None) == -1
    fake = 0x1000  # never dereferenced: every call below fails validation first
    # block size not a power of two in [4, 256]
    assert L.sparta_bcs_build(fake, 1, 60, 60, 12, 12, 1, 0, fake, fake, None, None, 25, fake, None, None,
                              fake, 1 << 20, None) == -2
    # mask not divisible by the block
    assert L.sparta_bcs_build(fake, 1, 100, 64, 32, 32, 1, 0, fake, fake, None, None, 25, fake, None, None,
                              fake, 1 << 20, None) == -2
    # workspace too small
    need = L.sparta_bcs_build_workspace_bytes(1, 64, 64, 32, 32)
    assert need > 0
    assert L.sparta_bcs_build(fake, 1, 64, 64, 32, 32, 1, 0, fake, fake, None, None, 4, fake, None, None,
                              fake, need - 1, None) == -4
    args = _lib.BsmmArgs(A=fake, B=fake, C=fake, ptr=fake, idx=fake, nnz=fake, batch=1, M=100, K=64, N=64,
                         BM=32, BK=32, BN=32, dtype=0, impl=0, n_index_sets=1)
    assert L.sparta_bsmm_dsd(ctypes.byref(args), None) == -2  # M % BM
    args.M = 128
    args.dtype = 9
    assert L.sparta_bsmm_dsd(ctypes.byref(args), None) == -1
    args.dtype = 0
    args.impl = _lib.IMPL_TCGEN05  # fp32 has no tensor-core kernel
    assert L.sparta_bsmm_dsd(ctypes.byref(args), None) == -3
    assert L.sparta_softmax_fwd(fake, fake, fake, fake, fake, None, 1.0, 1, 64, 60, 32, 32, 0, 0, 0, None) == -2
    assert L.sparta_bcs_gather(fake, fake, fake, fake, 1, 64, 64, 32, 32, 3, 1, 0, 4, 4, None) == -1


def test_tile_table():
    for op in range(3):
        f32 = _lib.tile_table(op, _lib.F32)
        assert len(f32) == 64 and all(e.impl == _lib.IMPL_SIMT for e in f32)
    assert len(_lib.tile_table(_lib.OP_SOFTMAX, _lib.F32)) == 20
    assert _lib.lib().sparta_tile_table(9, 0, None, 0) == -1


def test_missing_library_raises(monkeypatch):
    import pytest
    monkeypatch.setattr(_lib, '_LIB', None)
    monkeypatch.setattr(_lib, 'LIB_PATH', '/nonexistent/libsparta_b200.so')
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        _lib.lib()


def test_cpu_tensors_are_rejected():
    import pytest
    import torch
    from sparta_b200.tesa import get_bcs_function
    with pytest.raises(RuntimeError, match='no CPU fallback'):
        get_bcs_function(32, 32, True, False).build_indexes(torch.ones((64, 64), dtype=torch.uint8))
