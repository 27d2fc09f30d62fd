"""The allocation-free index build, ``sparta_bcs_build_static``.

Some users of the library cannot hand it a workspace: their device memory pool is frozen once the
service is up, or they run on a thread where the host framework forbids cudaMalloc.  For them the
scratch is a fixed 1 MiB array inside the library.  This file checks, through the C ABI, that the
entry point produces exactly what ``sparta_bcs_build`` produces with a caller workspace -- on two
consecutive calls, because the shared array still holds the first call's contents when the second one
starts -- and that requests beyond the fixed size are refused.  It is named to be collected last, so a
run that stops at the first failure has already been through every other test.
"""
import pytest
import torch

from sparta_b200 import _lib

STATIC_BYTES = 1 << 20


def _outputs(n, R, C, both, device):
    i32 = dict(dtype=torch.int32, device=device)
    return dict(
        row_ptr=torch.full((n, R + 1), -1, **i32), bcsr=torch.full((n, R * C), -1, **i32),
        col_ptr=torch.full((n, C + 1), -1, **i32),
        bcsc=torch.full((n, R * C), -1, dtype=torch.int64 if both else torch.int32, device=device),
        nnz=torch.full((n,), -1, **i32), uniform=torch.full((n,), -1, **i32))


def _build(mask, BH, BW, static):
    L = _lib.lib()
    n, H, W = mask.shape
    R, C = H // BH, W // BW
    o = _outputs(n, R, C, True, mask.device)
    common = (mask.data_ptr(), n, H, W, BH, BW, 1, 1, o['row_ptr'].data_ptr(), o['bcsr'].data_ptr(),
              o['col_ptr'].data_ptr(), o['bcsc'].data_ptr(), R * C, o['nnz'].data_ptr(), o['uniform'].data_ptr())
    stream = _lib.stream_ptr(mask.device)
    if static:
        _lib.check(L.sparta_bcs_build_static(*common, stream), 'sparta_bcs_build_static')
    else:
        nbytes = L.sparta_bcs_build_workspace_bytes(n, H, W, BH, BW)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=mask.device)
        _lib.check(L.sparta_bcs_build(*common, None, ws.data_ptr(), nbytes, stream), 'sparta_bcs_build')
    torch.cuda.synchronize()
    return o


@pytest.mark.gpu
def test_static_scratch_build_matches_workspace_build_twice():
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(123)
    # first call: a dense-ish set of masks; second call: a smaller, sparser problem, so anything the
    # first call left in the shared array (occupancy bytes, ranks, tickets) would show up as a difference
    cases = [
        ((4, 512, 768), (32, 32), 0.6),
        ((2, 256, 384), (8, 64), 0.97),
    ]
    for shape, (BH, BW), sparsity in cases:
        mask = (torch.rand(shape, generator=g) > sparsity).to(torch.uint8).to(dev)
        got = _build(mask, BH, BW, static=True)
        ref = _build(mask, BH, BW, static=False)
        assert torch.equal(got['nnz'], ref['nnz'])
        assert torch.equal(got['uniform'], ref['uniform'])
        assert torch.equal(got['row_ptr'], ref['row_ptr'])
        assert torch.equal(got['col_ptr'], ref['col_ptr'])
        for b in range(shape[0]):
            cnt = int(ref['nnz'][b])
            assert torch.equal(got['bcsr'][b, :cnt], ref['bcsr'][b, :cnt])
            assert torch.equal(got['bcsc'][b, :cnt], ref['bcsc'][b, :cnt])


def test_static_scratch_refuses_oversized_requests():
    """Host-side check, no launch: 64 masks of 4096 x 4096 at 4 x 4 blocks need far more than 1 MiB."""
    L = _lib.lib()
    fake = 0x1000  # never dereferenced: the size check comes first
    assert L.sparta_bcs_build_workspace_bytes(64, 4096, 4096, 4, 4) > STATIC_BYTES
    rc = L.sparta_bcs_build_static(fake, 64, 4096, 4096, 4, 4, 1, 0, fake, fake, None, None, 1 << 20, fake,
                                   None, None)
    assert rc == -4
    assert b'workspace' in L.sparta_status_string(rc)
    # and the largest supported shapes are accepted by the size check (rejected later only for the fake pointers)
    assert L.sparta_bcs_build_workspace_bytes(32, 2048, 2048, 32, 32) <= STATIC_BYTES
    assert L.sparta_bcs_build_workspace_bytes(1, 8192, 8192, 32, 32) <= STATIC_BYTES
