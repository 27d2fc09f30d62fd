"""Second parity pin: this library against the reference's OWN CUDA kernels on the same GPU.

``oracle/ref_kernels.py`` renders the reference's jinja2 templates from a checkout and compiles them for
sm_100a (cubins under ``oracle/_ref``); they are launched here with the reference's grid / block formulas
on the shapes of its unit tests (test/unit/test_sparse_matmul.py:16-29,133-138, test_sparse_softmax.py:17-25,
test_tesa.py:20-27) and compared with this library through the C-ABI.  Index arrays are compared as sets per
block row / column (the reference's order inside a row depends on ``atomicAdd``,
sparta/tesa/templates/block_compressed.cu.j2:112-116); fp32 results at rtol = atol = 1e-4.

Skipped (not failed) only when the cubins were never built, i.e. no checkout of the reference was
available to ``__graft_entry__.build()``.
"""
import numpy as np
import pytest
import torch

from oracle import oracle, ref_kernels
from sparta_b200.specializer.kernels import (SparTASparseMatMulKernel, OpenAISparseMatMulKernel,
                                             SparTASparseSoftmaxForwardKernel, SparTASparseSoftmaxBackwardKernel)
from sparta_b200.tesa import get_bcs_function

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_kernels.available(), reason='oracle/_ref was not built')]
TOL = dict(rtol=1e-4, atol=1e-4)
SPARSE_PORT = {'sdd': 'A', 'dsd': 'B', 'dds': 'C'}


@pytest.fixture(scope='module')
def ref():
    return ref_kernels.ReferenceKernels()


def _rows(ptr: torch.Tensor, idx: torch.Tensor):
    ptr, idx = ptr.cpu().tolist(), idx.cpu().tolist()
    return [sorted(int(v) & 0xffffffff for v in idx[ptr[i]:ptr[i + 1]]) for i in range(len(ptr) - 1)]


@pytest.mark.parametrize('BH,BW', [(8, 8), (16, 16), (32, 32), (32, 64), (64, 32), (64, 64)])
@pytest.mark.parametrize('form', ['BCSR', 'BCSC', 'BCSRC'])
def test_index_build_matches_reference_kernels(ref, BH, BW, form):
    g = torch.Generator().manual_seed(2023)
    mask = oracle.block_mask((1024, 768), (4, 4), 0.99, generator=g).cuda()
    bcsr, bcsc = form != 'BCSC', form != 'BCSR'
    theirs = ref.build_indexes(mask, BH, BW, bcsr, bcsc)
    ours = get_bcs_function(BH, BW, bcsr, bcsc).build_indexes(mask)
    assert ours.block_nnz == theirs['nnz']
    if bcsr:
        assert torch.equal(ours.row_ptr.cpu(), theirs['row_ptr'].cpu())
        assert _rows(ours.row_ptr, ours.BCSR_idx) == _rows(theirs['row_ptr'], theirs['BCSR_idx'])
    if bcsc:
        assert torch.equal(ours.col_ptr.cpu(), theirs['col_ptr'].cpu())
        assert _rows(ours.col_ptr, ours.BCSC_idx) == _rows(theirs['col_ptr'], theirs['BCSC_idx'])
    # dense -> compressed -> dense through either implementation gives back the masked tensor
    dense = torch.rand((2, 1024, 768), generator=g).cuda() * mask
    torch.testing.assert_close(ref.inverse(ref.convert(dense, theirs), theirs), dense, rtol=0, atol=0)
    torch.testing.assert_close(ours.inverse(ours.convert(dense)), dense, rtol=0, atol=0)
    if form == 'BCSRC':
        # the upper half of a 64-bit BCSC entry is the block's position in BCSR order: check it against the
        # reference's own BCSR array (positions differ between the two builds, the blocks they name must not)
        for build_idx, bcsr_idx in ((theirs['BCSC_idx'], theirs['BCSR_idx']), (ours.BCSC_idx, ours.BCSR_idx)):
            c = build_idx.cpu().numpy().astype(np.int64)
            r = bcsr_idx.cpu().numpy().astype(np.int64)
            named = r[c >> 32]
            assert np.array_equal(named >> 16, c & 0xffff) and np.array_equal(named & 0xffff, (c >> 16) & 0xffff)


def _block_of(mode, tile, trans_A, trans_B):
    BM, BK, BN = tile
    if mode == 'sdd':
        return (BK, BM) if trans_A else (BM, BK)
    if mode == 'dsd':
        return (BN, BK) if trans_B else (BK, BN)
    return (BM, BN)


@pytest.mark.parametrize('impl', ['sparta', 'openai'])
@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('biased', [False, True])
@pytest.mark.parametrize('trans_A', [False, True])
@pytest.mark.parametrize('trans_B', [False, True])
@pytest.mark.parametrize('compressed', [False, True])
def test_matmul_matches_reference_kernels(ref, impl, mode, biased, trans_A, trans_B, compressed):
    batch, M, K, N = 4, 128, 256, 192
    g = torch.Generator().manual_seed(2022)
    shapes = {'A': (K, M) if trans_A else (M, K), 'B': (N, K) if trans_B else (K, N), 'C': (M, N)}
    A = torch.rand((batch,) + shapes['A'], generator=g).cuda()
    B = torch.rand((batch,) + shapes['B'], generator=g).cuda()
    bias = torch.rand((batch, N), generator=g).cuda() if biased else None
    port = SPARSE_PORT[mode]
    mask = oracle.block_mask(shapes[port], (8, 8), 0.9, generator=g).cuda()
    if port == 'A':
        A = A * mask
    elif port == 'B':
        B = B * mask
    tile = (32, 32, 32) if impl == 'sparta' else (32, 64, 32)
    BH, BW = _block_of(mode, tile, trans_A, trans_B)

    # the reference's kernel, its own index build and its own compression
    by_row = ref_kernels._bcs_flags(mode, trans_A, trans_B)
    rix = ref.build_indexes(mask, BH, BW, *by_row)
    rA, rB = A, B
    if compressed and port == 'A':
        rA = ref.convert(A, rix)
    if compressed and port == 'B':
        rB = ref.convert(B, rix)
    theirs = ref.matmul(impl, mode, rA, rB, bias, rix, M, K, N, trans_A, trans_B, compressed)
    if compressed and port == 'C':
        theirs = ref.inverse(theirs, rix)

    # this library through the kernel object (C-ABI underneath)
    cls = SparTASparseMatMulKernel if impl == 'sparta' else OpenAISparseMatMulKernel
    kernel = cls(mode=mode, biased=biased, transpose_A=trans_A, transpose_B=trans_B, compressed=compressed)
    kernel.ports[port].set_mask(mask)
    kernel.set_shape(batch, M, K, N)
    kernel.compile({'_impl': impl, **({f'BLOCK_SIZE_{d}_VALUE': t for d, t in zip('MKN', tile)}
                                      if impl == 'sparta' else {})})
    ix = kernel.ports[port].indexes
    oA, oB = A, B
    if compressed and port == 'A':
        oA = ix.convert(A)
    if compressed and port == 'B':
        oB = ix.convert(B)
    ours = kernel(oA, oB, bias) if biased else kernel(oA, oB)
    if compressed and port == 'C':
        ours = ix.inverse(ours)
    torch.testing.assert_close(ours, theirs, **TOL)


@pytest.mark.parametrize('compressed', [False, True])
def test_softmax_matches_reference_kernels(ref, compressed):
    batch, H, W, BH, BW, RT = 4, 128, 256, 32, 32, 4
    g = torch.Generator().manual_seed(2022)
    x = torch.rand((batch, H, W), generator=g).cuda()
    grad = torch.rand((batch, H, W), generator=g).cuda()
    mask = oracle.block_mask((H, W), (8, 8), 0.9, generator=g).cuda()
    T = float(np.sqrt(W))
    rix = ref.build_indexes(mask, BH, BW, True, False)
    rmask = mask
    rx, rgrad = x * mask, grad * mask
    if compressed:
        rmask = ref.convert(mask.float().unsqueeze(0), rix).to(torch.uint8)
        rx, rgrad = ref.convert(rx, rix), ref.convert(rgrad, rix)
    ry = ref.softmax_forward(rx, rix, rmask, 1 / T, H, W, RT, compressed)
    rdx = ref.softmax_backward(rgrad, ry, rix, rmask, 1 / T, H, W, RT, compressed)
    if compressed:
        ry, rdx = ref.inverse(ry, rix), ref.inverse(rdx, rix)

    cfg = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': BH, 'BLOCK_SIZE_W_VALUE': BW, 'ROW_TILE_VALUE': RT}
    fwd = SparTASparseSoftmaxForwardKernel(compressed=compressed)
    bwd = SparTASparseSoftmaxBackwardKernel(compressed=compressed)
    for k in (fwd, bwd):
        k.ports['y'].set_mask(mask)
        k.set_shape(batch, H, W)
        k.compile(cfg)
    ix = fwd.ports['y'].indexes
    ox, ograd = x * mask, grad * mask
    if compressed:
        ox, ograd = ix.convert(ox), ix.convert(ograd)
    oy = fwd(ox, np.float32(1 / T))
    odx = bwd(ograd, oy, np.float32(1 / T))
    if compressed:
        oy, odx = ix.inverse(oy), ix.inverse(odx)
    torch.testing.assert_close(oy, ry, **TOL)
    torch.testing.assert_close(odx, rdx, **TOL)
    # and both agree with the CPU oracle
    want = oracle.softmax_forward_reference(x.cpu(), mask.cpu(), T)
    torch.testing.assert_close(ry.cpu(), want, **TOL)
