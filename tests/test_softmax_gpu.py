"""Sparse softmax through the C-ABI against the CPU oracle and the golden vectors, following
test/unit/test_sparse_softmax.py of the reference."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from sparta_b200.nn import SparseSoftmax
from sparta_b200.specializer.funtional import SparseBatchSoftmaxCtx, SparseBatchSoftmaxFunc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')
TOL = dict(rtol=1e-4, atol=1e-4)


def params(bh=32, bw=32):
    return {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': bh, 'BLOCK_SIZE_W_VALUE': bw, 'ROW_TILE_VALUE': 4}


def make_case(batch=4, H=128, W=256, granularity=(8, 8), sparsity=0.9, seed=2022):
    g = torch.Generator().manual_seed(seed)
    shape = (H, W) if batch is None else (batch, H, W)
    x = torch.rand(shape, generator=g)
    grad = torch.rand(shape, generator=g)
    mask = oracle.block_mask((H, W), granularity, sparsity, generator=g)
    T = float(np.sqrt(W))
    y = oracle.softmax_forward_reference(x, mask, T)
    dx = oracle.softmax_backward_reference(grad, y, mask, T)
    return x, grad, mask, T, y, dx


@pytest.mark.parametrize('compressed', [False, True])
def test_sparse_softmax_function(compressed):
    x, grad, mask, T, y, dx = make_case()
    ctx = SparseBatchSoftmaxCtx(compressed, T)
    names = list(ctx.get_kernel_placeholders(backward=True).keys())
    ctx.select_impls({n: 'sparta' for n in names})
    ctx.set_shape(4, 128, 256)
    for ports in ctx.sparse_ports.values():
        for p in ports:
            p.set_mask(mask.cuda())
    ctx.build({n: params() for n in names})
    ix = ctx.sparse_ports['y'][0].indexes
    xin, gin = x.cuda(), grad.cuda()
    if compressed:
        xin, gin = ix.convert(xin), ix.convert(gin)
    xin.requires_grad_()
    out = SparseBatchSoftmaxFunc.apply(ctx, xin)
    out.backward(gin)
    got_y, got_dx = out.detach(), xin.grad
    if compressed:
        got_y, got_dx = ix.inverse(got_y), ix.inverse(got_dx)
    torch.testing.assert_close(got_y.cpu(), y, **TOL)
    torch.testing.assert_close(got_dx.cpu(), dx, **TOL)


@pytest.mark.parametrize('batch', [None, 4])
@pytest.mark.parametrize('compressed', [False, True])
def test_sparse_softmax_operator_dynamic(compressed, batch):
    x, grad, mask, T, y, dx = make_case(batch)
    op = SparseSoftmax(mask.cuda(), T, compressed)
    op.build(config={n: params() for n in op.get_kernel_placeholders(backward=True)}, sample_inputs=[x.cuda()])
    for seed in range(3):
        ix = op.get_sparse_indexes('y')
        xin, gin = x.cuda(), grad.cuda()
        if compressed:
            xin, gin = ix.convert(xin), ix.convert(gin)
        xin.requires_grad_()
        out = op(xin)
        out.backward(gin)
        got_y, got_dx = out.detach(), xin.grad
        if compressed:
            got_y, got_dx = ix.inverse(got_y), ix.inverse(got_dx)
        torch.testing.assert_close(got_y.cpu(), y, **TOL)
        torch.testing.assert_close(got_dx.cpu(), dx, **TOL)
        x, grad, mask, T, y, dx = make_case(batch, seed=seed)
        op.update_mask(mask.cuda())


@pytest.mark.parametrize('compressed', [False, True])
@pytest.mark.parametrize('block', [(8, 16), (32, 32), (64, 128)])
def test_golden_vectors_and_fully_masked_rows(compressed, block):
    g = np.load(os.path.join(GOLDEN, 'softmax_attention.npz'))
    t = lambda k: torch.from_numpy(g[k])
    op = SparseSoftmax(t('mask').cuda(), float(g['T']), compressed)
    op.build({'forward:y': params(*block), 'backward:x': params(*block)}, sample_inputs=[t('x').cuda()])
    ix = op.get_sparse_indexes('y')
    xin = t('x').cuda()
    if compressed:
        xin = ix.convert(xin)
    out = op(xin)
    if compressed:
        out = ix.inverse(out)
    torch.testing.assert_close(out.cpu(), t('y'), **TOL)
    assert torch.all(out[:, 40:48] == 0)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_half_types_block_uniform_mask(dtype):
    g = torch.Generator().manual_seed(5)
    x = (torch.randn((3, 256, 512), generator=g) * 3).to(dtype)
    mask = oracle.block_mask((256, 512), (64, 64), 0.7, generator=g)
    op = SparseSoftmax(mask.cuda(), 2.0, compressed=True)
    op.build({'forward:y': params(64, 64)}, sample_inputs=[x.cuda()])
    ix = op.get_sparse_indexes('y')
    assert ix.block_uniform
    out = ix.inverse(op(ix.convert(x.cuda()))).float().cpu()
    torch.testing.assert_close(out, oracle.softmax_forward_reference(x.float(), mask, 2.0), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('compressed', [True, False])
def test_half_types_element_mask(dtype, compressed):
    """fp16 / bf16 with a mask finer than the block (8 x 8 inside 64 x 64 blocks, some rows fully masked
    inside kept blocks): the vector kernel overwrites masked values of the packed row before the maximum,
    and the backward pass sees the same element mask."""
    g = torch.Generator().manual_seed(6)
    x = (torch.randn((2, 256, 512), generator=g) * 3).to(dtype)
    grad = torch.randn((2, 256, 512), generator=g).to(dtype)
    mask = oracle.block_mask((256, 512), (8, 8), 0.6, generator=g)
    mask[72:80] = 0
    op = SparseSoftmax(mask.cuda(), 2.0, compressed=compressed)
    op.build({'forward:y': params(64, 64), 'backward:x': params(64, 64)}, sample_inputs=[x.cuda()])
    ix = op.get_sparse_indexes('y')
    assert not ix.block_uniform
    xin, gin = x.cuda(), grad.cuda()
    if compressed:
        xin, gin = ix.convert(xin), ix.convert(gin)
    xin.requires_grad_()
    out = op(xin)
    out.backward(gin)
    got_y, got_dx = out.detach(), xin.grad
    if compressed:
        got_y, got_dx = ix.inverse(got_y), ix.inverse(got_dx)
    want_y = oracle.softmax_forward_reference(x.float(), mask, 2.0)
    want_dx = oracle.softmax_backward_reference(grad.float(), want_y, mask, 2.0)
    torch.testing.assert_close(got_y.float().cpu(), want_y, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got_dx.float().cpu(), want_dx, rtol=2e-2, atol=2e-2)
    assert torch.all(got_y[:, 72:80] == 0)


@pytest.mark.parametrize('dtype,W', [(torch.float16, 8192), (torch.bfloat16, 8192), (torch.float32, 4096)])
@pytest.mark.parametrize('compressed', [True, False])
@pytest.mark.parametrize('element_mask', [False, True])
def test_row_lengths_across_the_kernel_paths(dtype, W, compressed, element_mask):
    """Block rows of very different lengths in one launch: a row that fits the registers (<= 4 KB of kept
    values), one that is processed in the shared-memory ring (<= 8 KB), one longer than the ring (scalar
    passes), and an empty one; 64-row blocks (eight rows per warp) and 16-row blocks (four).  The backward
    pass goes through its own ring (dy and y rows side by side) or scalar passes for the long rows."""
    esz = 4 if dtype == torch.float32 else 2
    g = torch.Generator().manual_seed(W + esz)
    for bh in (64, 16):
        H = 4 * bh
        x = (torch.randn((2, H, W), generator=g) * 2).to(dtype)
        blocks = torch.zeros((4, W // 64), dtype=torch.uint8)
        blocks[0, torch.randperm(W // 64, generator=g)[:3072 // esz // 64]] = 1        # 3 KB of kept values per row
        blocks[1, torch.randperm(W // 64, generator=g)[:7168 // esz // 64]] = 1        # 7 KB
        blocks[2] = 1                                                                   # 16 KB: the whole row
        mask = blocks.repeat_interleave(bh, 0).repeat_interleave(64, 1)
        if element_mask:
            mask = mask * (torch.rand((H, W), generator=g) > 0.3).to(torch.uint8)
            mask[bh + 3] = 0  # a fully masked row inside kept blocks
        grad = torch.randn((2, H, W), generator=g).to(dtype)
        op = SparseSoftmax(mask.cuda(), 3.0, compressed=compressed)
        op.build({'forward:y': params(bh, 64), 'backward:x': params(bh, 64)}, sample_inputs=[x.cuda()])
        ix = op.get_sparse_indexes('y')
        xin = (ix.convert(x.cuda()) if compressed else x.cuda()).requires_grad_()
        out = op(xin)
        out.backward(ix.convert(grad.cuda()) if compressed else grad.cuda())
        got = ix.inverse(out.detach()) if compressed else out.detach()
        got_dx = ix.inverse(xin.grad) if compressed else xin.grad
        want = oracle.softmax_forward_reference(x.float(), mask, 3.0)
        want_dx = oracle.softmax_backward_reference(grad.float(), want, mask, 3.0)
        tol = TOL if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(got.float().cpu(), want, **tol)
        torch.testing.assert_close(got_dx.float().cpu(), want_dx, **tol)
        assert torch.all(got[:, 3 * bh:] == 0) and torch.all(got_dx[:, 3 * bh:] == 0)
