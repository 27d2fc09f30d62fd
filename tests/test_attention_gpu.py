"""SparseAttention through the C-ABI against the CPU oracle, following
test/unit/test_sparse_attention.py of the reference (forward and q/k/v gradients over three rounds
of new masks), plus the fused half-precision forward kernel."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from sparta_b200.nn import SparseAttention

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')


def params(tile=32, softmax_tile=None):
    mm = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': tile, 'BLOCK_SIZE_K_VALUE': tile, 'BLOCK_SIZE_N_VALUE': tile}
    st = softmax_tile or tile
    sm = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': st, 'BLOCK_SIZE_W_VALUE': st, 'ROW_TILE_VALUE': 4}
    cfg = {}
    for k in ['forward:C', 'backward:A', 'backward:B']:
        cfg[f'qk/{k}'] = dict(mm)
        cfg[f'out/{k}'] = dict(mm)
    for k in ['forward:y', 'backward:x']:
        cfg[f'sm/{k}'] = dict(sm)
    return cfg


@pytest.mark.parametrize('H', [1, 4])
@pytest.mark.parametrize('Ns,Nt,E', [(256, 256, 256), (512, 256, 256), (256, 512, 512), (1024, 256, 256)])
def test_sparse_attention_operator(H, Ns, Nt, E):
    g = torch.Generator().manual_seed(2022)
    mask = oracle.block_mask((Nt, Ns), (8, 8), 0.95, generator=g)
    q = torch.rand((H, Nt, E), generator=g)
    k = torch.rand((H, Ns, E), generator=g)
    v = torch.rand((H, Ns, E), generator=g)
    grad = torch.rand((H, Nt, E), generator=g)
    op = SparseAttention(mask=mask.cuda())
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    op.build(config=params(), sample_inputs=[qc, kc, vc])
    for seed in range(3):
        qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
        target = oracle.attention_reference(qr, kr, vr, mask)
        target.backward(grad)
        qc.grad = kc.grad = vc.grad = None
        out = op(qc, kc, vc)
        out.backward(grad.cuda())
        tol = dict(atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(out.detach().cpu(), target.detach(), **tol)
        torch.testing.assert_close(qc.grad.cpu(), qr.grad, **tol)
        torch.testing.assert_close(kc.grad.cpu(), kr.grad, **tol)
        torch.testing.assert_close(vc.grad.cpu(), vr.grad, **tol)
        g2 = torch.Generator().manual_seed(seed)
        mask = oracle.block_mask((Nt, Ns), (8, 8), 0.95, generator=g2)
        op.update_mask(mask.cuda())


def test_golden_vector():
    g = np.load(os.path.join(GOLDEN, 'softmax_attention.npz'))
    t = lambda n: torch.from_numpy(g[n])
    op = SparseAttention(mask=t('amask').cuda())
    op.build(config=params(16, 16), sample_inputs=[t('q').cuda(), t('k').cuda(), t('v').cuda()])
    out = op(t('q').cuda(), t('k').cuda(), t('v').cuda())
    torch.testing.assert_close(out.cpu(), t('o'), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('E', [64, 128])
@pytest.mark.parametrize('fused', [False, 'auto'])
def test_half_precision_attention_band_mask(dtype, E, fused):
    """Band + global + random 64x64-block mask (the benchmark generator) at reduced size."""
    heads, S = 3, 1024
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn((heads, S, E), generator=g).to(dtype) for _ in range(3))
    mask = oracle.band_global_random_mask(S, S, 64, 2, 0.1, seed=4)
    op = SparseAttention(mask=mask.cuda(), fused=fused)
    op.build(config=params(64), sample_inputs=[q.cuda(), k.cuda(), v.cuda()])
    out = op(q.cuda(), k.cuda(), v.cuda())
    assert out.dtype == dtype
    target = oracle.attention_reference(q.float(), k.float(), v.float(), mask)
    torch.testing.assert_close(out.float().cpu(), target, atol=2e-2, rtol=2e-2)
    if fused == 'auto' and op._use_fused:
        assert op.fused_status() == [0, 0, 0, 0]


def _fused_case(dtype, E, heads, Nt, Ns, mask, seed=5, qscale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn((heads, Nt, E), generator=g) * qscale).to(dtype)
    k = torch.randn((heads, Ns, E), generator=g).to(dtype)
    v = torch.randn((heads, Ns, E), generator=g).to(dtype)
    op = SparseAttention(mask=mask.cuda(), fused=True)
    op.build(config=params(64), sample_inputs=[q.cuda(), k.cuda(), v.cuda()])
    assert op._use_fused
    out = op(q.cuda(), k.cuda(), v.cuda())
    assert op.fused_status() == [0, 0, 0, 0]
    target = oracle.attention_reference(q.float(), k.float(), v.float(), mask)
    torch.testing.assert_close(out.float().cpu(), target, atol=2e-2, rtol=2e-2)
    return op, (q, k, v)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('E', [64, 128])
def test_fused_attention_edge_masks(dtype, E):
    """Fused kernel: empty block rows, a single block, odd merged lists, rectangular masks."""
    g = torch.Generator().manual_seed(9)
    # rectangular, random blocks, one block row without any block and one Q tile without any block
    mask = oracle.block_mask((512, 768), (64, 64), 0.6, generator=g)
    mask[64:128] = 0
    mask[256:384] = 0
    _fused_case(dtype, E, 2, 512, 768, mask)
    # exactly one kept block
    one = torch.zeros((256, 256), dtype=torch.uint8)
    one[128:192, 64:128] = 1
    _fused_case(dtype, E, 1, 256, 256, one)
    # fully dense
    _fused_case(dtype, E, 1, 256, 384, torch.ones((256, 384), dtype=torch.uint8))


@pytest.mark.parametrize('E', [64, 128])
def test_fused_attention_element_mask_and_large_scores(E):
    """8x8-granular mask inside 64x64 blocks (element masking in the kernel) and scores whose running
    maximum keeps growing (exercises the rescale of the accumulator)."""
    g = torch.Generator().manual_seed(10)
    mask = oracle.block_mask((256, 512), (8, 8), 0.9, generator=g)
    mask[40:48] = 0  # rows that are fully masked inside kept blocks
    op, _ = _fused_case(torch.float16, E, 2, 256, 512, mask)
    assert not op.get_sparse_indexes().block_uniform
    dense = torch.ones((256, 1024), dtype=torch.uint8)
    _fused_case(torch.float16, E, 1, 256, 1024, dense, seed=11, qscale=6.0)


def test_fused_attention_dynamic_mask():
    g = torch.Generator().manual_seed(12)
    mask = oracle.block_mask((256, 256), (64, 64), 0.5, generator=g)
    op, (q, k, v) = _fused_case(torch.float16, 64, 2, 256, 256, mask)
    for seed in range(2):
        g2 = torch.Generator().manual_seed(seed)
        mask = oracle.block_mask((256, 256), (64, 64), 0.5, generator=g2)
        op.update_mask(mask.cuda())
        out = op(q.cuda(), k.cuda(), v.cuda())
        target = oracle.attention_reference(q.float(), k.float(), v.float(), mask)
        torch.testing.assert_close(out.float().cpu(), target, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_default_fused_setting_trains(dtype):
    """fused='auto' (the default) with half-precision inputs that require gradients: the forward must take
    the differentiable three-operator path, as the reference's operator does, and match oracle autograd."""
    heads, S, E = 2, 256, 64
    g = torch.Generator().manual_seed(13)
    q, k, v = (torch.randn((heads, S, E), generator=g).to(dtype) for _ in range(3))
    grad = torch.randn((heads, S, E), generator=g).to(dtype)
    mask = oracle.band_global_random_mask(S, S, 64, 1, 0.1, seed=5)
    op = SparseAttention(mask=mask.cuda())
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    op.build(config=params(64), sample_inputs=[qc, kc, vc])
    assert op._use_fused  # the configuration is fusable: inference calls take the fused kernel
    out = op(qc, kc, vc)
    out.backward(grad.cuda())
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    target = oracle.attention_reference(qr, kr, vr, mask)
    target.backward(grad.float())
    tol = dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.detach().float().cpu(), target.detach(), **tol)
    for got, want in ((qc.grad, qr.grad), (kc.grad, kr.grad), (vc.grad, vr.grad)):
        torch.testing.assert_close(got.float().cpu(), want, **tol)
    with torch.no_grad():
        fused_out = op(qc, kc, vc)
    assert op.fused_status() == [0, 0, 0, 0]
    torch.testing.assert_close(fused_out.float().cpu(), target.detach(), **tol)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('E', [64, 128])
def test_fused_attention_odd_tile_count(dtype, E):
    """384 query rows = three 128-row tiles: with a head dimension of 128 the kernel with two Q tiles per CTA
    does not apply (it wants a multiple of 256 rows) and the one-tile kernel runs; both must agree with the oracle."""
    g = torch.Generator().manual_seed(21)
    mask = oracle.block_mask((384, 640), (64, 64), 0.5, generator=g)
    _fused_case(dtype, E, 3, 384, 640, mask, seed=22)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_fused_attention_with_copies_of_the_output(dtype):
    """The forward that also stores every output tile to further buffers (the peers' gathered outputs when
    heads are sharded; here two more buffers on the same GPU): all destinations hold the same bits as the
    plain forward, including tiles without any block (zeros) and with an element mask."""
    from sparta_b200 import _lib
    g = torch.Generator().manual_seed(12)
    mask = oracle.block_mask((512, 768), (64, 64), 0.6, generator=g)
    mask[64:128] = 0
    mask[256:512] = 0                      # a whole pair of Q tiles without any block
    fine = oracle.block_mask((512, 768), (8, 8), 0.3, generator=g)
    for m in (mask, mask * fine):
        op, (q, k, v) = _fused_case(dtype, 128, 3, 512, 768, m)
        want = op(q.cuda(), k.cuda(), v.cuda())
        full = torch.full((3, 3, 512, 128), 7.0, dtype=dtype, device='cuda')  # [destination, heads, Nt, E]
        out = op.forward_gathered(q.cuda(), k.cuda(), v.cuda(), full[0], [full[1].data_ptr(), full[2].data_ptr()])
        assert op.fused_status() == [0, 0, 0, 0]
        assert out.data_ptr() == full[0].data_ptr()
        for d in range(3):
            assert torch.equal(full[d], want), f'destination {d}'
    # the one-tile kernel (E = 64, or an odd number of Q tiles) stores O only and says so
    op, (q, k, v) = _fused_case(dtype, 64, 1, 256, 256, torch.ones((256, 256), dtype=torch.uint8))
    buf = torch.empty((2, 1, 256, 64), dtype=dtype, device='cuda')
    with pytest.raises(_lib.SpartaError):
        op.forward_gathered(q.cuda(), k.cuda(), v.cuda(), buf[0], [buf[1].data_ptr()])


def tc_params():
    """Every matmul of the three-operator attention on a tcgen05 tile (32 x 32 sparse blocks): the two dds products
    on 32 x 64 x 32, the four sdd products (stored [K, N] dense operands included) on 32 x 32 x 128."""
    tc = {'_impl': 'sparta', '_family': 'tcgen05'}
    dds = {**tc, 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 32}
    sdd = {**tc, 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 128}
    sm = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': 32, 'BLOCK_SIZE_W_VALUE': 32, 'ROW_TILE_VALUE': 4}
    return {'qk/forward:C': dds, 'qk/backward:A': sdd, 'qk/backward:B': sdd,
            'out/forward:C': sdd, 'out/backward:A': dds, 'out/backward:B': sdd,
            'sm/forward:y': sm, 'sm/backward:x': sm}


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_three_operator_attention_trains_on_tcgen05(dtype):
    """Forward and q / k / v gradients of the composed attention with all six matmuls pinned to the tcgen05 kernels
    (a head dimension of 256 keeps the fused kernel out), against oracle autograd."""
    from sparta_b200 import _lib
    heads, Nt, Ns, E = 2, 256, 384, 256
    g = torch.Generator().manual_seed(14)
    q = torch.randn((heads, Nt, E), generator=g).to(dtype)
    k, v = (torch.randn((heads, Ns, E), generator=g).to(dtype) for _ in range(2))
    grad = torch.randn((heads, Nt, E), generator=g).to(dtype)
    mask = oracle.block_mask((Nt, Ns), (32, 32), 0.6, generator=g)
    mask[64:96] = 0
    op = SparseAttention(mask=mask.cuda())
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    op.build(config=tc_params(), sample_inputs=[qc, kc, vc])
    assert not op._use_fused
    out = op(qc, kc, vc)
    out.backward(grad.cuda())
    assert _lib.last_status() == [0, 0, 0, 0]
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    target = oracle.attention_reference(qr, kr, vr, mask)
    target.backward(grad.float())
    tol = dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out.detach().float().cpu(), target.detach(), **tol)
    for got, want in ((qc.grad, qr.grad), (kc.grad, kr.grad), (vc.grad, vr.grad)):
        torch.testing.assert_close(got.float().cpu(), want, **tol)
