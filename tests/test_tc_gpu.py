"""The tcgen05 / TMEM / TMA kernels through the C-ABI against the CPU oracle (2e-2 for fp16 / bf16),
forced with ``_family='tcgen05'`` so that a silent fall-back to the FMA kernel cannot pass."""
import pytest
import torch

from oracle import oracle
from sparta_b200 import _lib
from sparta_b200.specializer.kernels import SparTASparseMatMulKernel

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-2, atol=2e-2)


def _dsd_case(batch, M, K, N, sparsity, dtype, biased, seed, empty_rows=()):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((batch, M, K), generator=g).to(dtype)
    w = (torch.randn((batch, N, K), generator=g) * 0.1).to(dtype)
    b = torch.randn((batch, N), generator=g).to(dtype) if biased else None
    mask = oracle.block_mask((N, K), (32, 32), sparsity, generator=g)
    for r in empty_rows:
        mask[r * 32:(r + 1) * 32] = 0
    return x, w * mask, b, mask


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('biased', [False, True])
@pytest.mark.parametrize('batch,M,K,N,sparsity', [
    (1, 128, 64, 32, 0.0),      # one tile, two K blocks
    (2, 256, 256, 192, 0.5),    # partial panel (6 block columns), batch
    (1, 512, 1024, 1024, 0.9),  # several panels, sparse rows
    (1, 384, 2048, 544, 0.75),  # 17 block columns: a full and a one-column panel
    (1, 128, 96, 416, 0.5),     # odd number of K blocks (a half-empty last step), 13 block columns
    (3, 256, 4096, 384, 0.97),  # long K, most steps empty: the rings wrap many times with few blocks
])
def test_dsd_tcgen05(dtype, biased, batch, M, K, N, sparsity):
    x, w, b, mask = _dsd_case(batch, M, K, N, sparsity, dtype, biased, seed=M + K + N,
                              empty_rows=(1,) if N >= 192 else ())
    kernel = SparTASparseMatMulKernel(mode='dsd', biased=biased, transpose_A=False, transpose_B=True,
                                      compressed=True)
    kernel.ports['B'].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    kernel.compile({'_impl': 'sparta', '_family': 'tcgen05', 'BLOCK_SIZE_M_VALUE': 128,
                    'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 32})
    ix = kernel.ports['B'].indexes
    args = [x.cuda(), ix.convert(w.cuda())] + ([b.cuda()] if biased else [])
    out = kernel(*args)
    assert _lib.last_status() == [0, 0, 0, 0]
    expect = oracle.matmul_reference(x.float(), w.float(), b.float() if biased else None, mask, 'dsd',
                                     False, True, (32, 32))
    torch.testing.assert_close(out.float().cpu(), expect, **TOL)
    # same answer as the FMA kernel on the same inputs (tighter: both accumulate in fp32)
    kernel.compile({'_impl': 'sparta', '_family': 'simt', 'BLOCK_SIZE_M_VALUE': 64,
                    'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 32})
    ref = kernel(*args)
    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


def test_dsd_tcgen05_is_deterministic():
    x, w, b, mask = _dsd_case(1, 256, 512, 512, 0.8, torch.float16, True, seed=3)
    kernel = SparTASparseMatMulKernel(mode='dsd', biased=True, transpose_A=False, transpose_B=True,
                                      compressed=True)
    kernel.ports['B'].set_mask(mask.cuda())
    kernel.set_shape(1, 256, 512, 512)
    kernel.compile({'_impl': 'sparta', '_family': 'tcgen05', 'BLOCK_SIZE_M_VALUE': 128,
                    'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 32})
    ix = kernel.ports['B'].indexes
    args = [x.cuda(), ix.convert(w.cuda()), b.cuda()]
    a = kernel(*args)
    c = kernel(*args)
    assert torch.equal(a, c)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('trans_B', [True, False])
@pytest.mark.parametrize('compressed', [True, False])
@pytest.mark.parametrize('batch,M,K,N,sparsity,biased', [
    (1, 128, 64, 32, 0.0, False),      # one tile, one column, one K chunk
    (2, 256, 256, 320, 0.5, True),     # two groups (10 columns), batch, bias
    (1, 512, 1024, 1024, 0.9, False),  # sparse: most groups empty
    (1, 384, 128, 2048, 0.97, True),   # row tiles without any block
])
def test_dds_tcgen05(dtype, trans_B, compressed, batch, M, K, N, sparsity, biased):
    g = torch.Generator().manual_seed(M + K + N)
    A = torch.randn((batch, M, K), generator=g).to(dtype)
    B = (torch.randn((batch, N, K) if trans_B else (batch, K, N), generator=g) * 0.1).to(dtype)
    bias = torch.randn((batch, N), generator=g).to(dtype) if biased else None
    mask = oracle.block_mask((M, N), (32, 32), sparsity, generator=g)
    if M >= 384:
        mask[128:256] = 0
    kernel = SparTASparseMatMulKernel(mode='dds', biased=biased, transpose_A=False, transpose_B=trans_B,
                                      compressed=compressed)
    kernel.ports['C'].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 32}
    kernel.compile({**cfg, '_family': 'tcgen05'})
    ix = kernel.ports['C'].indexes
    args = [A.cuda(), B.cuda()] + ([bias.cuda()] if biased else [])
    out = kernel(*args)
    assert _lib.last_status() == [0, 0, 0, 0]
    dense = ix.inverse(out) if compressed else out
    expect = oracle.matmul_reference(A.float(), B.float(), bias.float() if biased else None, mask, 'dds',
                                     False, trans_B, (32, 32))
    torch.testing.assert_close(dense.float().cpu(), expect, **TOL)
    kernel.compile({**cfg, '_family': 'simt'})
    ref = kernel(*args)
    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


def test_dds_tcgen05_per_batch_masks():
    from sparta_b200.nn import SparseBatchMatMul
    batch, M, K, N = 4, 256, 128, 512
    g = torch.Generator().manual_seed(21)
    A = torch.randn((batch, M, K), generator=g).half()
    B = torch.randn((batch, K, N), generator=g).half()
    masks = torch.stack([oracle.block_mask((M, N), (32, 32), 0.85, generator=g) for _ in range(batch)]).cuda()
    op = SparseBatchMatMul(C_mask=masks, compressed=True, capacity=96)
    op.build({'forward:C': {'_impl': 'sparta', '_family': 'tcgen05', 'BLOCK_SIZE_M_VALUE': 32,
                            'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 32}},
             sample_inputs=[A.cuda(), B.cuda()])
    op.set_dynamic(True)
    out = op(A.cuda(), B.cuda())
    assert _lib.last_status() == [0, 0, 0, 0]
    ix = op.get_sparse_indexes('C')
    full = torch.bmm(A.float(), B.float())
    torch.testing.assert_close(ix.inverse(out).float().cpu(), full * masks.cpu().float(), **TOL)


def test_tune_reaches_the_tcgen05_kernel():
    """The three lines of the reference's README on half-precision inputs: ``tune`` walks the tile table,
    so it can return the 128 x 32 x 32 tile, and building that result launches the tcgen05 dsd kernel."""
    from sparta_b200.nn import SparseLinear, tune
    g = torch.Generator().manual_seed(7)
    dense = torch.nn.Linear(2048, 2048).half().cuda()
    mask = oracle.block_mask((2048, 2048), (32, 32), 0.75, generator=g).cuda()
    x = torch.randn((2048, 2048), generator=g).half().cuda()
    sparse_linear = SparseLinear(dense, weight_mask=mask)
    best = tune(sparse_linear, sample_inputs=[x], max_trials=10 ** 6)
    cfg = best['root']['forward:C']
    tile = tuple(cfg[f'BLOCK_SIZE_{d}_VALUE'] for d in 'MKN')
    assert cfg['_impl'] == 'sparta' and tile == (128, 32, 32), cfg
    sparse_linear.build(best['root'], sample_inputs=[x])
    kernel = sparse_linear.get_kernel_placeholders()['forward:C'].active_kernel()
    assert kernel.tile_shapes(torch.float16)[tile] == _lib.IMPL_TCGEN05
    y = sparse_linear(x)
    assert _lib.last_status() == [0, 0, 0, 0]
    expect = torch.nn.functional.linear(x.float().cpu(), (dense.weight.float() * mask).cpu(), dense.bias.float().cpu())
    torch.testing.assert_close(y.float().cpu(), expect, **TOL)
    # the same tile with the family pinned gives the same bits: AUTO did dispatch to tcgen05
    pinned = {'forward:C': {**cfg, '_family': 'tcgen05'}}
    sparse_linear.build(pinned, sample_inputs=[x])
    assert torch.equal(sparse_linear(x), y)


def _run_both_families(kernel, cfg, simt_cfg, args):
    kernel.compile({**cfg, '_family': 'tcgen05'})
    out = kernel(*args)
    assert _lib.last_status() == [0, 0, 0, 0]
    kernel.compile({**simt_cfg, '_family': 'simt'})
    return out, kernel(*args)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('both_forms', [False, True])  # BCSC alone (values in BCSC order), or 64-bit entries into BCSR order
@pytest.mark.parametrize('batch,M,K,N,sparsity', [
    (1, 128, 64, 32, 0.0),
    (2, 256, 256, 192, 0.5),
    (1, 512, 1024, 1024, 0.9),
    (1, 384, 2048, 544, 0.75),
    (1, 128, 96, 416, 0.5),
    (2, 256, 4096, 384, 0.97),
])
def test_dsd_nn_tcgen05(dtype, both_forms, batch, M, K, N, sparsity):
    """The SparseLinear input gradient: B stored [K, N] and indexed by column (BCSC), blocks MN-major."""
    g = torch.Generator().manual_seed(M + K + N + 1)
    x = torch.randn((batch, M, K), generator=g).to(dtype)
    w = (torch.randn((batch, K, N), generator=g) * 0.1).to(dtype)
    mask = oracle.block_mask((K, N), (32, 32), sparsity, generator=g)
    if N >= 192:
        mask[:, 32:64] = 0  # a block column without any block
    w = w * mask
    kernel = SparTASparseMatMulKernel(mode='dsd', biased=False, transpose_A=False, transpose_B=False,
                                      compressed=True)
    if both_forms:
        kernel.ports['B'].set_sparse(True, True)
    kernel.ports['B'].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    cfg = {'_impl': 'sparta', 'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 32}
    kernel.compile({**cfg, 'BLOCK_SIZE_M_VALUE': 128, '_family': 'tcgen05'})
    ix = kernel.ports['B'].indexes
    args = [x.cuda(), ix.convert(w.cuda())]
    out, ref = _run_both_families(kernel, {**cfg, 'BLOCK_SIZE_M_VALUE': 128}, {**cfg, 'BLOCK_SIZE_M_VALUE': 64}, args)
    expect = oracle.matmul_reference(x.float(), w.float(), None, mask, 'dsd', False, False, (32, 32))
    torch.testing.assert_close(out.float().cpu(), expect, **TOL)
    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('trans_A,both_forms', [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize('batch,M,K,N,sparsity,biased', [
    (1, 32, 64, 128, 0.0, False),
    (2, 192, 256, 256, 0.5, True),
    (1, 1024, 1024, 512, 0.9, False),
    (1, 544, 2048, 384, 0.75, True),
    (2, 384, 4096, 256, 0.97, True),
])
@pytest.mark.parametrize('trans_B', [True, False])
def test_sdd_tcgen05(dtype, trans_A, both_forms, batch, M, K, N, sparsity, biased, trans_B):
    """sdd against a dense B stored [N, K] runs as C^T = B A^T on the dsd kernel with a transposed store; a B
    stored [K, N] (the P V product of attention) gets there through a transposed copy."""
    g = torch.Generator().manual_seed(M + K + N + 2)
    a = (torch.randn((batch, K, M) if trans_A else (batch, M, K), generator=g) * 0.1).to(dtype)
    b = torch.randn((batch, N, K) if trans_B else (batch, K, N), generator=g).to(dtype)
    bias = torch.randn((batch, N), generator=g).to(dtype) if biased else None
    mask = oracle.block_mask((K, M) if trans_A else (M, K), (32, 32), sparsity, generator=g)
    if M >= 192:
        if trans_A:
            mask[:, 32:64] = 0
        else:
            mask[32:64] = 0  # a block row of A without any block: those rows of C are bias only
    a = a * mask
    kernel = SparTASparseMatMulKernel(mode='sdd', biased=biased, transpose_A=trans_A, transpose_B=trans_B,
                                      compressed=True)
    if both_forms:
        kernel.ports['A'].set_sparse(True, True)
    kernel.ports['A'].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 32}
    kernel.compile({**cfg, 'BLOCK_SIZE_N_VALUE': 128, '_family': 'tcgen05'})
    ix = kernel.ports['A'].indexes
    args = [ix.convert(a.cuda()), b.cuda()] + ([bias.cuda()] if biased else [])
    out, ref = _run_both_families(kernel, {**cfg, 'BLOCK_SIZE_N_VALUE': 128}, {**cfg, 'BLOCK_SIZE_N_VALUE': 64}, args)
    expect = oracle.matmul_reference(a.float(), b.float(), bias.float() if biased else None, mask, 'sdd',
                                     trans_A, trans_B, (32, 32))
    torch.testing.assert_close(out.float().cpu(), expect, **TOL)
    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('trans_B', [True, False])
@pytest.mark.parametrize('compressed', [True, False])
@pytest.mark.parametrize('batch,M,K,N,sparsity', [
    (1, 128, 64, 32, 0.0),
    (2, 256, 256, 320, 0.5),
    (1, 512, 1024, 1024, 0.9),
    (1, 384, 128, 2048, 0.97),
])
def test_dds_tn_tcgen05(dtype, trans_B, compressed, batch, M, K, N, sparsity):
    """The SparseLinear weight gradient: A stored [K, M] (MN-major A operand)."""
    g = torch.Generator().manual_seed(M + K + N + 3)
    A = torch.randn((batch, K, M), generator=g).to(dtype)
    B = (torch.randn((batch, N, K) if trans_B else (batch, K, N), generator=g) * 0.1).to(dtype)
    mask = oracle.block_mask((M, N), (32, 32), sparsity, generator=g)
    kernel = SparTASparseMatMulKernel(mode='dds', biased=False, transpose_A=True, transpose_B=trans_B,
                                      compressed=compressed)
    kernel.ports['C'].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 32}
    kernel.compile({**cfg, '_family': 'tcgen05'})
    ix = kernel.ports['C'].indexes
    out, ref = _run_both_families(kernel, cfg, cfg, [A.cuda(), B.cuda()])
    dense = ix.inverse(out) if compressed else out
    expect = oracle.matmul_reference(A.float(), B.float(), None, mask, 'dds', True, trans_B, (32, 32))
    torch.testing.assert_close(dense.float().cpu(), expect, **TOL)
    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_sparse_linear_trains_on_tcgen05(dtype):
    """Forward, input gradient and weight gradient of SparseLinear all on the tcgen05 kernels, against
    the oracle's autograd on the masked dense layer."""
    from sparta_b200.nn import SparseLinear
    M, K, N = 512, 768, 640
    g = torch.Generator().manual_seed(11)
    mask = oracle.block_mask((N, K), (32, 32), 0.8, generator=g)
    dense = torch.nn.Linear(K, N, dtype=dtype)
    with torch.no_grad():
        dense.weight.copy_((torch.randn((N, K), generator=g) * 0.05).to(dtype))
        dense.bias.copy_(torch.randn((N,), generator=g).to(dtype))
    x = torch.randn((M, K), generator=g).to(dtype)
    gy = (torch.randn((M, N), generator=g) * 0.1).to(dtype)
    op = SparseLinear(dense.cuda(), weight_mask=mask.cuda())
    tc = {'_impl': 'sparta', '_family': 'tcgen05'}
    op.build({
        'forward:C': {**tc, 'BLOCK_SIZE_M_VALUE': 128, 'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 32},
        'backward:A': {**tc, 'BLOCK_SIZE_M_VALUE': 128, 'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 32},
        'backward:B': {**tc, 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 32},
    }, sample_inputs=[x.cuda()])
    xg = x.cuda().requires_grad_(True)
    y = op(xg)
    y.backward(gy.cuda())
    assert _lib.last_status() == [0, 0, 0, 0]
    # oracle: fp32 autograd on the masked dense layer
    xr = x.float().requires_grad_(True)
    wr = (dense.weight.detach().float().cpu() * mask).requires_grad_(True)
    br = dense.bias.detach().float().cpu().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(gy.float())
    torch.testing.assert_close(y.float().cpu(), yr.detach(), **TOL)
    torch.testing.assert_close(xg.grad.float().cpu(), xr.grad, **TOL)
    gw = op.get_sparse_indexes('B').inverse(op.weight.grad.unsqueeze(0)).squeeze(0)  # the weight is held compressed
    torch.testing.assert_close(gw.float().cpu(), wr.grad * mask, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(op.bias.grad.float().cpu(), br.grad, rtol=2e-2, atol=1e-1)


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('biased', [False, True])
def test_dsd_tcgen05_panels_without_blocks(dtype, biased):
    """Masks that leave whole panels of block rows empty (and one that is empty but for a single block): those
    panels take the kernel's early exit and must come out as the bias (or zero)."""
    batch, M, K, N = 2, 256, 512, 1024
    g = torch.Generator().manual_seed(31)
    x = torch.randn((batch, M, K), generator=g).to(dtype)
    w = (torch.randn((batch, N, K), generator=g) * 0.1).to(dtype)
    b = torch.randn((batch, N), generator=g).to(dtype) if biased else None
    for variant in range(2):
        mask = torch.zeros((N, K), dtype=torch.uint8)
        if variant == 0:
            mask[640:672, 96:128] = 1            # a single block
        else:
            mask[:320] = oracle.block_mask((320, K), (32, 32), 0.7, generator=g)  # first panel(s) only
        kernel = SparTASparseMatMulKernel(mode='dsd', biased=biased, transpose_A=False, transpose_B=True, compressed=True)
        kernel.ports['B'].set_mask(mask.cuda())
        kernel.set_shape(batch, M, K, N)
        kernel.compile({'_impl': 'sparta', '_family': 'tcgen05', 'BLOCK_SIZE_M_VALUE': 128, 'BLOCK_SIZE_K_VALUE': 32,
                        'BLOCK_SIZE_N_VALUE': 32})
        ix = kernel.ports['B'].indexes
        args = [x.cuda(), ix.convert((w * mask).cuda())] + ([b.cuda()] if biased else [])
        out = kernel(*args)
        assert _lib.last_status() == [0, 0, 0, 0]
        expect = oracle.matmul_reference(x.float(), (w * mask).float(), b.float() if biased else None, mask, 'dsd',
                                         False, True, (32, 32))
        torch.testing.assert_close(out.float().cpu(), expect, **TOL)
