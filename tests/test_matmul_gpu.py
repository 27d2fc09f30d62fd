"""Block-sparse matmul through the C-ABI against the CPU oracle (masked-dense torch), following
test/unit/test_sparse_matmul.py of the reference: kernel matrix, autograd function, operators with
three rounds of new masks, SparseLinear.  fp32: rtol = atol = 1e-4; fp16 / bf16: 2e-2."""
from typing import Dict, Tuple

import pytest
import torch

from oracle import oracle
from sparta_b200.nn import SparseBatchMatMul, SparseLinear
from sparta_b200.specializer.funtional import SparseBatchMatMulCtx, SparseBatchMatMulFunc
from sparta_b200.specializer.kernels import SparTASparseMatMulKernel, OpenAISparseMatMulKernel

pytestmark = pytest.mark.gpu

TOL = {torch.float32: dict(rtol=1e-4, atol=1e-4), torch.float16: dict(rtol=2e-2, atol=2e-2),
       torch.bfloat16: dict(rtol=2e-2, atol=2e-2)}
SPARSE_PORT = {'sdd': 'A', 'dsd': 'B', 'dds': 'C'}


def make_case(batch=4, M=128, K=256, N=192, granularity=(8, 8), sparsity=0.9, mode='dds', trans_A=False,
              trans_B=False, biased=False, seed=2022, dtype=torch.float32, scale=1.0):
    """Seeded CPU inputs (values representable in ``dtype``) and the mask of the sparse tensor."""
    g = torch.Generator().manual_seed(seed)
    shapes = {'A': (K, M) if trans_A else (M, K), 'B': (N, K) if trans_B else (K, N), 'C': (M, N)}
    lead = (batch,) if batch > 0 else ()
    data = {n: (torch.rand(lead + shapes[n], generator=g) * scale).to(dtype).float() for n in 'AB'}
    if biased:
        data['bias'] = torch.rand(lead + (N,), generator=g).to(dtype).float()
    data['grad_C'] = torch.rand(lead + shapes['C'], generator=g).to(dtype).float()
    port = SPARSE_PORT[mode]
    mask = oracle.block_mask(shapes[port], granularity, sparsity, generator=g)
    if port in 'AB':
        data[port] = data[port] * mask
    return data, mask


def params(impl='sparta', tile=32):
    if impl == 'sparta':
        return {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': tile, 'BLOCK_SIZE_K_VALUE': tile,
                'BLOCK_SIZE_N_VALUE': tile, 'THREAD_SIZE_M_VALUE': 4, 'THREAD_SIZE_K_VALUE': 4,
                'THREAD_SIZE_N_VALUE': 4}
    return {'_impl': impl}


def block_of(mode, tile_m, tile_k, tile_n, trans_A, trans_B):
    if mode == 'sdd':
        return (tile_k, tile_m) if trans_A else (tile_m, tile_k)
    if mode == 'dsd':
        return (tile_n, tile_k) if trans_B else (tile_k, tile_n)
    return (tile_m, tile_n)


@pytest.mark.parametrize('impl', ['sparta', 'openai'])
@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('biased', [False, True])
@pytest.mark.parametrize('trans_A', [False, True])
@pytest.mark.parametrize('trans_B', [False, True])
@pytest.mark.parametrize('compressed', [False, True])
def test_sparse_matmul_kernel(impl, mode, biased, compressed, trans_A, trans_B):
    batch, M, K, N = 4, 128, 256, 192
    data, mask = make_case(batch, M, K, N, mode=mode, trans_A=trans_A, trans_B=trans_B, biased=biased)
    cls = SparTASparseMatMulKernel if impl == 'sparta' else OpenAISparseMatMulKernel
    kernel = cls(mode=mode, biased=biased, transpose_A=trans_A, transpose_B=trans_B, compressed=compressed)
    port = SPARSE_PORT[mode]
    kernel.ports[port].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    kernel.compile(params(impl))
    tiles = kernel.get_block_shape()
    ix = kernel.ports[port].indexes

    bias = data.get('bias')
    expect = oracle.matmul_reference(data['A'], data['B'], bias, mask, mode, trans_A, trans_B,
                                     block_of(mode, *tiles, trans_A, trans_B))
    inputs = [data['A'].cuda(), data['B'].cuda()]
    if compressed and port in 'AB':
        i = 'AB'.index(port)
        inputs[i] = ix.convert(inputs[i])
    if biased:
        inputs.append(bias.cuda())
    out = kernel(*inputs)
    if compressed and port == 'C':
        assert out.shape == (batch, ix.block_nnz * tiles[0] * tiles[2])
        out = ix.inverse(out)
    torch.testing.assert_close(out.cpu(), expect, **TOL[torch.float32])
    # the module's own self-test (reference: kernel.test -> check + profile) must agree too
    test_inputs = [data['A'].cuda(), data['B'].cuda()] + ([bias.cuda()] if biased else [])
    assert kernel.test(test_inputs, num_warmups=0, num_iters=1, cuda=False) < float('inf')


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('tile', [8, 16, 64])
def test_half_types_and_tile_sizes(dtype, mode, tile):
    batch, M, K, N = 2, 128, 256, 192
    data, mask = make_case(batch, M, K, N, mode=mode, trans_B=True, biased=True, dtype=dtype, seed=7)
    kernel = SparTASparseMatMulKernel(mode=mode, biased=True, transpose_A=False, transpose_B=True,
                                      compressed=True)
    port = SPARSE_PORT[mode]
    kernel.ports[port].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    kernel.compile(params('sparta', tile))
    ix = kernel.ports[port].indexes
    expect = oracle.matmul_reference(data['A'], data['B'], data['bias'], mask, mode, False, True,
                                     block_of(mode, tile, tile, tile, False, True))
    inputs = [data['A'].to(dtype).cuda(), data['B'].to(dtype).cuda()]
    if port in 'AB':
        i = 'AB'.index(port)
        inputs[i] = ix.convert(inputs[i])
    out = kernel(*inputs, data['bias'].to(dtype).cuda())
    assert out.dtype == dtype
    if port == 'C':
        out = ix.inverse(out)
    torch.testing.assert_close(out.float().cpu(), expect, **TOL[dtype])


def reference_grads(data, mask, mode, trans_A, trans_B, biased, block):
    """Autograd through the masked-dense oracle: target C, dA, dB, dbias."""
    A = data['A'].clone().requires_grad_()
    B = data['B'].clone().requires_grad_()
    bias = data['bias'].clone().requires_grad_() if biased else None
    # data['A'] / data['B'] are already multiplied by the element mask; differentiate with respect to
    # that masked tensor, so its gradient is the dense gradient restricted to the covered blocks
    ones = torch.ones_like(mask)
    C = oracle.matmul_reference(A, B, bias, mask if mode == 'dds' else ones, mode, trans_A, trans_B, block)
    cover = torch.from_numpy(oracle.block_cover_mask(mask.numpy(), *block)).float()
    grad_C = data['grad_C'] * cover if mode == 'dds' else data['grad_C']
    C.backward(grad_C)
    gA, gB = A.grad, B.grad
    port = SPARSE_PORT[mode]
    if port == 'A':
        gA = gA * cover
    elif port == 'B':
        gB = gB * cover
    return C.detach(), gA, gB, (bias.grad if biased else None), grad_C


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('biased', [False, True])
@pytest.mark.parametrize('trans_A', [False, True])
@pytest.mark.parametrize('trans_B', [False, True])
@pytest.mark.parametrize('compressed', [False, True])
def test_sparse_matmul_function(mode, biased, compressed, trans_A, trans_B):
    batch, M, K, N = 4, 128, 256, 192
    data, mask = make_case(batch, M, K, N, mode=mode, trans_A=trans_A, trans_B=trans_B, biased=biased)
    ctx = SparseBatchMatMulCtx(mode, trans_A, trans_B, biased, compressed)
    names = list(ctx.get_kernel_placeholders(backward=True).keys())
    ctx.select_impls({n: 'sparta' for n in names})
    ctx.set_shape(batch, M, K, N)
    for port_name, ports in ctx.sparse_ports.items():
        for p in ports:
            p.set_mask(mask.cuda())
    ctx.build({n: params() for n in names})
    port = SPARSE_PORT[mode]
    block = block_of(mode, 32, 32, 32, trans_A, trans_B)
    C, gA, gB, gbias, grad_C = reference_grads(data, mask, mode, trans_A, trans_B, biased, block)
    ix = ctx.sparse_ports[port][0].indexes

    inp = {'A': data['A'].cuda(), 'B': data['B'].cuda()}
    g_out = grad_C.cuda()
    if compressed:
        if port in 'AB':
            inp[port] = ix.convert(inp[port])
        else:
            g_out = ix.convert(g_out)
    for t in inp.values():
        t.requires_grad_()
    args = [inp['A'], inp['B']]
    if biased:
        b = data['bias'].cuda().requires_grad_()
        args.append(b)
    out = SparseBatchMatMulFunc.apply(ctx, *args)
    out.backward(g_out)

    def dense(t, name):
        return ix.inverse(t) if (compressed and name == port) else t

    torch.testing.assert_close(dense(out.detach(), 'C').cpu(), C, **TOL[torch.float32])
    # gradients of the sparse tensor are defined on the covered blocks only and read 0 elsewhere
    torch.testing.assert_close(dense(inp['A'].grad, 'A').cpu(), gA, **TOL[torch.float32])
    torch.testing.assert_close(dense(inp['B'].grad, 'B').cpu(), gB, **TOL[torch.float32])
    if biased:
        torch.testing.assert_close(b.grad.cpu(), gbias, **TOL[torch.float32])


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('compressed', [False, True])
def test_sparse_matmul_operator_dynamic(mode, compressed):
    batch, M, K, N = 4, 128, 256, 192
    port = SPARSE_PORT[mode]
    data, mask = make_case(batch, M, K, N, mode=mode, trans_B=True)
    op = SparseBatchMatMul(**{f'{port}_mask': mask.cuda()}, transpose_A=False, transpose_B=True,
                           compressed=compressed)
    op.build(config={n: params() for n in op.get_kernel_placeholders(backward=True)},
             sample_inputs=[data['A'].cuda(), data['B'].cuda()])
    block = block_of(mode, 32, 32, 32, False, True)
    for seed in range(3):  # dynamic sparsity: new data and a new mask each round
        ix = op.get_sparse_indexes(port)
        expect = oracle.matmul_reference(data['A'], data['B'], None, mask, mode, False, True, block)
        inp = [data['A'].cuda(), data['B'].cuda()]
        if compressed and port in 'AB':
            i = 'AB'.index(port)
            inp[i] = ix.convert(inp[i])
        out = op(*inp)
        if compressed and port == 'C':
            out = ix.inverse(out)
        torch.testing.assert_close(out.cpu(), expect, **TOL[torch.float32])
        data, mask = make_case(batch, M, K, N, mode=mode, trans_B=True, seed=seed)
        op.update_mask(**{f'{port}_mask': mask.cuda()})


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('biased', [False, True])
def test_sparse_linear_operator(mode, biased):
    batch, in_dims, out_dims = 128, 256, 192
    port = SPARSE_PORT[mode]
    mask_name = {'sdd': 'input_mask', 'dsd': 'weight_mask', 'dds': 'output_mask'}[mode]
    data, mask = make_case(-1, batch, in_dims, out_dims, mode=mode, trans_B=True, biased=biased)
    dense = torch.nn.Linear(in_dims, out_dims, bias=biased, device='cuda')
    state = {'weight': data['B'].cuda()}
    if biased:
        state['bias'] = data['bias'].cuda()
    dense.load_state_dict(state)
    op = SparseLinear(dense, **{mask_name: mask.cuda()})
    op.build(config={n: params() for n in op.get_kernel_placeholders(backward=True)},
             sample_inputs=[data['A'].cuda()])
    block = block_of(mode, 32, 32, 32, False, True)
    for seed in range(3):
        b3 = {k: v.unsqueeze(0) for k, v in data.items()}
        C, gA, gB, gbias, grad_C = reference_grads(b3, mask, mode, False, True, biased, block)
        x = data['A'].cuda().requires_grad_()
        y = op(x)
        y.backward(grad_C[0].cuda())
        torch.testing.assert_close(y.detach().cpu(), C[0], **TOL[torch.float32])
        cover = torch.from_numpy(oracle.block_cover_mask(mask.numpy(), *block)).float()
        gx = x.grad.cpu() * (cover if port == 'A' else 1)
        torch.testing.assert_close(gx, gA[0], **TOL[torch.float32])
        gw = op.weight.grad
        if mode == 'dsd':
            gw = op.get_sparse_indexes('B').inverse(gw)
        torch.testing.assert_close(gw.reshape(out_dims, in_dims).cpu(), gB[0], **TOL[torch.float32])
        if biased:
            torch.testing.assert_close(op.bias.grad.cpu(), gbias[0], **TOL[torch.float32])
        data, mask = make_case(-1, batch, in_dims, out_dims, mode=mode, trans_B=True, biased=biased, seed=seed)
        if biased:
            op.bias = torch.nn.Parameter(data['bias'].cuda())
        op._raw_weight = data['B'].cuda()
        op.update_mask(**{mask_name: mask.cuda()})


def test_readme_workload_fp32_8x8_blocks():
    """x[1024,1024] W[1024,1024] (8x8-block mask, 90 % sparse) b[1024] uniform[0,1): y = x W^T + b with
    8x8 BCSR blocks."""
    g = torch.Generator().manual_seed(2022)
    x = torch.rand((1024, 1024), generator=g)
    w = torch.rand((1024, 1024), generator=g)
    b = torch.rand((1024,), generator=g)
    mask = oracle.block_mask((1024, 1024), (8, 8), 0.9, generator=g)
    w = w * mask
    dense = torch.nn.Linear(1024, 1024, device='cuda')
    dense.load_state_dict({'weight': w.cuda(), 'bias': b.cuda()})
    op = SparseLinear(dense, weight_mask=mask.cuda())
    cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 64, 'BLOCK_SIZE_K_VALUE': 8, 'BLOCK_SIZE_N_VALUE': 8}
    op.build({'forward:C': cfg}, sample_inputs=[x.cuda()])
    assert op.get_sparse_indexes('B').block_H == 8
    expect = torch.nn.functional.linear(x, w, b)
    torch.testing.assert_close(op(x.cuda()).cpu(), expect, rtol=1e-4, atol=1e-4)


def test_per_batch_masks_dds():
    """One fresh mask per batch element, indexes rebuilt on the GPU inside every forward."""
    batch, M, K, N, blk = 4, 256, 128, 256, 32
    g = torch.Generator().manual_seed(3)
    A = torch.randn((batch, M, K), generator=g).half()
    B = torch.randn((batch, K, N), generator=g).half()
    masks = torch.stack([oracle.block_mask((M, N), (blk, blk), 0.8, generator=g) for _ in range(batch)]).cuda()
    op = SparseBatchMatMul(C_mask=masks, compressed=True)
    cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': blk, 'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': blk}
    op.build({'forward:C': cfg}, sample_inputs=[A.cuda(), B.cuda()])
    op.set_dynamic(True)
    for round_ in range(2):
        out = op(A.cuda(), B.cuda())
        ix = op.get_sparse_indexes('C')
        dense = ix.inverse(out).float().cpu()
        full = torch.bmm(A.float(), B.float())
        torch.testing.assert_close(dense, full * masks.cpu().float(), **TOL[torch.float16])
        new = torch.stack([oracle.block_mask((M, N), (blk, blk), 0.8, generator=g) for _ in range(batch)])
        masks.copy_(new.cuda())  # rewritten in place: no update_mask call


@pytest.mark.parametrize('dtype', [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize('M,K,N,sparsity', [
    (128, 64, 32, 0.0),      # one row tile, one chunk, half a panel
    (192, 256, 160, 0.5),    # 64-row tiles (192 is no multiple of 128), five block rows: the last panel holds one
    (256, 1024, 320, 0.9),   # most chunks of a panel empty: they are neither fetched nor walked
    (384, 512, 256, 1.0),    # a single block left: every other panel is bias only
])
def test_dsd_32x32_blocks_on_the_fma_units(dtype, M, K, N, sparsity):
    """The register-tiled FMA kernel for 32 x 32 blocks (fp32 lives here; the 16-bit types reach it with _family='simt')."""
    batch = 2
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn((batch, M, K), generator=g).to(dtype)
    w = (torch.randn((batch, N, K), generator=g) * 0.1).to(dtype)
    b = torch.randn((batch, N), generator=g).to(dtype)
    mask = oracle.block_mask((N, K), (32, 32), sparsity, generator=g)
    if sparsity == 1.0:
        mask.zero_()
        mask[64:96, 128:160] = 1
    w = w * mask
    kernel = SparTASparseMatMulKernel(mode='dsd', biased=True, transpose_A=False, transpose_B=True, compressed=True)
    kernel.ports['B'].set_mask(mask.cuda())
    kernel.set_shape(batch, M, K, N)
    kernel.compile({'_impl': 'sparta', '_family': 'simt', 'BLOCK_SIZE_M_VALUE': 64, 'BLOCK_SIZE_K_VALUE': 32,
                    'BLOCK_SIZE_N_VALUE': 32})
    ix = kernel.ports['B'].indexes
    out = kernel(x.cuda(), ix.convert(w.cuda()), b.cuda())
    expect = oracle.matmul_reference(x.float(), w.float(), b.float(), mask, 'dsd', False, True, (32, 32))
    tol = TOL[dtype] if dtype != torch.float32 else dict(rtol=1e-4, atol=2e-4)  # sums over up to 1024 terms
    torch.testing.assert_close(out.float().cpu(), expect, **tol)
