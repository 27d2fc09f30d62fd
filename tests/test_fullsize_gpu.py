"""The benchmark configurations at FULL size against the CPU oracle (the other GPU tests use reduced
shapes): the fp16 SparseLinear of 4096 tokens x 4096 -> 4096 with a 32 x 32-block weight mask in its dsd
and dds forms, four heads of the B4 H16 S4096 D64 attention, one call of the dynamic-mask batched dds
(32 masks of 2048 x 2048: index arrays bit-exact), and two heads of the S8192 D128 bf16 attention.
Tolerances: 2e-2 for fp16 / bf16 results, bit-exact for index arrays and block counts."""
import numpy as np
import pytest
import torch

from oracle import oracle
from sparta_b200 import _lib
from sparta_b200.nn import SparseLinear, SparseBatchMatMul, SparseAttention
from sparta_b200.tesa import get_bcs_function

pytestmark = pytest.mark.gpu
TOL = dict(rtol=2e-2, atol=2e-2)


def _linear_case(sparsity):
    g = torch.Generator().manual_seed(2023)
    x = torch.randn((4096, 4096), generator=g).half()
    w = (torch.randn((4096, 4096), generator=g) * 0.02).half()
    b = torch.randn((4096,), generator=g).half()
    mask = oracle.block_mask((4096, 4096), (32, 32), sparsity, generator=g)
    return x, w * mask, b, mask


@pytest.mark.parametrize('sparsity', [0.75, 0.9, 0.95])
def test_sparse_linear_dsd_full_size(sparsity):
    x, w, b, mask = _linear_case(sparsity)
    dense = torch.nn.Linear(4096, 4096, device='cuda', dtype=torch.float16)
    dense.load_state_dict({'weight': w.cuda(), 'bias': b.cuda()})
    op = SparseLinear(dense, weight_mask=mask.cuda())
    op.build({'forward:C': {'_impl': 'sparta', '_family': 'tcgen05', 'BLOCK_SIZE_M_VALUE': 128,
                            'BLOCK_SIZE_K_VALUE': 32, 'BLOCK_SIZE_N_VALUE': 32}}, sample_inputs=[x.cuda()])
    row_ptr, idx, nnz = oracle.bcsr_from_mask(mask.numpy(), 32, 32)
    ix = op.get_sparse_indexes('B')
    assert ix.block_nnz == nnz
    assert np.array_equal(ix.row_ptr.cpu().numpy(), row_ptr) and np.array_equal(ix.BCSR_idx.cpu().numpy(), idx)
    with torch.no_grad():
        y = op(x.cuda())
    assert _lib.last_status() == [0, 0, 0, 0]
    want = torch.nn.functional.linear(x.float(), w.float(), b.float())
    torch.testing.assert_close(y.float().cpu(), want, **TOL)


def test_sparse_linear_dds_full_size():
    x, w, b, mask = _linear_case(0.75)
    op = SparseBatchMatMul(C_mask=mask.cuda(), transpose_B=True, compressed=True)
    xd, wd = x.cuda().unsqueeze(0), (torch.randn((4096, 4096), generator=torch.Generator().manual_seed(5)) * 0.02).half().cuda().unsqueeze(0)
    op.build({'forward:C': {'_impl': 'sparta', '_family': 'tcgen05', 'BLOCK_SIZE_M_VALUE': 32,
                            'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 32}}, sample_inputs=[xd, wd])
    with torch.no_grad():
        out = op(xd, wd)
    assert _lib.last_status() == [0, 0, 0, 0]
    ix = op.get_sparse_indexes('C')
    want = oracle.matmul_reference(xd.float().cpu(), wd.float().cpu(), None, mask, 'dds', False, True, (32, 32))
    torch.testing.assert_close(ix.inverse(out).float().cpu(), want, **TOL)


def _attention_heads(heads, S, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn((heads, S, D), generator=g).to(dtype) for _ in range(3))
    mask = oracle.band_global_random_mask(S, S, 64, 8, 0.05, seed=0)
    op = SparseAttention(mask=mask.cuda())
    mm = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 64, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 64}
    sm = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': 64, 'BLOCK_SIZE_W_VALUE': 64, 'ROW_TILE_VALUE': 4}
    op.build({'qk/forward:C': mm, 'sm/forward:y': sm, 'out/forward:C': mm}, sample_inputs=[q.cuda(), k.cuda(), v.cuda()])
    assert op._use_fused
    with torch.no_grad():
        out = op(q.cuda(), k.cuda(), v.cuda())
    assert op.fused_status() == [0, 0, 0, 0]
    return out, (q, k, v), mask, op


def test_attention_s4096_d64_four_heads():
    out, (q, k, v), mask, op = _attention_heads(4, 4096, 64, torch.float16, 2024)
    assert op.get_sparse_indexes().block_nnz == 1286  # the block count of this generator and seed
    for h in range(4):  # one head at a time: 64 MB of dense fp32 scores each on the host
        want = oracle.attention_reference(q[h:h + 1].float(), k[h:h + 1].float(), v[h:h + 1].float(), mask)
        torch.testing.assert_close(out[h:h + 1].float().cpu(), want, **TOL)


def test_attention_s8192_d128_bf16_two_heads():
    out, (q, k, v), mask, op = _attention_heads(2, 8192, 128, torch.bfloat16, 2025)
    assert op.get_sparse_indexes().block_nnz == 3082
    for h in range(2):
        want = oracle.attention_reference(q[h:h + 1].float(), k[h:h + 1].float(), v[h:h + 1].float(), mask)
        torch.testing.assert_close(out[h:h + 1].float().cpu(), want, **TOL)


def test_dynamic_masks_32x2048x2048_indexes_bit_exact():
    """The dynamic-sparsity configuration: 32 fresh masks of 2048 x 2048 per call (134 MB), 32 x 32 blocks at
    90 %; every mask's row_ptr, BCSR entries and block count against the oracle, then the dds product."""
    g = torch.Generator().manual_seed(99)
    coarse = (torch.rand((32, 64, 64), generator=g) > 0.9).to(torch.uint8)
    masks = coarse.repeat_interleave(32, 1).repeat_interleave(32, 2).contiguous()
    ix = get_bcs_function(32, 32, True, False).build_indexes(masks.cuda(), 1024)
    nnz_dev = ix.nnz_dev.cpu().numpy()
    for m in range(32):
        row_ptr, idx, nnz = oracle.bcsr_from_mask(masks[m].numpy(), 32, 32)
        assert nnz_dev[m] == nnz
        assert np.array_equal(ix.row_ptr[m].cpu().numpy(), row_ptr)
        assert np.array_equal(ix.bcsr_buf[m, :nnz].cpu().numpy(), idx)
    A = torch.randn((32, 2048, 128), generator=g).half()
    B = torch.randn((32, 128, 2048), generator=g).half()
    op = SparseBatchMatMul(C_mask=masks.cuda(), compressed=True, capacity=1024)
    op.build({'forward:C': {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 64,
                            'BLOCK_SIZE_N_VALUE': 32}}, sample_inputs=[A.cuda(), B.cuda()])
    op.set_dynamic(True)
    with torch.no_grad():
        out = op(A.cuda(), B.cuda())
    assert _lib.last_status() == [0, 0, 0, 0]
    dense = op.get_sparse_indexes('C').inverse(out).float().cpu()
    for m in (0, 13, 31):
        want = (A[m].float() @ B[m].float()) * masks[m]
        torch.testing.assert_close(dense[m], want, **TOL)
