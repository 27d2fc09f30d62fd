"""The CPU oracle against the golden vectors produced by the reference's own CPU code
(tests/golden/make_golden.py) and against its own invariants."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')


def test_block_mask_matches_reference_generator():
    g = np.load(os.path.join(GOLDEN, 'masks.npz'))
    for i in range(3):
        H, W, bh, bw, sp, seed = g[f'mask{i}_args'].tolist()
        gen = torch.Generator().manual_seed(seed)
        m = oracle.block_mask((H, W), (bh, bw), sp / 10000, generator=gen)
        np.testing.assert_array_equal(m.numpy(), g[f'mask{i}'])


@pytest.mark.parametrize('BH', [4, 8, 16, 32, 64, 128])
@pytest.mark.parametrize('BW', [4, 8, 16, 32, 64, 128])
def test_block_occupancy_matches_reduce_mask_ref(BH, BW):
    g = np.load(os.path.join(GOLDEN, 'tesa.npz'))
    occ = oracle.block_occupancy(g['mask'], BH, BW)
    np.testing.assert_array_equal(occ.astype(np.uint8), g[f'occ_{BH}_{BW}'].astype(np.uint8))


@pytest.mark.parametrize('BH,BW', [(4, 4), (8, 32), (32, 8), (64, 64), (128, 16)])
def test_index_forms_are_consistent(BH, BW):
    g = np.load(os.path.join(GOLDEN, 'tesa.npz'))
    mask = g['mask']
    occ = g[f'occ_{BH}_{BW}'].astype(bool)
    row_ptr, bcsr, col_ptr, bcsc64, nnz = oracle.bcsrc_from_mask(mask, BH, BW)
    assert nnz == occ.sum() == row_ptr[-1] == col_ptr[-1]
    # rebuild the block mask from each form (what test/unit/test_tesa.py:36-38 checks)
    rebuilt = np.zeros_like(occ)
    rebuilt[bcsr >> 16, bcsr & 0xffff] = True
    np.testing.assert_array_equal(rebuilt, occ)
    lo = (bcsc64 & 0xffffffff).astype(np.int64)
    rebuilt = np.zeros_like(occ)
    rebuilt[lo & 0xffff, lo >> 16] = True
    np.testing.assert_array_equal(rebuilt, occ)
    # cross-consistency of the BCSR position (test/unit/test_tesa.py:101-107)
    pos = bcsc64 >> 32
    np.testing.assert_array_equal(bcsr[pos] >> 16, lo & 0xffff)
    np.testing.assert_array_equal(bcsr[pos] & 0xffff, lo >> 16)
    # ascending columns inside each row, ascending rows inside each column
    for r in range(len(row_ptr) - 1):
        cols = bcsr[row_ptr[r]:row_ptr[r + 1]] & 0xffff
        assert np.all(np.diff(cols) > 0)
    # convert / inverse round trip (test/unit/test_tesa.py:41-43)
    rng = np.random.default_rng(0)
    dense = rng.random((2,) + mask.shape, dtype=np.float32) * mask
    vals = oracle.bcs_convert(dense, bcsr, BH, BW, True)
    assert vals.shape == (2, nnz * BH * BW)
    np.testing.assert_array_equal(oracle.bcs_inverse(vals, bcsr, *mask.shape, BH, BW, True), dense)
    _, bcsc32, _ = oracle.bcsc_from_mask(mask, BH, BW)
    vals_c = oracle.bcs_convert(dense, bcsc32, BH, BW, False)
    np.testing.assert_array_equal(oracle.bcs_inverse(vals_c, bcsc32, *mask.shape, BH, BW, False), dense)


def test_softmax_and_attention_match_reference_math():
    g = np.load(os.path.join(GOLDEN, 'softmax_attention.npz'))
    t = lambda k: torch.from_numpy(g[k])
    T = float(g['T'])
    y = oracle.softmax_forward_reference(t('x'), t('mask'), T)
    torch.testing.assert_close(y, t('y'), rtol=0, atol=0)
    dx = oracle.softmax_backward_reference(t('grad'), y, t('mask'), T)
    torch.testing.assert_close(dx, t('dx'), rtol=0, atol=0)
    o = oracle.attention_reference(t('q'), t('k'), t('v'), t('amask'))
    torch.testing.assert_close(o, t('o'), rtol=1e-6, atol=1e-6)
    # fully masked rows give zeros
    assert torch.all(y[:, 40:48] == 0)


def test_package_reference_formulas_equal_oracle():
    """sparta_b200.testing mirrors sparta.testing; it must agree with the oracle bit for bit."""
    from sparta_b200.testing import (sparse_softmax_forward_reference, sparse_softmax_backward_reference,
                                     sparse_multi_head_attention_reference)
    g = np.load(os.path.join(GOLDEN, 'softmax_attention.npz'))
    t = lambda k: torch.from_numpy(g[k])
    T = float(g['T'])
    torch.testing.assert_close(sparse_softmax_forward_reference(t('x'), t('mask'), T), t('y'), rtol=0, atol=0)
    torch.testing.assert_close(sparse_softmax_backward_reference(t('grad'), t('y'), t('mask'), T), t('dx'),
                               rtol=0, atol=0)
    torch.testing.assert_close(sparse_multi_head_attention_reference(t('q'), t('k'), t('v'), t('amask')), t('o'),
                               rtol=1e-6, atol=1e-6)


def test_matmul_reference_dds_uses_block_coverage():
    gen = torch.Generator().manual_seed(1)
    A = torch.rand((2, 64, 32), generator=gen)
    B = torch.rand((2, 48, 32), generator=gen)
    mask = oracle.block_mask((64, 48), (8, 8), 0.7, generator=gen)
    C = oracle.matmul_reference(A, B, None, mask, 'dds', False, True, (32, 16))
    cover = torch.from_numpy(oracle.block_cover_mask(mask.numpy(), 32, 16)).bool()
    dense = torch.einsum('bmk,bnk->bmn', A, B)
    torch.testing.assert_close(C[:, cover], dense[:, cover])
    assert torch.all(C[:, ~cover] == 0)


def test_band_global_random_mask_density():
    m = oracle.band_global_random_mask(4096, 4096, 64, 8, 0.05, 0)
    occ = oracle.block_occupancy(m.numpy(), 64, 64)
    assert occ[0].all() and occ[:, 0].all()
    assert 1150 < occ.sum() < 1400  # ~1286 of 4096 blocks


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('trans_A', [False, True])
@pytest.mark.parametrize('trans_B', [False, True])
def test_matmul_reference_matches_the_reference_method(mode, trans_A, trans_B):
    """``oracle.matmul_reference`` against vectors produced by ``SparseMatMulKernel.reference`` itself
    (extracted from the reference's class by tests/golden/make_golden.py).  Before ``compile`` the reference
    multiplies a dds output by the element mask -- a block coverage with 1 x 1 blocks -- and after it by the
    coverage of the kernel's BM x BN blocks."""
    g = np.load(os.path.join(GOLDEN, 'matmul.npz'))
    batch, M, K, N, BM, BN = g['shape'].tolist()
    key = f'{mode}_{int(trans_A)}{int(trans_B)}'
    A, B, bias, mask = (torch.from_numpy(g[f'{key}_{n}']) for n in ('A', 'B', 'bias', 'mask'))
    for biased in (False, True):
        for ready, block in ((False, (1, 1)), (True, (BM, BN))):
            got = oracle.matmul_reference(A, B, bias if biased else None, mask, mode, trans_A, trans_B, block)
            want = torch.from_numpy(g[f'{key}_C_b{int(biased)}_r{int(ready)}'])
            torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-6)
