"""GPU index build / value movement through the C-ABI against the CPU oracle: bit-exact.
Follows test/unit/test_tesa.py of the reference (block-size grid, BCSR / BCSC / BCSRC, convert,
inverse, sums) and adds the edge cases (empty, full, ragged widths, per-batch masks)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from sparta_b200.tesa import get_bcs_function

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')
SIZES = [4, 8, 16, 32, 64, 128]


def _mask(H=1024, W=768, sparsity=0.999, seed=2023, block=(1, 1)):
    g = torch.Generator().manual_seed(seed)
    return oracle.block_mask((H, W), block, sparsity, generator=g)


def _check_bcsr(ix, mask_np, BH, BW):
    row_ptr, idx, nnz = oracle.bcsr_from_mask(mask_np, BH, BW)
    assert ix.block_nnz == nnz and int(ix.nnz) == nnz
    np.testing.assert_array_equal(ix.row_ptr.cpu().numpy(), row_ptr)
    np.testing.assert_array_equal(ix.BCSR_idx.cpu().numpy(), idx)


def _check_bcsc(ix, mask_np, BH, BW, with_pos):
    col_ptr, idx, nnz = oracle.bcsc_from_mask(mask_np, BH, BW)
    assert ix.block_nnz == nnz
    np.testing.assert_array_equal(ix.col_ptr.cpu().numpy(), col_ptr)
    got = ix.BCSC_idx.cpu().numpy()
    if with_pos:
        exp = oracle.bcsrc_from_mask(mask_np, BH, BW)[3]
        assert got.dtype == np.int64
        np.testing.assert_array_equal(got, exp)
    else:
        assert got.dtype == np.int32
        np.testing.assert_array_equal(got, idx)


@pytest.mark.parametrize('BH', SIZES)
@pytest.mark.parametrize('BW', SIZES)
def test_bcsr(BH, BW):
    mask = _mask()
    ix = get_bcs_function(BH, BW, True, False).build_indexes(mask.cuda())
    _check_bcsr(ix, mask.numpy(), BH, BW)
    occ = torch.from_numpy(oracle.block_occupancy(mask.numpy(), BH, BW)).to(torch.uint8)
    torch.testing.assert_close(ix.get_block_mask().cpu(), occ)
    g = torch.Generator().manual_seed(1)
    dense = torch.rand((2, 1024, 768), generator=g) * mask
    vals = ix.convert(dense.cuda())
    np.testing.assert_array_equal(vals.cpu().numpy(),
                                  oracle.bcs_convert(dense.numpy(), ix.BCSR_idx.cpu().numpy(), BH, BW))
    torch.testing.assert_close(ix.inverse(vals).cpu(), dense, rtol=0, atol=0)
    torch.testing.assert_close(ix.sum(vals, axis=-1).cpu(), dense.sum(-1))
    torch.testing.assert_close(ix.sum(vals, axis=-2).cpu(), dense.sum(-2))


@pytest.mark.parametrize('BH', SIZES)
@pytest.mark.parametrize('BW', SIZES)
def test_bcsc(BH, BW):
    mask = _mask()
    ix = get_bcs_function(BH, BW, False, True).build_indexes(mask.cuda())
    _check_bcsc(ix, mask.numpy(), BH, BW, False)
    g = torch.Generator().manual_seed(2)
    dense = torch.rand((2, 1024, 768), generator=g) * mask
    vals = ix.convert(dense.cuda())
    np.testing.assert_array_equal(vals.cpu().numpy(),
                                  oracle.bcs_convert(dense.numpy(), ix.BCSC_idx.cpu().numpy(), BH, BW, False))
    torch.testing.assert_close(ix.inverse(vals).cpu(), dense, rtol=0, atol=0)
    torch.testing.assert_close(ix.sum(vals, axis=-1).cpu(), dense.sum(-1))
    torch.testing.assert_close(ix.sum(vals, axis=-2).cpu(), dense.sum(-2))


@pytest.mark.parametrize('BH', SIZES)
@pytest.mark.parametrize('BW', SIZES)
def test_bcsrc(BH, BW):
    mask = _mask()
    ix = get_bcs_function(BH, BW, True, True).build_indexes(mask.cuda())
    _check_bcsr(ix, mask.numpy(), BH, BW)
    _check_bcsc(ix, mask.numpy(), BH, BW, True)
    # the cross-check of the reference: BCSR entry at the stored position names the same block
    bcsr = ix.BCSR_idx
    bcsc = ix.BCSC_idx
    pos = bcsc >> 32
    torch.testing.assert_close((bcsr >> 16)[pos], (bcsc & 0xffff).to(torch.int32))
    torch.testing.assert_close((bcsr & 0xffff)[pos], ((bcsc >> 16) & 0xffff).to(torch.int32))
    g = torch.Generator().manual_seed(3)
    dense = torch.rand((2, 1024, 768), generator=g) * mask
    vals = ix.convert(dense.cuda())
    torch.testing.assert_close(ix.inverse(vals).cpu(), dense, rtol=0, atol=0)
    torch.testing.assert_close(ix.sum(vals, axis=-1).cpu(), dense.sum(-1))
    torch.testing.assert_close(ix.sum(vals, axis=-2).cpu(), dense.sum(-2))


def test_golden_masks():
    g = np.load(os.path.join(GOLDEN, 'tesa.npz'))
    mask = torch.from_numpy(g['mask'])
    for BH in SIZES:
        for BW in SIZES:
            ix = get_bcs_function(BH, BW, True, False).build_indexes(mask.cuda())
            torch.testing.assert_close(ix.get_block_mask().cpu(),
                                       torch.from_numpy(g[f'occ_{BH}_{BW}'].astype(np.uint8)))


@pytest.mark.parametrize('kind', ['empty', 'full', 'one_last', 'one_first'])
def test_edge_masks(kind):
    H, W, BH, BW = 256, 512, 32, 64
    mask = torch.zeros((H, W), dtype=torch.uint8)
    if kind == 'full':
        mask[:] = 1
    elif kind == 'one_last':
        mask[-1, -1] = 7
    elif kind == 'one_first':
        mask[0, 0] = 255
    ix = get_bcs_function(BH, BW, True, True).build_indexes(mask.cuda())
    _check_bcsr(ix, mask.numpy(), BH, BW)
    _check_bcsc(ix, mask.numpy(), BH, BW, True)
    assert ix.block_uniform == (kind in ('empty', 'full'))
    dense = torch.arange(H * W, dtype=torch.float32).reshape(1, H, W)
    vals = ix.convert(dense.cuda())
    assert vals.shape == (1, ix.block_nnz * BH * BW)
    cover = torch.from_numpy(oracle.block_cover_mask(mask.numpy(), BH, BW))
    torch.testing.assert_close(ix.inverse(vals).cpu(), dense * cover, rtol=0, atol=0)


@pytest.mark.parametrize('H,W,BH,BW', [(64, 72, 8, 8), (128, 100, 32, 4), (40, 24, 8, 4), (512, 1040, 256, 16),
                                       (256, 4096, 4, 256), (2048, 2048, 4, 4)])
def test_ragged_and_extreme_shapes(H, W, BH, BW):
    mask = _mask(H, W, 0.97, seed=5)
    ix = get_bcs_function(BH, BW, True, True).build_indexes(mask.cuda())
    _check_bcsr(ix, mask.numpy(), BH, BW)
    _check_bcsc(ix, mask.numpy(), BH, BW, True)


def test_per_batch_masks_and_repeat_calls():
    n, H, W, B = 5, 512, 384, 32
    fn = get_bcs_function(B, B, True, False)
    for seed in range(3):  # the workspace (tickets) must be reusable call after call
        masks = torch.stack([_mask(H, W, 0.9, seed=seed * 10 + i, block=(B, B)) for i in range(n)])
        ix = fn.build_indexes(masks.cuda())
        assert ix.batched and ix.n_masks == n
        nnz = ix.nnz_dev.cpu().numpy()
        for i in range(n):
            row_ptr, idx, cnt = oracle.bcsr_from_mask(masks[i].numpy(), B, B)
            assert nnz[i] == cnt
            np.testing.assert_array_equal(ix.row_ptr[i].cpu().numpy(), row_ptr)
            np.testing.assert_array_equal(ix.bcsr_buf[i, :cnt].cpu().numpy(), idx)
        assert ix.block_uniform


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.uint8])
def test_convert_other_dtypes(dtype):
    mask = _mask(256, 384, 0.9, seed=9, block=(8, 8))
    ix = get_bcs_function(32, 32, True, False).build_indexes(mask.cuda())
    g = torch.Generator().manual_seed(4)
    dense = (torch.rand((3, 256, 384), generator=g) * 100).to(dtype)
    vals = ix.convert(dense.cuda())
    exp = oracle.bcs_convert(dense.view(torch.uint8 if dtype == torch.uint8 else torch.int16).numpy(),
                             ix.BCSR_idx.cpu().numpy(), 32, 32)
    got = vals.cpu().view(torch.uint8 if dtype == torch.uint8 else torch.int16).numpy()
    np.testing.assert_array_equal(got, exp)
    assert not ix.block_uniform  # 8x8 granularity inside 32x32 blocks


def test_size_independent_properties_at_benchmark_size():
    """32 masks of 2048 x 2048 (the dynamic-sparsity configuration): count conservation, sortedness,
    idempotence -- no oracle pass over the 134 MB input."""
    g = torch.Generator(device='cuda').manual_seed(0)
    coarse = (torch.rand((32, 64, 64), device='cuda', generator=g) > 0.9).to(torch.uint8)
    masks = coarse.repeat_interleave(32, 1).repeat_interleave(32, 2).contiguous()
    fn = get_bcs_function(32, 32, True, False)
    ix = fn.build_indexes(masks)
    nnz = ix.nnz_dev
    torch.testing.assert_close(nnz.to(torch.int64), coarse.sum((1, 2)).to(torch.int64))
    torch.testing.assert_close(ix.row_ptr[:, -1], nnz)
    for b in (0, 17, 31):
        cnt = int(nnz[b])
        idx = ix.bcsr_buf[b, :cnt].to(torch.int64)
        assert torch.all(idx[1:] > idx[:-1])  # packed (row << 16 | col) strictly ascending
        rebuilt = torch.zeros((64, 64), dtype=torch.uint8, device='cuda')
        rebuilt[idx >> 16, idx & 0xffff] = 1
        torch.testing.assert_close(rebuilt, coarse[b])
    ix2 = fn.build_indexes(masks)
    torch.testing.assert_close(ix2.bcsr_buf[0, :int(nnz[0])], ix.bcsr_buf[0, :int(nnz[0])])
