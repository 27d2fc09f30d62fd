"""CPU oracle for the block-sparse operator path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import this module; the
product path (``sparta_b200``) never does and raises when its CUDA library is missing.

Every function restates, with numpy / CPU torch, what the reference (microsoft/SparTA) computes or
what its own unit tests compare against; the reference location is cited per function (paths relative
to the reference project root).  Parity pins: ``tests/golden/*.npz`` were produced by importing the
reference's CPU-capable modules (``sparta/testing/math.py``, ``sparta/testing/mask.py``) and the
``reduce_mask_ref`` helper of ``test/unit/test_tesa.py`` by file path; ``tests/test_oracle.py``
checks this module against those vectors.
"""
from typing import Optional, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------------------------
# masks
# --------------------------------------------------------------------------------------------

def block_mask(shape: Tuple[int, int], block: Tuple[int, int] = (1, 1), sparsity: float = 0.99,
               generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """uint8 mask whose ``block``-sized tiles are kept with probability ``1 - sparsity``.

    Follows ``random_block_mask`` / ``random_mask`` (sparta/testing/mask.py:34-60): draw
    ``rand(shape / block) > sparsity`` and tile it; here on the CPU with an explicit generator.
    """
    assert shape[0] % block[0] == 0 and shape[1] % block[1] == 0
    rows, cols = shape[0] // block[0], shape[1] // block[1]
    coarse = (torch.rand((rows, cols), generator=generator) > sparsity).to(torch.uint8)
    return coarse.repeat_interleave(block[0], 0).repeat_interleave(block[1], 1).contiguous()


def band_global_random_mask(n_tgt: int, n_src: int, block: int = 64, band: int = 8,
                            extra: float = 0.05, seed: int = 0) -> torch.Tensor:
    """Attention mask of the benchmark configurations: a band of ``band`` blocks either side of the
    diagonal, the first block row and block column, plus ``extra`` additional random blocks."""
    rows, cols = n_tgt // block, n_src // block
    i = torch.arange(rows).unsqueeze(1)
    j = torch.arange(cols).unsqueeze(0)
    keep = (i - j).abs() <= band
    keep |= (i == 0) | (j == 0)
    g = torch.Generator().manual_seed(seed)
    keep |= torch.rand((rows, cols), generator=g) < extra
    coarse = keep.to(torch.uint8)
    return coarse.repeat_interleave(block, 0).repeat_interleave(block, 1).contiguous()


# --------------------------------------------------------------------------------------------
# block-compressed indexes
# --------------------------------------------------------------------------------------------

def block_occupancy(mask, BH: int, BW: int) -> np.ndarray:
    """bool [H/BH, W/BW]: which blocks hold any non-zero (``reduce_mask_ref``,
    test/unit/test_tesa.py:11-17; the kernel-side rule is block_compressed.cu.j2:100-111)."""
    m = np.asarray(mask)
    H, W = m.shape
    return (m.reshape(H // BH, BH, W // BW, BW) != 0).any(axis=(1, 3))


def bcsr_from_mask(mask, BH: int, BW: int):
    """Canonical BCSR: (row_ptr int32[R+1], idx int32[nnz] = (row << 16) | col, nnz).

    ``row_ptr`` and ``nnz`` equal what ``_build_BCSR_indexes`` returns
    (sparta/tesa/block_compressed.py:267-287); the reference's idx order inside a row depends on
    atomics (block_compressed.cu.j2:112-116), the canonical form is ascending column.
    """
    occ = block_occupancy(mask, BH, BW)
    rows, cols = np.nonzero(occ)  # row-major order = ascending column inside each row
    row_ptr = np.zeros(occ.shape[0] + 1, dtype=np.int32)
    row_ptr[1:] = np.cumsum(occ.sum(axis=1))
    idx = ((rows.astype(np.int64) << 16) | cols).astype(np.int32)
    return row_ptr, idx, int(idx.size)


def bcsc_from_mask(mask, BH: int, BW: int):
    """Canonical BCSC: (col_ptr int32[C+1], idx int32[nnz] = (col << 16) | row, nnz)
    (sparta/tesa/block_compressed.py:289-309, block_compressed.cu.j2:166)."""
    occ = block_occupancy(mask, BH, BW)
    cols, rows = np.nonzero(occ.T)
    col_ptr = np.zeros(occ.shape[1] + 1, dtype=np.int32)
    col_ptr[1:] = np.cumsum(occ.sum(axis=0))
    idx = ((cols.astype(np.int64) << 16) | rows).astype(np.int32)
    return col_ptr, idx, int(idx.size)


def bcsrc_from_mask(mask, BH: int, BW: int):
    """Both formats; the BCSC entries are int64 with the BCSR position of the block in the upper
    32 bits (sparta/tesa/block_compressed.py:242-265, block_compressed.cu.j2:163-164)."""
    row_ptr, bcsr_idx, nnz = bcsr_from_mask(mask, BH, BW)
    col_ptr, bcsc_idx, _ = bcsc_from_mask(mask, BH, BW)
    occ = block_occupancy(mask, BH, BW)
    pos = np.full(occ.shape, -1, dtype=np.int64)
    pos[occ] = np.arange(nnz)
    c = bcsc_idx.astype(np.int64) >> 16
    r = bcsc_idx.astype(np.int64) & 0xffff
    bcsc64 = (pos[r, c] << 32) | bcsc_idx.astype(np.int64)
    return row_ptr, bcsr_idx, col_ptr, bcsc64, nnz


def block_cover_mask(mask, BH: int, BW: int) -> np.ndarray:
    """uint8 [H, W]: 1 wherever the enclosing block is kept (``BCSIndexes.get_mask``,
    sparta/tesa/block_compressed.py:47-50)."""
    occ = block_occupancy(mask, BH, BW).astype(np.uint8)
    return np.repeat(np.repeat(occ, BH, axis=0), BW, axis=1)


def _unpack(idx, bcsr: bool):
    v = np.asarray(idx).astype(np.int64) & 0xffffffff
    hi, lo = v >> 16, v & 0xffff
    return (hi, lo) if bcsr else (lo, hi)  # (block_row, block_col)


def bcs_convert(dense, idx, BH: int, BW: int, bcsr: bool = True) -> np.ndarray:
    """dense [..., H, W] -> compressed [..., nnz*BH*BW], blocks in index order, row-major inside a
    block in the stored orientation (``dense_to_bcs_val``, block_compressed.cu.j2:172-195)."""
    d = np.asarray(dense)
    lead = d.shape[:-2]
    H, W = d.shape[-2:]
    br, bc = _unpack(idx, bcsr)
    blocks = d.reshape(-1, H // BH, BH, W // BW, BW).transpose(0, 1, 3, 2, 4)  # [b, R, C, BH, BW]
    return blocks[:, br, bc].reshape(*lead, -1)


def bcs_inverse(vals, idx, H: int, W: int, BH: int, BW: int, bcsr: bool = True) -> np.ndarray:
    """compressed -> zero-filled dense (``bcs_val_to_dense``, block_compressed.cu.j2:197-220)."""
    v = np.asarray(vals)
    lead = v.shape[:-1]
    br, bc = _unpack(idx, bcsr)
    v = v.reshape(-1, br.size, BH, BW)
    out = np.zeros((v.shape[0], H // BH, W // BW, BH, BW), dtype=v.dtype)
    out[:, br, bc] = v
    return out.transpose(0, 1, 3, 2, 4).reshape(*lead, H, W)


# --------------------------------------------------------------------------------------------
# operators (CPU torch, fp32 unless the caller passes something else)
# --------------------------------------------------------------------------------------------

def matmul_reference(A: torch.Tensor, B: torch.Tensor, bias: Optional[torch.Tensor], mask: torch.Tensor,
                     mode: str, trans_A: bool, trans_B: bool, block: Tuple[int, int]) -> torch.Tensor:
    """Masked-dense batched matmul, the oracle of the matmul kernels
    (``SparseMatMulKernel.reference``, sparta/specializer/kernels/matmul.py:211-227).

    ``mask`` applies to A (sdd), B (dsd) in their stored orientation; for dds the output is multiplied
    by the block-coverage mask of ``block`` = (BM, BN) -- not the element mask (matmul.py:222-226).
    """
    if mode == 'sdd':
        A = A * mask
    elif mode == 'dsd':
        B = B * mask
    a = 'bkm' if trans_A else 'bmk'
    b = 'bnk' if trans_B else 'bkn'
    C = torch.einsum(f'{a}, {b} -> bmn', A, B)
    if bias is not None:
        C = C + bias.unsqueeze(1)
    if mode == 'dds':
        C = C * torch.from_numpy(block_cover_mask(mask.numpy(), *block)).to(C.dtype)
    return C


def softmax_forward_reference(x: torch.Tensor, mask: torch.Tensor, temperature: float = 1.) -> torch.Tensor:
    """Masked softmax; fully masked rows give 0 (``sparse_softmax_forward_reference``,
    sparta/testing/math.py:8-27): exp((x - rowmax) / T) * mask / (sum + 1e-10)."""
    c_max = x.max(dim=-1, keepdim=True).values
    c_exp = torch.exp((x - c_max) / temperature) * mask
    return c_exp / (c_exp.sum(dim=-1, keepdim=True) + 1e-10)


def softmax_backward_reference(grad: torch.Tensor, output: torch.Tensor, mask: torch.Tensor,
                               temperature: float = 1.) -> torch.Tensor:
    """(``sparse_softmax_backward_reference``, sparta/testing/math.py:30-50)."""
    y = output * mask
    prod = grad * y
    return (prod - y * prod.sum(dim=-1, keepdim=True)) / temperature


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor,
                        temperature: Optional[float] = None) -> torch.Tensor:
    """softmax_mask(q k^T / T) v with T = sqrt(E) by default
    (``sparse_multi_head_attention_reference``, sparta/testing/math.py:53-79)."""
    if temperature is None:
        temperature = float(np.sqrt(q.shape[-1]))
    qk = torch.einsum('...mk,...nk->...mn', q, k)
    return torch.einsum('...mn,...nk->...mk', softmax_forward_reference(qk, mask, temperature), v)
