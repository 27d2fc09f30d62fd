"""Block-compressed (BCSR / BCSC / BCSRC) indexes built on the GPU in one launch.

Host-side mirror of ``sparta/tesa/block_compressed.py``: same class and attribute names
(``row_ptr``, ``BCSR_idx``, ``col_ptr``, ``BCSC_idx``, ``block_nnz``, ``nnz``, ``get_block_mask``,
``get_mask``, ``convert``, ``inverse``, ``sum``), but the index build is a single kernel
(``sparta_bcs_build``) with no ``cumsum`` and no host synchronisation: ``block_nnz`` is fetched from
the device lazily, the first time host code asks for it.  Entries inside a block row (column) are in
ascending column (row) order, where the reference's order depends on atomics.

Extension: ``build_indexes`` also accepts a 3-D mask ``[n, H, W]`` (one mask per batch element); the
index arrays then carry a leading dimension and compressed tensors use ``capacity`` blocks per
batch element.
"""
from __future__ import annotations

import abc
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from sparta_b200 import _lib
from sparta_b200.tesa.tesa_base import TeSAIndexes, TeSAFunctionContext

_VALID_BLOCK = (4, 8, 16, 32, 64, 128, 256)
_ELEM_BYTES = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.uint8: 1, torch.int8: 1,
               torch.bool: 1}

# zero-filled scratch of the index build, cached per (device, stream, size) like the reference's
# _extra_buffer_cache (sparta/tesa/block_compressed.py:199,231-240); calls sharing an entry must not
# overlap on the GPU
_workspace_cache: Dict[Tuple, torch.Tensor] = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, nbytes)
    ws = _workspace_cache.get(key)
    if ws is None:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _workspace_cache[key] = ws
    return ws


class BCSIndexes(TeSAIndexes):
    """Common part of the three index forms (sparta/tesa/block_compressed.py:23-76)."""

    BCSR = False
    BCSC = False

    def __init__(self, function_context: 'BCSFunctionContext', raw_mask: torch.Tensor,
                 block_H: int, block_W: int, capacity: int, nnz_dev: torch.Tensor,
                 uniform_dev: torch.Tensor):
        super().__init__(function_context, raw_mask)
        self.block_H = block_H
        self.block_W = block_W
        self.H, self.W = raw_mask.shape[-2:]
        self.row_num = self.H // block_H
        self.col_num = self.W // block_W
        self.n_masks = raw_mask.shape[0] if raw_mask.dim() == 3 else 1
        self.batched = raw_mask.dim() == 3
        self.capacity = capacity
        self.nnz_dev = nnz_dev            # int32 [n_masks] on the device, read by every kernel
        self.uniform_dev = uniform_dev    # int32 [n_masks]: 1 when kept blocks have no zero element
        self._block_nnz: Optional[int] = None
        self._uniform: Optional[bool] = None

    # -- host views of device-side counts (one synchronisation, on first use) --
    def _fetch(self):
        host = torch.stack([self.nnz_dev, self.uniform_dev]).cpu()
        self._nnz_host = host[0].tolist()
        if max(self._nnz_host) > self.capacity:
            raise RuntimeError(f'mask keeps {max(self._nnz_host)} blocks but the index arrays were built with '
                               f'capacity {self.capacity}: rebuild with a larger capacity')
        self._block_nnz = int(max(self._nnz_host)) if self.batched else int(self._nnz_host[0])
        self._uniform = bool(host[1].min().item())

    @property
    def block_nnz(self) -> int:
        """Kept blocks (largest count over the masks when batched)."""
        if self._block_nnz is None:
            self._fetch()
        return self._block_nnz

    @property
    def nnz(self) -> np.int32:
        return np.int32(self.block_nnz)

    @property
    def block_uniform(self) -> bool:
        """True when every kept block is fully non-zero: element masking equals block masking."""
        if self._uniform is None:
            self._fetch()
        return self._uniform

    @property
    def val_stride_blocks(self) -> int:
        """Blocks per batch element in compressed tensors built with these indexes."""
        return self.capacity if self.batched else self.block_nnz

    @abc.abstractmethod
    def get_block_mask(self) -> torch.Tensor:
        """Rebuild the [row_num, col_num] block mask from the index arrays."""

    def get_mask(self) -> torch.Tensor:
        """Element mask covering every kept block (sparta/tesa/block_compressed.py:47-50)."""
        bm = self.get_block_mask()
        return bm.repeat_interleave(self.block_H, -2).repeat_interleave(self.block_W, -1).contiguous()

    def _order_idx(self) -> Tuple[torch.Tensor, bool, bool]:
        """(index buffer, is_bcsr, is_64bit) that defines the order of compressed values."""
        raise NotImplementedError

    def convert(self, dense: torch.Tensor) -> torch.Tensor:
        idx, is_bcsr, is64 = self._order_idx()
        return self.function_context.convert(dense, self, idx, is_bcsr, is64)

    def inverse(self, sparse_val: torch.Tensor) -> torch.Tensor:
        idx, is_bcsr, is64 = self._order_idx()
        return self.function_context.inverse(sparse_val, self, idx, is_bcsr, is64)

    def _row_sum(self, sparse_val: torch.Tensor) -> torch.Tensor:
        return self.inverse(sparse_val).sum(-1)

    def _col_sum(self, sparse_val: torch.Tensor) -> torch.Tensor:
        return self.inverse(sparse_val).sum(-2)

    def sum(self, sparse_val: torch.Tensor, axis: int = -1) -> torch.Tensor:
        inverse_axis = -axis if axis < 0 else len(sparse_val.shape) - axis
        if inverse_axis == 1:
            return self._row_sum(sparse_val)
        elif inverse_axis == 2:
            return self._col_sum(sparse_val)
        raise ValueError(f'axis #{axis} is not sparsed, please use torch.sum() instead.')

    def _dense_block_mask(self, idx: torch.Tensor, row_major: bool) -> torch.Tensor:
        if self.batched:
            raise NotImplementedError('get_block_mask() is defined for a single 2-D mask')
        v = idx[:self.block_nnz].to(torch.int64) & 0xffffffff
        hi, lo = v >> 16, v & 0xffff
        r, c = (hi, lo) if row_major else (lo, hi)
        out = torch.zeros((self.row_num, self.col_num), dtype=torch.uint8, device=idx.device)
        out[r, c] = 1
        return out


class BCSRIndexes(BCSIndexes):
    """(sparta/tesa/block_compressed.py:79-124)"""

    BCSR = True

    def __init__(self, function_context, raw_mask, row_ptr, bcsr_buf, block_H, block_W, capacity,
                 nnz_dev, uniform_dev):
        super().__init__(function_context, raw_mask, block_H, block_W, capacity, nnz_dev, uniform_dev)
        self.row_ptr = row_ptr
        self.bcsr_buf = bcsr_buf  # capacity-sized; BCSR_idx is its valid prefix

    @property
    def BCSR_idx(self) -> torch.Tensor:
        return self.bcsr_buf if self.batched else self.bcsr_buf[:self.block_nnz]

    def get_block_mask(self):
        return self._dense_block_mask(self.bcsr_buf, True)

    def _order_idx(self):
        return self.bcsr_buf, True, False

    def _row_sum(self, sparse_val: torch.Tensor):
        return self.function_context.row_sum(sparse_val, self)


class BCSCIndexes(BCSIndexes):
    """(sparta/tesa/block_compressed.py:127-168)"""

    BCSC = True

    def __init__(self, function_context, raw_mask, col_ptr, bcsc_buf, block_H, block_W, capacity,
                 nnz_dev, uniform_dev):
        super().__init__(function_context, raw_mask, block_H, block_W, capacity, nnz_dev, uniform_dev)
        self.col_ptr = col_ptr
        self.bcsc_buf = bcsc_buf

    @property
    def BCSC_idx(self) -> torch.Tensor:
        return self.bcsc_buf if self.batched else self.bcsc_buf[:self.block_nnz]

    def get_block_mask(self):
        return self._dense_block_mask(self.bcsc_buf, False)

    def _order_idx(self):
        return self.bcsc_buf, False, False


class BCSRCIndexes(BCSRIndexes):
    """Both forms; values live in BCSR order and ``BCSC_idx`` is int64 with that position in its
    upper half (sparta/tesa/block_compressed.py:171-196)."""

    BCSC = True

    def __init__(self, function_context, raw_mask, row_ptr, col_ptr, bcsr_buf, bcsc_buf, block_H,
                 block_W, capacity, nnz_dev, uniform_dev):
        super().__init__(function_context, raw_mask, row_ptr, bcsr_buf, block_H, block_W, capacity,
                         nnz_dev, uniform_dev)
        self.col_ptr = col_ptr
        self.bcsc_buf = bcsc_buf

    @property
    def BCSC_idx(self) -> torch.Tensor:
        return self.bcsc_buf if self.batched else self.bcsc_buf[:self.block_nnz]

    def _col_sum(self, sparse_val: torch.Tensor):
        return self.function_context.col_sum(sparse_val, self)


class BCSFunctionContext(TeSAFunctionContext):
    """Index builder and value converters for one (block_H, block_W, BCSR, BCSC) combination
    (sparta/tesa/block_compressed.py:202-403).  Nothing is compiled here: the kernels are prebuilt."""

    def __init__(self, block_H: int, block_W: int, BCSR: bool, BCSC: bool):
        assert block_H in _VALID_BLOCK
        assert block_W in _VALID_BLOCK
        assert BCSR or BCSC
        self._block_H = block_H
        self._block_W = block_W
        self._block_size = block_H * block_W
        self._BCSR = BCSR
        self._BCSC = BCSC

    def build_indexes(self, mask: torch.Tensor, capacity: Optional[int] = None) -> BCSIndexes:
        """mask: uint8 ``[H, W]`` (the reference form) or ``[n, H, W]`` (one mask per batch element).
        ``capacity`` bounds the index entries kept per mask (default: every block)."""
        _lib.require_cuda(mask)
        if mask.dtype == torch.bool:
            mask = mask.to(torch.uint8)
        if mask.dtype != torch.uint8:
            mask = (mask != 0).to(torch.uint8)
        if not mask.is_contiguous():
            mask = mask.contiguous()
        assert mask.dim() in (2, 3), 'expected a [H, W] or [n, H, W] mask'
        n = mask.shape[0] if mask.dim() == 3 else 1
        H, W = mask.shape[-2:]
        BH, BW = self._block_H, self._block_W
        assert H % BH == 0 and W % BW == 0, f'mask shape ({H}, {W}) is not a multiple of the block ({BH}, {BW})'
        R, C = H // BH, W // BW
        cap = R * C if capacity is None else int(capacity)
        dev = mask.device
        lead = (n,) if mask.dim() == 3 else ()
        # one int32 allocation carries every 32-bit output (host-side cost matters: the kernel itself
        # takes tens of microseconds)
        both = self._BCSR and self._BCSC
        sizes = [n * (R + 1) if self._BCSR else 0, n * cap if self._BCSR else 0,
                 n * (C + 1) if self._BCSC else 0, n * cap if (self._BCSC and not both) else 0, 2 * n]
        # keep every piece 16-byte aligned
        offs, total = [], 0
        for sz in sizes:
            offs.append(total)
            total += (sz + 3) // 4 * 4
        pool = torch.empty(total, dtype=torch.int32, device=dev)
        piece = lambda i, shape: pool[offs[i]:offs[i] + sizes[i]].view(shape)
        row_ptr = piece(0, lead + (R + 1,)) if self._BCSR else None
        bcsr = piece(1, lead + (cap,)) if self._BCSR else None
        col_ptr = piece(2, lead + (C + 1,)) if self._BCSC else None
        bcsc = None
        if self._BCSC:
            bcsc = torch.empty(lead + (cap,), dtype=torch.int64, device=dev) if both else piece(3, lead + (cap,))
        counts = piece(4, (2, n))  # row 0: nnz, row 1: uniform flag
        L = _lib.lib()
        ws_bytes = L.sparta_bcs_build_workspace_bytes(n, H, W, BH, BW)
        ws = _workspace(dev, ws_bytes)
        if torch.cuda.current_device() != dev.index:
            torch.cuda.set_device(dev)
        _lib.check(L.sparta_bcs_build(
            mask.data_ptr(), n, H, W, BH, BW, int(self._BCSR), int(self._BCSC),
            _lib.ptr(row_ptr), _lib.ptr(bcsr), _lib.ptr(col_ptr), _lib.ptr(bcsc), cap,
            counts[0].data_ptr(), counts[1].data_ptr(), None,
            ws.data_ptr(), ws_bytes, _lib.stream_ptr(dev)), 'sparta_bcs_build')
        if self._BCSR and self._BCSC:
            return BCSRCIndexes(self, mask, row_ptr, col_ptr, bcsr, bcsc, BH, BW, cap, counts[0], counts[1])
        if self._BCSR:
            return BCSRIndexes(self, mask, row_ptr, bcsr, BH, BW, cap, counts[0], counts[1])
        return BCSCIndexes(self, mask, col_ptr, bcsc, BH, BW, cap, counts[0], counts[1])

    # -- value movement --------------------------------------------------------------------
    def convert(self, dense: torch.Tensor, indexes: BCSIndexes, idx: torch.Tensor, is_bcsr: bool,
                is64: bool) -> torch.Tensor:
        _lib.require_cuda(dense)
        H, W = indexes.H, indexes.W
        assert dense.shape[-2] == H and dense.shape[-1] == W
        esz = _ELEM_BYTES[dense.dtype]
        dense = dense.contiguous()
        lead = dense.shape[:-2]
        batch = int(np.prod(lead)) if len(lead) else 1
        stride = indexes.val_stride_blocks
        vals = torch.empty((batch, stride * self._block_size), dtype=dense.dtype, device=dense.device)
        if stride > 0:
            self._move('sparta_bcs_gather', dense, vals, indexes, idx, batch, esz, is_bcsr, is64, stride)
        return vals.reshape(lead + (-1,))

    def inverse(self, sparse_val: torch.Tensor, indexes: BCSIndexes, idx: torch.Tensor, is_bcsr: bool,
                is64: bool) -> torch.Tensor:
        _lib.require_cuda(sparse_val)
        H, W = indexes.H, indexes.W
        stride = indexes.val_stride_blocks
        assert sparse_val.shape[-1] == stride * self._block_size
        esz = _ELEM_BYTES[sparse_val.dtype]
        sparse_val = sparse_val.contiguous()
        lead = sparse_val.shape[:-1]
        batch = int(np.prod(lead)) if len(lead) else 1
        dense = torch.empty((batch, H, W), dtype=sparse_val.dtype, device=sparse_val.device)
        if stride > 0:
            self._move('sparta_bcs_scatter', sparse_val, dense, indexes, idx, batch, esz, is_bcsr, is64, stride)
        else:
            dense.zero_()
        return dense.reshape(lead + (H, W))

    def _move(self, fn, src, dst, indexes, idx, batch, esz, is_bcsr, is64, stride):
        if indexes.batched:
            assert batch == indexes.n_masks, 'per-batch masks need one batch element per mask'
            # one launch per mask keeps the C entry point simple: each mask has its own index row
            for b in range(batch):
                self._launch_move(fn, src[b], dst[b], idx[b], indexes.nnz_dev[b:b + 1], 1, indexes,
                                  esz, is_bcsr, is64, stride)
        else:
            self._launch_move(fn, src, dst, idx, indexes.nnz_dev, batch, indexes, esz, is_bcsr, is64, stride)

    def _launch_move(self, fn, src, dst, idx, nnz_dev, batch, indexes, esz, is_bcsr, is64, stride):
        dev = src.device
        with torch.cuda.device(dev):
            _lib.check(getattr(_lib.lib(), fn)(
                src.data_ptr(), dst.data_ptr(), idx.data_ptr(), nnz_dev.data_ptr(), batch,
                indexes.H, indexes.W, self._block_H, self._block_W, esz, int(is_bcsr), int(is64),
                stride, stride, _lib.stream_ptr(dev)), fn)

    def _sum(self, sparse_val: torch.Tensor, indexes: BCSRIndexes, row: bool) -> torch.Tensor:
        assert not indexes.batched
        sparse_val = sparse_val.contiguous()
        lead = sparse_val.shape[:-1]
        batch = int(np.prod(lead)) if len(lead) else 1
        n_out = indexes.H if row else indexes.W
        out = torch.empty((batch, n_out), dtype=sparse_val.dtype, device=sparse_val.device)
        dev = sparse_val.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().sparta_bcs_sum(
                sparse_val.data_ptr(), out.data_ptr(), indexes.row_ptr.data_ptr(),
                indexes.bcsr_buf.data_ptr(), indexes.nnz_dev.data_ptr(), batch, indexes.H, indexes.W,
                self._block_H, self._block_W, _lib.dtype_code(sparse_val), int(row),
                indexes.val_stride_blocks, _lib.stream_ptr(dev)), 'sparta_bcs_sum')
        return out.reshape(lead + (n_out,))

    def row_sum(self, sparse_val: torch.Tensor, indexes: BCSRIndexes) -> torch.Tensor:
        return self._sum(sparse_val, indexes, True)

    def col_sum(self, sparse_val: torch.Tensor, indexes: BCSRIndexes) -> torch.Tensor:
        return self._sum(sparse_val, indexes, False)


_bcs_function_cache: Dict[str, BCSFunctionContext] = {}


def get_bcs_function(block_H: int, block_W: int, BCSR: bool, BCSC: bool) -> BCSFunctionContext:
    """(sparta/tesa/block_compressed.py:406-413)"""
    key = f'{block_H},{block_W},{BCSR},{BCSC}'
    if key not in _bcs_function_cache:
        _bcs_function_cache[key] = BCSFunctionContext(block_H, block_W, BCSR, BCSC)
    return _bcs_function_cache[key]
