"""``SparseBatchMatMul``: C = op(A) op(B) with a mask on A, B or C
(host-side mirror of sparta/specializer/operators/sparse_matmul.py:12-136)."""
from typing import Optional

import torch

from sparta_b200.specializer.operators.operator_base import OperatorBase
from sparta_b200.specializer.funtional import SparseBatchMatMulCtx, SparseBatchMatMulFunc


class SparseBatchMatMul(OperatorBase):
    r"""Sparse batched matrix multiplication :math:`C = AB`.

    Exactly one of ``A_mask`` (sdd), ``B_mask`` (dsd), ``C_mask`` (dds) is given.  Inputs are 3-D:
    A is :math:`(B, M, K)` (or :math:`(B, K, M)` with ``transpose_A``), B is :math:`(B, K, N)` (or
    :math:`(B, N, K)`), C is :math:`(B, M, N)`.  With ``compressed`` the masked tensor is exchanged as
    :math:`(B, *)` block-compressed values.

    Extension: a 3-D mask ``(B, H, W)`` gives every batch element its own mask; compressed tensors
    then hold ``capacity`` blocks per batch element (``get_sparse_indexes(port).capacity``) and the
    per-element block counts stay on the device (``.nnz_dev``).
    """

    __sparse_func__ = SparseBatchMatMulFunc

    def __init__(self, A_mask: Optional[torch.Tensor] = None, B_mask: Optional[torch.Tensor] = None,
                 C_mask: Optional[torch.Tensor] = None, transpose_A: bool = False,
                 transpose_B: bool = False, compressed: bool = True, capacity: Optional[int] = None):
        super().__init__()
        self._transpose_A = transpose_A
        self._transpose_B = transpose_B
        ctx_args = dict(transpose_A=transpose_A, transpose_B=transpose_B, biased=False, compressed=compressed)
        batch_size, M, K, N = None, None, None, None
        if A_mask is not None:
            self._sparse_ctx = SparseBatchMatMulCtx(mode='sdd', **ctx_args)
            K, M = A_mask.shape[-2:] if transpose_A else A_mask.shape[-2:][::-1]
        elif B_mask is not None:
            self._sparse_ctx = SparseBatchMatMulCtx(mode='dsd', **ctx_args)
            N, K = B_mask.shape[-2:] if transpose_B else B_mask.shape[-2:][::-1]
        elif C_mask is not None:
            self._sparse_ctx = SparseBatchMatMulCtx(mode='dds', **ctx_args)
            M, N = C_mask.shape[-2:]
        else:
            raise ValueError('expected a sparse mask on A / B / C')
        if capacity is not None:
            for ports in self._sparse_ctx.sparse_ports.values():
                for port in ports:
                    port.capacity = capacity
        self._capacity = capacity
        self._shape = {'batch_size': batch_size, 'M': M, 'K': K, 'N': N}
        self.update_mask(A_mask, B_mask, C_mask)

    def build(self, config, sample_inputs):
        super().build(config, sample_inputs)
        if self._capacity is not None:  # select_impls may have merged ports: keep the bound on them
            for ports in self._sparse_ctx.sparse_ports.values():
                for port in ports:
                    port.capacity = self._capacity

    def update_mask(self, A_mask: Optional[torch.Tensor] = None, B_mask: Optional[torch.Tensor] = None,
                    C_mask: Optional[torch.Tensor] = None):
        if sum(m is not None for m in (A_mask, B_mask, C_mask)) > 1:
            raise ValueError('linear operators with multiple sparse masks are not supported')
        if A_mask is not None:
            self._set_mask({'A': A_mask})
        elif B_mask is not None:
            self._set_mask({'B': B_mask})
        elif C_mask is not None:
            self._set_mask({'C': C_mask})
        else:
            raise ValueError('expected a sparse mask on A / B / C')

    def _read_sample_inputs(self, A: torch.Tensor, B: torch.Tensor):
        if self._transpose_A:
            batch_size, K, M = A.shape
        else:
            batch_size, M, K = A.shape
        if self._transpose_B:
            batch_size, N, K = B.shape
        else:
            batch_size, K, N = B.shape
        self._shape = {'batch_size': batch_size, 'M': M, 'K': K, 'N': N}
