"""``SparseAttention``: softmax_mask(Q K^T / sqrt(E)) V over the kept blocks of the mask
(host-side mirror of sparta/specializer/operators/sparse_attention.py:14-238).

Two execution paths share the reference's API:

* the composed path of the reference -- dds(Q, K^T) -> sparse softmax -> sdd(P, V), three kernels
  that share one BCSR index set -- for every dtype and tile size, with backward;
* the fused forward kernel (``sparta_attn_fwd``) for fp16 / bf16, E in {64, 128} and 64 x 64 tiles,
  where the score tensor never reaches global memory.  It is chosen automatically when the
  configuration allows it (``fused='auto'``) and provides no backward: with ``'auto'`` a forward whose
  inputs require gradients takes the composed path.
"""
from typing import Any, Dict, List, Optional
import os
import warnings

import numpy as np
import torch

from sparta_b200 import _lib
from sparta_b200.specializer.operators.operator_base import OperatorBase
from sparta_b200.specializer.operators.sparse_matmul import SparseBatchMatMul
from sparta_b200.specializer.operators.sparse_softmax import SparseSoftmax
from sparta_b200.specializer.kernels import KernelBase, PortConfig

FUSED_BLOCK = 64
FUSED_HEAD_DIMS = (64, 128)


class _FusedAttentionFunc(torch.autograd.Function):

    @staticmethod
    def forward(ctx, op: 'SparseAttention', query, key, value):
        return op._fused_forward(query.detach(), key.detach(), value.detach())

    @staticmethod
    def backward(ctx, grad):
        raise NotImplementedError(
            'the fused sparse attention kernel has no backward; build with fused=False to train')


class SparseAttention(OperatorBase):
    r"""Sparse attention :math:`\text{Softmax}(Q K^T) V`.

    Args:
        mask: :math:`(N_{target}, N_{source})` uint8 mask.
        fused: ``'auto'`` (default), ``True`` or ``False`` -- see the module docstring.

    Shape: Q :math:`(B \times H, N_{target}, E)`; K, V :math:`(B \times H, N_{source}, E)`;
    output like Q.
    """

    def __init__(self, mask: torch.Tensor, fused: Any = 'auto'):
        super().__init__()
        self.mask = mask
        self._Nt, self._Ns = mask.shape
        self._matmul_qk = SparseBatchMatMul(C_mask=mask, transpose_A=False, transpose_B=True, compressed=True)
        self._softmax = SparseSoftmax(mask=mask, compressed=True)
        self._matmul_out = SparseBatchMatMul(A_mask=mask, transpose_A=False, transpose_B=False, compressed=True)
        self._sparse_port: PortConfig = None
        self._fused_request = fused
        self._use_fused = False
        self._scale = 1.0
        self._attn_ws: Optional[torch.Tensor] = None
        self._attn_status: Optional[torch.Tensor] = None
        #: debugging aid: read the kernel's status words after every fused forward (one device
        #: synchronisation per call) and raise when a bounded wait gave up
        self.check_status = os.environ.get('SPARTA_B200_CHECK_STATUS', '0') == '1'
        self.ready = False

    # ---- forward paths ------------------------------------------------------------------
    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor):
        if self.ready and self.dynamic:
            self._sparse_port.refresh()
        if self.ready and self._use_fused:
            # the fused kernel is forward-only: with fused='auto' a call that autograd will differentiate
            # takes the three-operator path, which the reference trains through
            # (test/unit/test_sparse_attention.py:86-92); fused=True keeps the fused kernel and raises in backward
            wants_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value))
            if self._fused_request is True or not wants_grad:
                return _FusedAttentionFunc.apply(self, query, key, value)
        qk = self._matmul_qk.forward(query, key)
        sm = self._softmax.forward(qk)
        return self._matmul_out.forward(sm, value)

    def forward_gathered(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                         out: torch.Tensor, copies: List[int]) -> torch.Tensor:
        """Fused forward (no autograd) that writes the result into ``out`` and, tile by tile from the same
        kernel, into every address of ``copies``: device addresses of buffers laid out like ``out``,
        normally this rank's slice of the peers' gathered outputs (``sparta_b200.parallel.GatheredHeads``).
        Raises when the fused kernel for this shape cannot store copies (gather with a collective then)."""
        assert self.ready and self._use_fused, 'forward_gathered needs an operator built on the fused kernel'
        return self._fused_forward(query.detach(), key.detach(), value.detach(), out=out, copies=copies)

    def _fused_forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                       copies: Optional[List[int]] = None) -> torch.Tensor:
        _lib.require_cuda(q, k, v)
        idx = self._sparse_port.indexes
        shape = q.shape
        E = shape[-1]
        q = q.reshape(-1, self._Nt, E).contiguous()
        k = k.reshape(-1, self._Ns, E).contiguous()
        v = v.reshape(-1, self._Ns, E).contiguous()
        heads = q.shape[0]
        if out is None:
            out = torch.empty_like(q)
        else:
            assert out.is_contiguous() and out.dtype == q.dtype and out.numel() == q.numel() and out.device == q.device
        L = _lib.lib()
        ws_bytes = L.sparta_attn_fwd_workspace_bytes(heads, self._Nt, self._Ns, E, FUSED_BLOCK)
        if self._attn_ws is None or self._attn_ws.numel() < ws_bytes or self._attn_ws.device != q.device:
            self._attn_ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
            self._attn_status = torch.zeros(4, dtype=torch.int32, device=q.device)
        mask = None if idx.block_uniform else idx.raw_mask
        if copies:
            import ctypes
            addresses = (ctypes.c_void_p * len(copies))(*copies)
            with torch.cuda.device(q.device):
                _lib.check(L.sparta_attn_fwd_gather(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                    idx.row_ptr.data_ptr(), idx.bcsr_buf.data_ptr(), idx.nnz_dev.data_ptr(),
                    _lib.ptr(mask), float(self._scale), heads, self._Nt, self._Ns, E, FUSED_BLOCK,
                    _lib.dtype_code(q), None, self._attn_status.data_ptr(), addresses, len(copies),
                    _lib.stream_ptr(q.device)), 'sparta_attn_fwd_gather')
            if self.check_status and any(self.fused_status()):
                raise RuntimeError(f'fused sparse attention: a bounded wait ran out on the device, status words '
                                   f'{self.fused_status()}; the output is invalid')
            return out.reshape(shape)
        with torch.cuda.device(q.device):
            _lib.check(L.sparta_attn_fwd(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                idx.row_ptr.data_ptr(), idx.bcsr_buf.data_ptr(), idx.nnz_dev.data_ptr(),
                _lib.ptr(mask), float(self._scale), heads, self._Nt, self._Ns, E, FUSED_BLOCK,
                _lib.dtype_code(q), None, self._attn_status.data_ptr(),
                self._attn_ws.data_ptr(), self._attn_ws.numel(), _lib.stream_ptr(q.device)), 'sparta_attn_fwd')
        if self.check_status and any(self.fused_status()):
            raise RuntimeError(f'fused sparse attention: a bounded wait ran out on the device, status words '
                               f'{self.fused_status()}; the output is invalid')
        return out.reshape(shape)

    def fused_status(self) -> List[int]:
        """Device status words of the fused kernel (all zero unless a bounded wait ran out)."""
        return [] if self._attn_status is None else self._attn_status.tolist()

    # ---- masks ----------------------------------------------------------------------------
    def update_mask(self, mask: torch.Tensor):
        self.mask = mask
        if self.ready:
            self._sparse_port.set_mask(mask)
            for op in (self._matmul_qk, self._softmax, self._matmul_out):
                op._sparse_ctx.update_func()
        else:
            for op in (self._matmul_qk, self._softmax, self._matmul_out):
                for ports in op._sparse_ctx.sparse_ports.values():
                    for port in ports:
                        port.set_mask(mask)

    # ---- build ----------------------------------------------------------------------------
    def _fused_possible(self, config: Dict[str, Any], query: torch.Tensor) -> bool:
        if query.dtype not in (torch.float16, torch.bfloat16) or query.shape[-1] not in FUSED_HEAD_DIMS:
            return False
        qk, sm, out = config['qk/forward:C'], config['sm/forward:y'], config['out/forward:C']
        sizes = [qk.get('BLOCK_SIZE_M_VALUE'), qk.get('BLOCK_SIZE_N_VALUE'), sm.get('BLOCK_SIZE_H_VALUE'),
                 sm.get('BLOCK_SIZE_W_VALUE'), out.get('BLOCK_SIZE_M_VALUE'), out.get('BLOCK_SIZE_K_VALUE')]
        if any(s != FUSED_BLOCK for s in sizes):
            return False
        if self._Nt % (2 * FUSED_BLOCK) or self._Ns % FUSED_BLOCK or self._Ns // FUSED_BLOCK > 1024:
            return False
        return _lib.lib().sparta_tile_table(_lib.OP_ATTENTION, _lib.DTYPE_CODE[query.dtype], None, 0) > 0

    def build(self, config: Dict[str, Any], sample_inputs: List[torch.Tensor]):
        query, key, value = sample_inputs
        qB, kB, vB = (int(np.prod(t.shape[:-2])) for t in (query, key, value))
        (qN, qE), (kN, kE), (vN, vE) = (t.shape[-2:] for t in (query, key, value))
        assert qB == kB == vB, 'query, key and value should have the same batch size'
        assert self._Nt == qN, f'expect query shape (?, {self._Nt}, ?), got {query.shape}'
        assert self._Ns == kN, f'expect key shape (?, {self._Ns}, ?), got {key.shape}'
        assert self._Ns == vN, f'expect value shape (?, {self._Ns}, ?), got {value.shape}'
        assert qE == kE == vE, 'query, key and value should have the same embed dim'

        self._softmax.set_temperature(np.sqrt(qE))
        self._scale = 1.0 / float(np.sqrt(qE))

        ops: Dict[str, OperatorBase] = {'qk': self._matmul_qk, 'sm': self._softmax, 'out': self._matmul_out}
        port_of = {'qk': 'C', 'sm': 'y', 'out': 'A'}

        # one sparse port for the three operators: one BCSR index set serves qk.C, sm.y and out.A
        kernels: List[KernelBase] = []
        names: List[str] = []
        for op_name, op in ops.items():
            for slot, placeholder in op._sparse_ctx.get_kernel_placeholders().items():
                kernels.append(placeholder.possible_kernels[config[f'{op_name}/{slot}']['_impl']])
                names.append(placeholder.port_map[port_of[op_name]])
        self._sparse_port = kernels[0].ports[names[0]]
        for kernel, name in zip(kernels[1:], names[1:]):
            self._sparse_port.connect(kernel, name)

        fusable = self._fused_possible(config, query)
        if self._fused_request is True and not fusable:
            raise ValueError('fused sparse attention needs fp16/bf16 inputs, E in {64, 128} and 64x64 tiles')
        self._use_fused = fusable and self._fused_request in (True, 'auto')

        # shapes of the intermediate tensors are not needed to bind prebuilt kernels, so no dense
        # pre-pass is run here (the reference computes qk and sm densely for shape inference)
        heads = qB
        qk_stub = torch.empty((heads, 0), dtype=query.dtype, device=query.device)
        sample = {'qk': [query.reshape(heads, qN, qE), key.reshape(heads, kN, kE)],
                  'sm': None, 'out': [qk_stub, value.reshape(heads, vN, vE)]}
        for op_name, op in ops.items():
            sub_config = {k.split('/')[1]: v for k, v in config.items() if k.startswith(f'{op_name}/')}
            if op_name == 'sm':
                op._shape['batch_size'] = heads
                op._sparse_ctx.select_impls({k: v['_impl'] for k, v in sub_config.items()})
                op._sparse_ctx.set_shape(**op._shape)
                op._compile(config=sub_config)
            elif op_name == 'out':
                op._shape = {'batch_size': heads, 'M': self._Nt, 'K': self._Ns, 'N': vE}
                op._sparse_ctx.select_impls({k: v['_impl'] for k, v in sub_config.items()})
                op._sparse_ctx.set_shape(**op._shape)
                op._compile(config=sub_config)
            else:
                op.build(config=sub_config, sample_inputs=sample[op_name])
        self.ready = True

    # ---- tuning interface -------------------------------------------------------------------
    def set_sample_inputs(self, sample_inputs: List[torch.Tensor],
                          sample_grads: Optional[List[torch.Tensor]] = None):
        query, key, value = sample_inputs
        self._softmax.set_temperature(np.sqrt(query.shape[-1]))
        if sample_grads is not None:
            query.requires_grad = True
            key.requires_grad = True
            value.requires_grad = True
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            qk = self._matmul_qk.forward(query, key)
            sm = self._softmax.forward(qk)
        grad_qk = grad_sm = None
        if sample_grads is not None:
            qk.retain_grad()
            sm.retain_grad()
            with warnings.catch_warnings():
                warnings.simplefilter('ignore')
                out = self._matmul_out.forward(sm, value)
                out.backward(sample_grads[0])
            grad_sm, grad_qk = [sm.grad], [qk.grad]
            query, key, value = query.detach(), key.detach(), value.detach()
        self._matmul_qk.set_sample_inputs([query, key], grad_qk)
        self._softmax.set_sample_inputs([qk], grad_sm)
        self._matmul_out.set_sample_inputs([sm, value], sample_grads)

    def _combine(self, qk: Dict[str, Any], sm: Dict[str, Any], out: Dict[str, Any], backward: bool):
        merged = {}
        for prefix, part in (('qk', qk), ('sm', sm), ('out', out)):
            for k, v in part.items():
                if backward or k.startswith('forward'):
                    merged[f'{prefix}/{k}'] = v
        return merged

    def get_search_space(self, backward: bool = False):
        return self._combine(self._matmul_qk.get_search_space(backward=True),
                             self._softmax.get_search_space(backward=True),
                             self._matmul_out.get_search_space(backward=True), backward)

    def get_connections(self, backward: bool = False):
        return [
            self._combine(qk, sm, out, backward)
            for qk, sm, out in zip(self._matmul_qk.get_connections(backward=True),
                                   self._softmax.get_connections(backward=True),
                                   self._matmul_out.get_connections(backward=True))
        ]

    def get_kernel_placeholders(self, backward: bool = False):
        return self._combine(self._matmul_qk.get_kernel_placeholders(backward=True),
                             self._softmax.get_kernel_placeholders(backward=True),
                             self._matmul_out.get_kernel_placeholders(backward=True), backward)

    def get_sparse_indexes(self, port_name: str = 'qk'):
        return None if self._sparse_port is None else self._sparse_port.indexes
