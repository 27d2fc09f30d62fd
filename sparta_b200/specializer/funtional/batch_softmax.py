"""Context and autograd function of the masked softmax.

Public surface as in sparta/specializer/funtional/batch_softmax.py (``SparseBatchSoftmaxCtx`` :13-79,
``SparseBatchSoftmaxFunc`` :82-98): two slots, ``forward:y`` and ``backward:x``, both keyed on the sparse
tensor ``y``.  The kernels take the *reciprocal* temperature (:19), which the context keeps as ``_T``.
"""
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from sparta_b200.specializer.kernels import SparTASparseSoftmaxForwardKernel, SparTASparseSoftmaxBackwardKernel
from sparta_b200.specializer.funtional.sparse_ctx_base import SparseCtxBase, KernelPlaceholder

_FWD, _BWD = 'forward:y', 'backward:x'
_SLOT_KERNELS = {_FWD: SparTASparseSoftmaxForwardKernel, _BWD: SparTASparseSoftmaxBackwardKernel}
_SHARED_BLOCK_PARAMS = ('BLOCK_SIZE_H_VALUE', 'BLOCK_SIZE_W_VALUE')


class SparseBatchSoftmaxCtx(SparseCtxBase):

    def __init__(self, compressed: bool, temperature: float = 1):
        super().__init__()
        self._compressed = compressed
        self._batch_size: Optional[int] = None
        self.set_temperature(temperature)
        for slot, kernel_class in _SLOT_KERNELS.items():
            self._kernels[slot] = KernelPlaceholder(
                name=slot, impls={'sparta': kernel_class}, args={'compressed': compressed},
                port_map={'y': 'y'}, connectable=compressed)
        self._init_sparse_ports(['y'])

    def set_temperature(self, temperature: float):
        self._T = np.float32(1 / temperature)

    def set_shape(self, batch_size: int, H: int, W: int):
        self._batch_size = batch_size
        for slot in _SLOT_KERNELS:
            self._kernels[slot].set_shape(batch_size, H, W)

    # the temperature is read at call time, so set_temperature() after build() takes effect
    def _run_forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._kernels[_FWD].active_kernel()(x, self._T)

    def _run_backward(self, grad: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
        return self._kernels[_BWD].active_kernel()(grad, output, self._T)

    def build(self, config: Dict[str, Dict[str, Any]]):
        super().build(config)
        if self._kernels[_FWD].active_kernel() is not None:
            self.forward = self._run_forward
        if self._kernels[_BWD].active_kernel() is not None:
            self.backward = self._run_backward

    def set_sample_inputs(self, sample_inputs: List[torch.Tensor],
                          sample_grads: Optional[List[torch.Tensor]] = None):
        x = sample_inputs[0]
        self._kernels[_FWD].set_sample_inputs([x, self._T])
        if sample_grads is None:
            return
        y = self.dense_forward(x)
        self._kernels[_BWD].set_sample_inputs([sample_grads[0], y, self._T])

    def get_connections(self, backward: bool = False):
        """Forward and backward share ``y``'s indexes when it is stored compressed, so their block
        sizes must agree."""
        if not (backward and self._compressed):
            return []
        return [{slot: param for slot in _SLOT_KERNELS} for param in _SHARED_BLOCK_PARAMS]

    def dense_forward(self, *args):
        return self._kernels[_FWD].dense_func(*args, self._T)


class SparseBatchSoftmaxFunc(torch.autograd.Function):

    @staticmethod
    def forward(ctx, sparta_ctx: SparseBatchSoftmaxCtx, x: torch.Tensor):
        y = sparta_ctx.forward(x.detach())
        ctx.sparta_ctx = sparta_ctx
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad: torch.Tensor):
        y, = ctx.saved_tensors
        return None, ctx.sparta_ctx.backward(grad.detach(), y.detach())
