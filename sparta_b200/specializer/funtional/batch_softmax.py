"""Context and autograd function of the sparse softmax
(host-side mirror of sparta/specializer/funtional/batch_softmax.py)."""
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from sparta_b200.specializer.kernels import SparTASparseSoftmaxForwardKernel, SparTASparseSoftmaxBackwardKernel
from sparta_b200.specializer.funtional.sparse_ctx_base import SparseCtxBase, KernelPlaceholder


class SparseBatchSoftmaxCtx(SparseCtxBase):

    def __init__(self, compressed: bool, temperature: float = 1):
        super().__init__()
        self._compressed = compressed
        self._T = np.float32(1 / temperature)  # kernels multiply by the reciprocal temperature
        self._batch_size: Optional[int] = None
        for kernel_name, kernel_class in [('forward:y', SparTASparseSoftmaxForwardKernel),
                                          ('backward:x', SparTASparseSoftmaxBackwardKernel)]:
            self._kernels[kernel_name] = KernelPlaceholder(
                name=kernel_name, impls={'sparta': kernel_class}, args={'compressed': compressed},
                port_map={'y': 'y'}, connectable=compressed,
            )
        self._init_sparse_ports(['y'])

    def set_temperature(self, temperature: float):
        self._T = np.float32(1 / temperature)

    def set_shape(self, batch_size: int, H: int, W: int):
        self._kernels['forward:y'].set_shape(batch_size, H, W)
        self._kernels['backward:x'].set_shape(batch_size, H, W)
        self._batch_size = batch_size

    def build(self, config: Dict[str, Dict[str, Any]]):
        super().build(config)
        fwd = self._kernels['forward:y'].active_kernel()
        if fwd is not None:
            self.forward = lambda x: fwd(x, self._T)
        bwd = self._kernels['backward:x'].active_kernel()
        if bwd is not None:
            self.backward = lambda grad, output: bwd(grad, output, self._T)

    def set_sample_inputs(self, sample_inputs: List[torch.Tensor],
                          sample_grads: Optional[List[torch.Tensor]] = None):
        x = sample_inputs[0]
        self._kernels['forward:y'].set_sample_inputs([x, self._T])
        if sample_grads is not None:
            y = self._kernels['forward:y'].dense_func(x, self._T)
            self._kernels['backward:x'].set_sample_inputs([sample_grads[0], y, self._T])

    def get_connections(self, backward: bool = False):
        if self._compressed and backward:
            return [
                {'forward:y': 'BLOCK_SIZE_H_VALUE', 'backward:x': 'BLOCK_SIZE_H_VALUE'},
                {'forward:y': 'BLOCK_SIZE_W_VALUE', 'backward:x': 'BLOCK_SIZE_W_VALUE'},
            ]
        return []

    def dense_forward(self, *args):
        return self._kernels['forward:y'].dense_func(*args, self._T)


class SparseBatchSoftmaxFunc(torch.autograd.Function):

    @staticmethod
    def forward(ctx, sparta_ctx: SparseBatchSoftmaxCtx, x: torch.Tensor):
        ctx.sparta_ctx = sparta_ctx
        output = sparta_ctx.forward(x.detach())
        ctx.save_for_backward(output)
        return output

    @staticmethod
    def backward(ctx, grad: torch.Tensor):
        output, = ctx.saved_tensors
        return None, ctx.sparta_ctx.backward(grad.detach(), output.detach())
