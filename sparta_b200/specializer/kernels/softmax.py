"""Masked softmax kernel objects (host-side mirror of sparta/specializer/kernels/softmax.py).

The closures call ``sparta_softmax_fwd`` / ``sparta_softmax_bwd``.  ``T`` handed to a kernel call is
the reciprocal temperature, as in the reference (funtional/batch_softmax.py:19).  The element mask
is only sent to the kernel when some kept block contains a zero; block-uniform masks skip the byte
traffic.
"""
from typing import Any, Dict

import numpy as np
import torch

from sparta_b200 import _lib
from sparta_b200.common.tuning import TunableItemCfg
from sparta_b200.specializer.kernels.kernel_base import KernelBase, PortConfig
from sparta_b200.testing import sparse_softmax_forward_reference, sparse_softmax_backward_reference


class SparseSoftmaxKernel(KernelBase):

    __algo__: str = ''
    __direction__: str = ''

    def __init__(self, compressed: bool = False, dtype: str = 'float'):
        self._compressed = compressed
        self._dtype = dtype
        self._mask_cache = (None, None)
        super().__init__()

    def _add_parameters(self):
        self._add_parameter('BATCH_SIZE')
        self._add_parameter('GLOBAL_H_VALUE')
        self._add_parameter('GLOBAL_W_VALUE')
        self._add_parameter('COMPRESSED', value=self._compressed)

    def set_parameters(self, params: Dict[str, Any]):
        super().set_parameters(params)
        BH, BW = self.get_block_shape()
        self.ports['y'].set_block_size(BH, BW)

    def set_shape(self, batch_size: int, H: int, W: int):
        self.set_parameter('BATCH_SIZE', batch_size)
        self.set_parameter('GLOBAL_H_VALUE', H)
        self.set_parameter('GLOBAL_W_VALUE', W)

    def get_shape(self):
        return tuple(self.get_parameter(n) for n in ['BATCH_SIZE', 'GLOBAL_H_VALUE', 'GLOBAL_W_VALUE'])

    def get_block_shape(self):
        return self.get_parameter('BLOCK_SIZE_H_VALUE'), self.get_parameter('BLOCK_SIZE_W_VALUE')

    def _element_mask(self, indexes):
        """uint8 mask in the layout of x (compressed or dense), or None when kept blocks are full."""
        if indexes.block_uniform:
            return None
        cached_for, mask = self._mask_cache
        if cached_for is not indexes:
            mask = indexes.raw_mask
            if self._compressed:
                mask = indexes.convert(mask)
            self._mask_cache = (indexes, mask)
        return mask

    def _launch(self, fn_name, tensors, out, T):
        _, H, W = self.get_shape()
        BH, BW = self.get_block_shape()
        indexes = self.ports['y'].indexes
        assert not indexes.batched, 'softmax takes one 2-D mask'
        mask = self._element_mask(indexes)
        first = tensors[0]
        batch = first.numel() // (out.shape[-1] if self._compressed else H * W)
        with torch.cuda.device(first.device):
            _lib.check(getattr(_lib.lib(), fn_name)(
                *[t.data_ptr() for t in tensors], out.data_ptr(),
                indexes.row_ptr.data_ptr(), indexes.bcsr_buf.data_ptr(), indexes.nnz_dev.data_ptr(),
                _lib.ptr(mask), float(T), batch, H, W, BH, BW, int(self._compressed),
                _lib.dtype_code(first), indexes.val_stride_blocks, _lib.stream_ptr(first.device),
            ), fn_name)
        return out


class SparseSoftmaxForwardKernel(SparseSoftmaxKernel):

    __direction__ = 'forward'

    def _set_ports(self):
        self.ports['x'] = PortConfig(name='x', is_input=True, is_sparse=True, BCSR=True)
        self.ports['y'] = PortConfig(name='y', is_input=False, is_sparse=True, BCSR=True)
        self.ports['x'].connect(self, 'y')

    def update_func(self):
        def softmax_forward_func(x: torch.Tensor, T: np.float32):
            _lib.require_cuda(x)
            x = x.contiguous()
            y = torch.empty_like(x)
            if y.numel() == 0:
                return y
            return self._launch('sparta_softmax_fwd', [x], y, T)

        self._func = softmax_forward_func

    def _convert_data(self, inputs, outputs):
        mask = self.ports['y'].mask
        inputs[0] = (inputs[0].reshape(self.get_shape()) * mask).detach()
        outputs[0] = (outputs[0].reshape(self.get_shape()) * mask).detach()
        if self._compressed:
            indexes = self.ports['y'].indexes
            inputs[0] = indexes.convert(inputs[0])
            outputs[0] = indexes.convert(outputs[0])

    def reference(self, *args):
        x, T = args
        return sparse_softmax_forward_reference(x, self.ports['y'].mask, 1 / T)


class SparseSoftmaxBackwardKernel(SparseSoftmaxKernel):

    __direction__ = 'backward'

    def _set_ports(self):
        self.ports['grad_y'] = PortConfig(name='grad_y', is_input=True, is_sparse=True, BCSR=True)
        self.ports['y'] = PortConfig(name='y', is_input=True, is_sparse=True, BCSR=True)
        self.ports['grad_x'] = PortConfig(name='grad_x', is_input=False, is_sparse=True, BCSR=True)
        self.ports['grad_y'].connect(self, 'y')
        self.ports['grad_y'].connect(self, 'grad_x')

    def update_func(self):
        def softmax_backward_func(grad_y: torch.Tensor, y: torch.Tensor, T: np.float32):
            _lib.require_cuda(grad_y, y)
            grad_y = grad_y.contiguous()
            y = y.contiguous()
            grad_x = torch.empty_like(grad_y)
            if grad_x.numel() == 0:
                return grad_x
            return self._launch('sparta_softmax_bwd', [grad_y, y], grad_x, T)

        self._func = softmax_backward_func

    def _convert_data(self, inputs, outputs):
        mask = self.ports['y'].mask
        inputs[0] = (inputs[0].reshape(self.get_shape()) * mask).detach()
        inputs[1] = (inputs[1].reshape(self.get_shape()) * mask).detach()
        outputs[0] = (outputs[0].reshape(self.get_shape()) * mask).detach()
        if self._compressed:
            indexes = self.ports['y'].indexes
            inputs[0] = indexes.convert(inputs[0])
            inputs[1] = indexes.convert(inputs[1])
            outputs[0] = indexes.convert(outputs[0])

    def reference(self, *args):
        grad_y, y, T = args
        return sparse_softmax_backward_reference(grad_y, y, self.ports['y'].indexes.raw_mask, 1 / T)


class SparTASoftmaxKernel(SparseSoftmaxKernel):
    """Search space of the reference (softmax.py:160-180).  ROW_TILE_VALUE is accepted for
    configuration compatibility; the prebuilt kernel always runs one warp per row, eight rows per
    CTA."""

    __algo__ = 'sparta'

    def _add_parameters(self):
        super()._add_parameters()
        self._add_parameter('BLOCK_SIZE_H_VALUE', is_tunable=True,
                            search_space=TunableItemCfg('choice', [8, 16, 32, 64, 128]))
        self._add_parameter('BLOCK_SIZE_W_VALUE', is_tunable=True,
                            search_space=TunableItemCfg('choice', [16, 32, 64, 128]))
        self._add_parameter('ROW_TILE_VALUE', is_tunable=True,
                            search_space=TunableItemCfg('choice', [1, 2, 4, 8, 16]))

    def _check_parameters(self, params: Dict[str, Any]):
        BH = params['BLOCK_SIZE_H_VALUE']
        RT = params['ROW_TILE_VALUE']
        assert BH > RT
        _, H, W = self.get_shape()
        if H is not None:
            assert H % BH == 0 and W % params['BLOCK_SIZE_W_VALUE'] == 0


class SparTASparseSoftmaxForwardKernel(SparseSoftmaxForwardKernel, SparTASoftmaxKernel):
    pass


class SparTASparseSoftmaxBackwardKernel(SparseSoftmaxBackwardKernel, SparTASoftmaxKernel):
    pass
