"""Context and autograd function of the sparse batched matmul
(host-side mirror of sparta/specializer/funtional/batch_matmul.py).

The two backward products reuse the forward kernel families with permuted roles:

    forward:C   C  = op(A) op(B)
    backward:A  dA = dC op(B)^T          (A stored [M, K])   or   op(B) dC^T   (A stored [K, M])
    backward:B  dB = op(A)^T dC          (B stored [K, N])   or   dC^T op(A)   (B stored [N, K])

so the sparsity letter of each tensor travels with it to its new position.
"""
from typing import Any, Dict, List, Optional, Tuple

import torch

from sparta_b200.specializer.kernels import SparTASparseMatMulKernel, OpenAISparseMatMulKernel
from sparta_b200.specializer.funtional.sparse_ctx_base import SparseCtxBase, KernelPlaceholder


def _tesa_dims(mode: str, trans_A: bool, trans_B: bool) -> Tuple[str, str]:
    """Which tile dimensions give the (H, W) block shape of the sparse tensor as stored."""
    if mode == 'sdd':
        return ('K', 'M') if trans_A else ('M', 'K')
    if mode == 'dsd':
        return ('N', 'K') if trans_B else ('K', 'N')
    return ('M', 'N')


class SparseBatchMatMulCtx(SparseCtxBase):

    def __init__(self, mode: str, transpose_A: bool, transpose_B: bool, biased: bool, compressed: bool):
        super().__init__()
        self._mode = mode
        self._transpose_A = transpose_A
        self._transpose_B = transpose_B
        self._biased = biased
        self._compressed = compressed

        letter = dict(zip('ABC', mode))          # sparsity letter of each forward tensor
        sparse_tensor = 'ABC'[mode.find('s')]
        tA, tB = transpose_A, transpose_B
        # kernel slot -> (bias, which forward tensors sit at its A, B, C positions, its transposes)
        plan = {
            'forward:C': (biased, 'ABC', tA, tB),
            'backward:A': (False, 'BCA' if tA else 'CBA', tA and tB, tA or not tB),
            'backward:B': (False, 'CAB' if tB else 'ACB', (not tA) or tB, tA and tB),
        }
        self._tesa_shapes: Dict[str, Tuple[str, str]] = {}
        for kernel_name, (bias, order, k_tA, k_tB) in plan.items():
            k_mode = ''.join(letter[t] for t in order)
            self._kernels[kernel_name] = KernelPlaceholder(
                name=kernel_name,
                impls={'sparta': SparTASparseMatMulKernel, 'openai': OpenAISparseMatMulKernel},
                args=dict(mode=k_mode, biased=bias, transpose_A=k_tA, transpose_B=k_tB,
                          compressed=compressed),
                port_map={sparse_tensor: 'ABC'[order.find(sparse_tensor)]},
                connectable=compressed,
            )
            self._tesa_shapes[kernel_name] = _tesa_dims(k_mode, k_tA, k_tB)
        self._init_sparse_ports([sparse_tensor])

    def set_shape(self, batch_size: int, M: int, K: int, N: int):
        self._kernels['forward:C'].set_shape(batch_size, M, K, N)
        if self._transpose_A:
            self._kernels['backward:A'].set_shape(batch_size, K, N, M)
        else:
            self._kernels['backward:A'].set_shape(batch_size, M, N, K)
        if self._transpose_B:
            self._kernels['backward:B'].set_shape(batch_size, N, M, K)
        else:
            self._kernels['backward:B'].set_shape(batch_size, K, M, N)

    def build(self, config: Dict[str, Dict[str, Any]]):
        super().build(config)
        fwd = self._kernels['forward:C'].active_kernel()
        if fwd is not None:
            if self._biased:
                self.forward_C = lambda A, B, bias: fwd(A, B, bias)
            else:
                self.forward_C = lambda A, B: fwd(A, B)
            if self._mode == 'dds' and self._compressed:
                c_port = fwd.ports['C']
                self.backward_bias = lambda grad_C: c_port.indexes.sum(grad_C, axis=-2)
            else:
                self.backward_bias = lambda grad_C: grad_C.sum(-2)
        bwd_A = self._kernels['backward:A'].active_kernel()
        if bwd_A is not None:
            if self._transpose_A:
                self.backward_A = lambda grad_C, B: bwd_A(B, grad_C)
            else:
                self.backward_A = lambda grad_C, B: bwd_A(grad_C, B)
        bwd_B = self._kernels['backward:B'].active_kernel()
        if bwd_B is not None:
            if self._transpose_B:
                self.backward_B = lambda grad_C, A: bwd_B(grad_C, A)
            else:
                self.backward_B = lambda grad_C, A: bwd_B(A, grad_C)

    def set_sample_inputs(self, sample_inputs: List[torch.Tensor],
                          sample_grads: Optional[List[torch.Tensor]] = None):
        A, B = sample_inputs[0], sample_inputs[1]
        if self._biased:
            self._kernels['forward:C'].set_sample_inputs([A, B, sample_inputs[2].detach()])
        else:
            self._kernels['forward:C'].set_sample_inputs([A, B])
        if sample_grads is not None:
            grad_C = sample_grads[0]
            self._kernels['backward:A'].set_sample_inputs([B, grad_C] if self._transpose_A else [grad_C, B])
            self._kernels['backward:B'].set_sample_inputs([grad_C, A] if self._transpose_B else [A, grad_C])

    def get_connections(self, backward: bool = False):
        """With compressed tensors and backward kernels, the two block dimensions of the sparse
        tensor must agree across the three kernels."""
        if not (self._compressed and backward):
            return []
        conditions = [{}, {}]
        for kernel_name, dims in self._tesa_shapes.items():
            for k, dim in enumerate(dims):
                conditions[k][kernel_name] = f'BLOCK_SIZE_{dim}_VALUE'
        return conditions

    def dense_forward(self, *args):
        return self._kernels['forward:C'].dense_func(*args)


class SparseBatchMatMulFunc(torch.autograd.Function):

    @staticmethod
    def forward(ctx, sparta_ctx: SparseBatchMatMulCtx, input: torch.Tensor, weight: torch.Tensor,
                bias: Optional[torch.Tensor] = None):
        input = input.detach()
        weight = weight.detach()
        ctx.save_for_backward(input, weight, bias)
        ctx.sparta_ctx = sparta_ctx
        if bias is None:
            return sparta_ctx.forward_C(input, weight)
        return sparta_ctx.forward_C(input, weight, bias.detach())

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        input, weight, bias = ctx.saved_tensors
        grad_input = grad_weight = grad_bias = None
        grad_output = grad_output.detach()
        if ctx.needs_input_grad[1]:
            grad_input = ctx.sparta_ctx.backward_A(grad_output, weight)
        if ctx.needs_input_grad[2]:
            grad_weight = ctx.sparta_ctx.backward_B(grad_output, input)
        if bias is not None and ctx.needs_input_grad[3]:
            grad_bias = ctx.sparta_ctx.backward_bias(grad_output)
        return None, grad_input, grad_weight, grad_bias
