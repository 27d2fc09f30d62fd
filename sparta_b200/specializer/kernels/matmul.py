"""Block-sparse matmul kernel objects (host-side mirror of sparta/specializer/kernels/matmul.py).

``mode`` letters name A, B, C in that order (matmul.py:60-84): ``sdd`` = A sparse, ``dsd`` = B
sparse, ``dds`` = C sparse.  The CTA tile (BLOCK_SIZE_{M,K,N}_VALUE) is also the block size of the
sparse operand in its two dimensions.  The launch closure calls ``sparta_bsmm_{sdd,dsd,dds}``; which
prebuilt kernel runs (tcgen05 or FMA) is decided by the library's tile table unless ``_family`` is
given in the parameters.
"""
from typing import Any, Dict

import torch

from sparta_b200 import _lib
from sparta_b200.common.tuning import TunableItemCfg
from sparta_b200.specializer.kernels.kernel_base import KernelBase, PortConfig

_FAMILY = {'auto': _lib.IMPL_AUTO, 'simt': _lib.IMPL_SIMT, 'tcgen05': _lib.IMPL_TCGEN05}
_ENTRY = {'sdd': 'sparta_bsmm_sdd', 'dsd': 'sparta_bsmm_dsd', 'dds': 'sparta_bsmm_dds'}
_OP_CODE = {'sdd': _lib.OP_SDD, 'dsd': _lib.OP_DSD, 'dds': _lib.OP_DDS}


class SparseMatMulKernel(KernelBase):

    __algo__: str = ''

    def __init__(self, mode: str, dtype: str = 'float', biased: bool = True, transpose_A: bool = False,
                 transpose_B: bool = True, compressed: bool = True):
        if mode not in ['sdd', 'dsd', 'dds']:
            raise ValueError(f'invalid sparse type: {mode}')
        self._mode = mode
        self._dtype = dtype
        self._biased = biased
        self._transpose_A = transpose_A
        self._transpose_B = transpose_B
        self._compressed = compressed
        self._family = 'auto'
        self._sample_dtype = torch.float32  # element type the tile table is read for, see set_sample_dtype
        # which port is sparse, which tile sizes give its block shape, which index form it uses
        if mode == 'sdd':
            self._sparse_port = 'A'
            hw = ('K', 'M') if transpose_A else ('M', 'K')
            self._bcs_mode = 'BCSC' if transpose_A else 'BCSR'
        elif mode == 'dsd':
            self._sparse_port = 'B'
            hw = ('N', 'K') if transpose_B else ('K', 'N')
            self._bcs_mode = 'BCSR' if transpose_B else 'BCSC'
        else:
            self._sparse_port = 'C'
            hw = ('M', 'N')
            self._bcs_mode = 'BCSR'
        self._sparse_block_H = f'BLOCK_SIZE_{hw[0]}_VALUE'
        self._sparse_block_W = f'BLOCK_SIZE_{hw[1]}_VALUE'
        if self._bcs_mode == 'BCSR':
            self._tesa_vars = ['row_ptr', 'BCSR_idx', 'nnz']
        else:
            self._tesa_vars = ['col_ptr', 'BCSC_idx', 'nnz']
        if mode == 'dds':
            self._tesa_vars = self._tesa_vars[1:]
        super().__init__()

    def _set_ports(self):
        self.ports['A'] = PortConfig(name='A', is_input=True)
        self.ports['B'] = PortConfig(name='B', is_input=True)
        if self._biased:
            self.ports['bias'] = PortConfig(name='bias', is_input=True)
        self.ports['C'] = PortConfig(name='C', is_input=False)
        self.ports[self._sparse_port].set_sparse(self._bcs_mode == 'BCSR', self._bcs_mode == 'BCSC')

    def _add_parameters(self):
        for name in ['BATCH_SIZE', 'GLOBAL_M_VALUE', 'GLOBAL_K_VALUE', 'GLOBAL_N_VALUE', 'BCSR', 'BCSC']:
            self._add_parameter(name)
        self._add_parameter('BIASED', value=self._biased)
        self._add_parameter('TRANSPOSE_A', value=self._transpose_A)
        self._add_parameter('TRANSPOSE_B', value=self._transpose_B)
        self._add_parameter('COMPRESSED', value=self._compressed)

    def set_sample_dtype(self, dtype: torch.dtype):
        """Element type of the tensors the kernel will be tuned / run on: the prebuilt tile shapes depend
        on it (the tcgen05 kernels take fp16 / bf16 only)."""
        if dtype in _lib.DTYPE_CODE:
            self._sample_dtype = dtype

    def tile_shapes(self, dtype: torch.dtype = None) -> Dict[Any, int]:
        """``{(BM, BK, BN): kernel family}`` of the library's tile table for this kernel's mode, transposes
        and storage, preferred entries first.  This is what replaces the reference's tuned look-up table
        (sparta/specializer/kernels/matmul.py:246-264): a configuration names a prebuilt tile."""
        code = _lib.DTYPE_CODE[self._sample_dtype if dtype is None else dtype]
        shapes: Dict[Any, int] = {}
        for e in _lib.tile_table(_OP_CODE[self._mode], code):
            # sdd against a dense B stored [K, N] reaches the tcgen05 kernel (which wants B stored [N, K])
            # through a transposed copy of B made by the launch closure, see update_func
            b_ok = e.trans_b in (-1, int(self._transpose_B)) or \
                (self._mode == 'sdd' and e.impl == _lib.IMPL_TCGEN05 and e.trans_b == 1)
            if e.trans_a not in (-1, int(self._transpose_A)) or not b_ok:
                continue
            if e.compressed not in (-1, int(self._compressed)):
                continue
            shapes.setdefault((e.block_m, e.block_k, e.block_n), e.impl)
        return shapes

    def set_parameter(self, name: str, value: Any):
        if name == '_family':
            assert value in _FAMILY, f'unknown kernel family {value}'
            self._family = value
            return
        super().set_parameter(name, value)

    def set_parameters(self, params: Dict[str, Any]):
        super().set_parameters(params)
        port = self.ports[self._sparse_port]
        if self._bcs_mode == 'BCSR':
            self.set_parameter('BCSR', True)
            self.set_parameter('BCSC', False)
        else:
            self.set_parameter('BCSR', port.BCSR)
            self.set_parameter('BCSC', True)
        port.set_block_size(self.get_parameter(self._sparse_block_H),
                            self.get_parameter(self._sparse_block_W))

    def set_shape(self, batch_size: int, M: int, K: int, N: int):
        self.set_parameter('BATCH_SIZE', batch_size)
        self.set_parameter('GLOBAL_M_VALUE', M)
        self.set_parameter('GLOBAL_K_VALUE', K)
        self.set_parameter('GLOBAL_N_VALUE', N)

    def get_shape(self):
        return tuple(self.get_parameter(n) for n in
                     ['BATCH_SIZE', 'GLOBAL_M_VALUE', 'GLOBAL_K_VALUE', 'GLOBAL_N_VALUE'])

    def get_block_shape(self):
        return tuple(self.get_parameter(f'BLOCK_SIZE_{d}_VALUE') for d in 'MKN')

    def _check_parameters(self, params: Dict[str, Any]):
        for d in 'MKN':
            key = f'BLOCK_SIZE_{d}_VALUE'
            size = params.get(key, self._parameters[key].value if key in self._parameters else None)
            assert size is not None, f'{key} is required'
        _, M, K, N = self.get_shape()
        for d, total in zip('MKN', (M, K, N)):
            size = params.get(f'BLOCK_SIZE_{d}_VALUE', self._parameters[f'BLOCK_SIZE_{d}_VALUE'].value)
            if total is not None:
                assert total % size == 0, f'{d} = {total} is not a multiple of the tile size {size}'

    def update_func(self):
        batch_size, M, K, N = self.get_shape()
        BM, BK, BN = self.get_block_shape()
        port = self.ports[self._sparse_port]
        mode, biased, compressed = self._mode, self._biased, self._compressed
        trans_a, trans_b = self._transpose_A, self._transpose_B
        entry = getattr(_lib.lib(), _ENTRY[mode])
        impl = _FAMILY[self._family]
        by_row = self._bcs_mode == 'BCSR'
        via_transposed_b = (mode == 'sdd' and not trans_b and compressed and (BM, BK, BN) == (32, 32, 128)
                            and self._family != 'simt')

        cache = {}

        def matmul_func(A: torch.Tensor, B: torch.Tensor, bias: torch.Tensor = None):
            _lib.require_cuda(A, B, bias)
            idx = port.indexes
            assert idx is not None, 'the sparse port has no mask'
            assert A.dtype == B.dtype, 'A and B must share a dtype'
            A = A.contiguous()
            B = B.contiguous()
            # sdd with B stored [K, N] on a tcgen05 tile: the kernel reads its dense operand with the reduction
            # dimension contiguous, so B is transposed first -- one extra pass over B (in attention: over V,
            # which is small beside the probabilities); the FMA kernels take B as it is
            b_transposed = via_transposed_b and A.dtype in (torch.float16, torch.bfloat16)
            if b_transposed:
                B = B.transpose(1, 2).contiguous()
            batch = A.shape[0]
            stride = idx.val_stride_blocks
            if mode == 'dds' and compressed:
                C = torch.empty((batch, stride * BM * BN), dtype=A.dtype, device=A.device)
            else:
                C = torch.empty((batch, M, N), dtype=A.dtype, device=A.device)
            if mode == 'dds' and compressed and stride == 0:
                return C
            if by_row:
                ptr_t, idx_t, is64 = idx.row_ptr, idx.bcsr_buf, False
            else:
                ptr_t, idx_t, is64 = idx.col_ptr, idx.bcsc_buf, idx.BCSR
            if idx.batched:
                assert idx.n_masks == batch, 'per-batch masks need one mask per batch element'
            key = (ptr_t.data_ptr(), idx_t.data_ptr(), idx.nnz_dev.data_ptr(), stride, idx.capacity, batch, A.dtype)
            args = cache.get('args') if cache.get('key') == key else None
            if args is None:  # everything but the data pointers is fixed until the indexes, batch or dtype change
                args = _lib.BsmmArgs(
                    ptr=ptr_t.data_ptr(), idx=idx_t.data_ptr(), nnz=idx.nnz_dev.data_ptr(),
                    batch=batch, M=M, K=K, N=N, BM=BM, BK=BK, BN=BN,
                    trans_a=int(trans_a), trans_b=int(trans_b or b_transposed), compressed=int(compressed),
                    idx_is_64=int(is64), dtype=_lib.dtype_code(A), impl=impl,
                    n_index_sets=idx.n_masks if idx.batched else 1,
                    ptr_stride=ptr_t.shape[-1], idx_stride=idx.capacity,
                    val_stride_blocks=stride if compressed else 0,
                    grid_blocks_hint=idx.capacity if idx.batched else max(stride, 1),
                )
                cache['key'], cache['args'] = key, args
            args.A, args.B, args.C = A.data_ptr(), B.data_ptr(), C.data_ptr()
            args.bias = _lib.ptr(bias.contiguous()) if biased else None
            if A.device.index == torch.cuda.current_device():
                _lib.check(entry(args, _lib.stream_ptr(A.device)), _ENTRY[mode])
            else:
                with torch.cuda.device(A.device):
                    _lib.check(entry(args, _lib.stream_ptr(A.device)), _ENTRY[mode])
            return C

        self._func = matmul_func

    def _convert_data(self, inputs, outputs):
        if self._mode == 'sdd':
            inputs[0] = inputs[0] * self.ports['A'].mask
        elif self._mode == 'dsd':
            inputs[1] = inputs[1] * self.ports['B'].mask
        for i in range(len(inputs)):
            inputs[i] = inputs[i].detach()
        outputs[0] = outputs[0].detach()
        if self._compressed:
            indexes = self.ports[self._sparse_port].indexes
            if self._sparse_port == 'A':
                inputs[0] = indexes.convert(inputs[0])
            elif self._sparse_port == 'B':
                inputs[1] = indexes.convert(inputs[1])
            else:
                outputs[0] = indexes.convert(outputs[0])

    def reference(self, *args):
        """Masked-dense einsum; a dds output is multiplied by the block coverage of the mask, not by
        the element mask (matmul.py:211-227)."""
        A, B = args[0], args[1]
        if self._mode == 'sdd':
            A = A * self.ports['A'].mask
        elif self._mode == 'dsd':
            B = B * self.ports['B'].mask
        a = 'bkm' if self._transpose_A else 'bmk'
        b = 'bnk' if self._transpose_B else 'bkn'
        C = torch.einsum(f'{a}, {b} -> bmn', A, B)
        if self._biased:
            C = C + args[2].unsqueeze(1)
        if self._mode == 'dds':
            if self.ready:
                C = C * self.ports['C'].indexes.get_mask()
            else:
                C = C * self.ports['C'].mask
        return C


class SparTASparseMatMulKernel(SparseMatMulKernel):
    """Free tile sizes.  Where the reference searches 16/32/64 per dimension and compiles each point
    (matmul.py:230-264), the search space here is read from the library's tile table for the dtype of
    the sample inputs: every FMA tile (8 .. 64 per dimension, which includes the reference's choices, so
    its saved configurations still build) plus the tcgen05 tiles that exist for this mode, e.g.
    128 x 32 x 32 for the SparseLinear weight layout in fp16 / bf16.  A grid walk visits the product of
    the per-dimension choices; combinations that are no table entry fail ``_check_parameters`` and count
    as infinitely slow, like invalid points in the reference.  THREAD_SIZE_* keys of reference
    configurations are accepted and ignored: the prebuilt kernels fix their own thread tiling."""

    __algo__ = 'sparta'

    def _add_parameters(self):
        super()._add_parameters()
        for dim in 'MKN':
            self._add_parameter(f'BLOCK_SIZE_{dim}_VALUE', is_tunable=True,
                                search_space=TunableItemCfg('choice', [8, 16, 32, 64]))
            self._add_parameter(f'THREAD_SIZE_{dim}_VALUE')

    def set_sample_dtype(self, dtype: torch.dtype):
        super().set_sample_dtype(dtype)
        shapes = list(self.tile_shapes())
        for k, dim in enumerate('MKN'):
            choices = sorted({shape[k] for shape in shapes})
            self._parameters[f'BLOCK_SIZE_{dim}_VALUE'].search_space = TunableItemCfg('choice', choices)

    def _check_parameters(self, params: Dict[str, Any]):
        super()._check_parameters(params)
        tile = tuple(params[f'BLOCK_SIZE_{d}_VALUE'] for d in 'MKN')
        known = any(tile in self.tile_shapes(dtype) for dtype in _lib.DTYPE_CODE)
        assert known, f'no prebuilt kernel for tile {tile[0]} x {tile[1]} x {tile[2]} in this layout'


class OpenAISparseMatMulKernel(SparseMatMulKernel):
    """Fixed 32 x 64 x 32 tile (matmul.py:297-331).  Kept as a configuration name; it runs the same
    prebuilt kernels with that tile."""

    __algo__ = 'openai'

    def _add_parameters(self):
        super()._add_parameters()
        for dim, size in zip('MKN', (32, 64, 32)):
            self._add_parameter(f'BLOCK_SIZE_{dim}_VALUE', value=size, is_tunable=True,
                                search_space=TunableItemCfg('choice', [size]))

    def _check_parameters(self, params: Dict[str, Any]):
        for dim, size in zip('MKN', (32, 64, 32)):
            key = f'BLOCK_SIZE_{dim}_VALUE'
            if key in params:
                assert params[key] == size
        super()._check_parameters({**{f'BLOCK_SIZE_{d}_VALUE': s for d, s in zip('MKN', (32, 64, 32))},
                                   **params})
