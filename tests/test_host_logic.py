"""Host-side logic that needs no GPU: search spaces, connections, tuner trial counts, config schema.
Mirrors test/unit/test_search_space.py and test/unit/test_tuners.py of the reference (those run on
CUDA tensors only because the reference allocates everything there)."""
import random
import sys
from typing import Any, Dict, List, Optional

import pytest
import torch

from sparta_b200.nn import tune, SparseLinear, SparseBatchMatMul, SparseSoftmax, SparseAttention
from sparta_b200.nn.module_tuner import GridSearchTuner, RandomSearchTuner
from sparta_b200.common.tuning import TunableItemCfg
from sparta_b200.specializer.funtional import SparseBatchMatMulCtx


@pytest.mark.parametrize('mode', ['sdd', 'dsd', 'dds'])
@pytest.mark.parametrize('trans_A', [False, True])
@pytest.mark.parametrize('trans_B', [False, True])
@pytest.mark.parametrize('compressed', [False, True])
@pytest.mark.parametrize('backward', [False, True])
def test_sparse_matmul_search_space(mode, compressed, trans_A, trans_B, backward):
    mask = torch.zeros((64, 64))
    sparse_tensor = {'sdd': 'A', 'dsd': 'B', 'dds': 'C'}[mode]
    op = SparseBatchMatMul(**{f'{sparse_tensor}_mask': mask}, transpose_A=trans_A, transpose_B=trans_B,
                           compressed=compressed)
    space = op.get_search_space(backward=backward)
    kernel_names = ['forward:C'] + (['backward:A', 'backward:B'] if backward else [])
    params = {f'BLOCK_SIZE_{d}_VALUE' for d in 'MKN'}
    assert set(space.keys()) == set(kernel_names)
    for kernel_space in space.values():
        assert set(kernel_space.keys()) == {'sparta', 'openai'}
        assert set(kernel_space['sparta'].keys()) == params
        assert set(kernel_space['openai'].keys()) == params
    connections = op.get_connections(backward=backward)
    assert len(connections) == (2 if compressed and backward else 0)


def test_backward_kernel_modes_follow_the_tensors():
    # dsd(tB) forward (SparseLinear with a weight mask): dA = dC W is dsd(nn); dW = dC^T A is dds(tA)
    ctx = SparseBatchMatMulCtx('dsd', False, True, True, True)
    k = {n: p.possible_kernels['sparta'] for n, p in ctx.get_kernel_placeholders(True).items()}
    assert (k['forward:C']._mode, k['forward:C']._transpose_A, k['forward:C']._transpose_B) == ('dsd', False, True)
    assert (k['backward:A']._mode, k['backward:A']._transpose_A, k['backward:A']._transpose_B) == ('dsd', False, False)
    assert (k['backward:B']._mode, k['backward:B']._transpose_A, k['backward:B']._transpose_B) == ('dds', True, False)
    # attention qk: dds(tB) => dQ = dS K : sdd(nn); dK = dS^T Q : sdd(tA)
    ctx = SparseBatchMatMulCtx('dds', False, True, False, True)
    k = {n: p.possible_kernels['sparta'] for n, p in ctx.get_kernel_placeholders(True).items()}
    assert (k['backward:A']._mode, k['backward:A']._transpose_A, k['backward:A']._transpose_B) == ('sdd', False, False)
    assert (k['backward:B']._mode, k['backward:B']._transpose_A, k['backward:B']._transpose_B) == ('sdd', True, False)


def _count_trials(module, sample_inputs: List[torch.Tensor], sample_grads: Optional[List[torch.Tensor]] = None):
    def debug_func(idx: int, params: Dict[Any, Any]):
        debug_func.count += 1
        return random.random()
    debug_func.count = 0
    try:
        tune(module=module, sample_inputs=sample_inputs, sample_grads=sample_grads, algo='grid',
             max_trials=sys.maxsize, backward_weight=0 if sample_grads is None else 0.5, verbose=False,
             debug_func=debug_func)
    except AssertionError:
        pass
    return debug_func.count


@pytest.mark.parametrize('backward', [False, True])
def test_tune_sparse_linear_trial_count(backward):
    dense = torch.nn.Linear(128, 128)
    x = torch.zeros((128, 128))
    g = torch.zeros((128, 128))
    op = SparseLinear(dense, weight_mask=torch.ones((128, 128), dtype=torch.uint8))
    count = _count_trials(op, [x], [g] if backward else None)
    assert count == (4 * 4 * 4 + 1) * (3 if backward else 1)


@pytest.mark.parametrize('backward', [False, True])
def test_tune_sparse_matmul_trial_count(backward):
    A = torch.zeros((4, 128, 128))
    B = torch.zeros((4, 128, 128))
    g = torch.zeros((4, 128, 128))
    op = SparseBatchMatMul(C_mask=torch.ones((128, 128), dtype=torch.uint8), transpose_B=True, compressed=True)
    count = _count_trials(op, [A, B], [g] if backward else None)
    assert count == (4 * 4 * 4 + 1) * (3 if backward else 1)


@pytest.mark.parametrize('backward', [False, True])
def test_tune_sparse_softmax_trial_count(backward):
    x = torch.zeros((128, 128))
    g = torch.zeros((128, 128))
    op = SparseSoftmax(mask=torch.ones((128, 128), dtype=torch.uint8), temperature=128, compressed=True)
    count = _count_trials(op, [x], [g] if backward else None)
    assert count == (5 * 4 * 5) * (2 if backward else 1)


@pytest.mark.parametrize('backward', [False, True])
def test_tune_sparse_attention_trial_count(backward):
    torch.manual_seed(2022)
    q, k, v, g = (torch.rand((1, 128, 128)) for _ in range(4))
    op = SparseAttention(mask=torch.ones((128, 128), dtype=torch.uint8))
    count = _count_trials(op, [q, k, v], [g] if backward else None)
    if backward:
        assert count == (4 * 3 * 4 + 1) * 6 + (4 * 3 * 5) * 2
    else:
        assert count == (4 * 3 * 4 + 1) * 2 + (4 * 3 * 5) * 1


def test_search_space_follows_the_tile_table():
    """The tunable block sizes are the library's prebuilt tiles for the sample dtype: fp32 sees the FMA tiles
    only; fp16 on the SparseLinear weight layout also sees the 128 x 32 x 32 tcgen05 tile, and a
    configuration saved by the reference (16 / 32 / 64) still passes the parameter check."""
    from sparta_b200 import _lib
    op = SparseLinear(torch.nn.Linear(256, 256), weight_mask=torch.ones((256, 256), dtype=torch.uint8))
    op.set_sample_inputs([torch.zeros((256, 256))])
    space = op.get_search_space()['forward:C']['sparta']
    assert [space[f'BLOCK_SIZE_{d}_VALUE']._value for d in 'MKN'] == [[8, 16, 32, 64]] * 3
    op.set_sample_inputs([torch.zeros((256, 256), dtype=torch.float16)])
    space = op.get_search_space()['forward:C']['sparta']
    assert space['BLOCK_SIZE_M_VALUE']._value == [8, 16, 32, 64, 128]
    assert space['BLOCK_SIZE_K_VALUE']._value == [8, 16, 32, 64]
    kernel = op.get_kernel_placeholders()['forward:C'].possible_kernels['sparta']
    assert kernel.tile_shapes()[(128, 32, 32)] == _lib.IMPL_TCGEN05
    assert next(iter(kernel.tile_shapes())) == (128, 32, 32)  # preferred entries come first
    kernel._check_parameters({f'BLOCK_SIZE_{d}_VALUE': v for d, v in zip('MKN', (128, 32, 32))})
    kernel._check_parameters({f'BLOCK_SIZE_{d}_VALUE': v for d, v in zip('MKN', (64, 16, 32))})
    with pytest.raises(AssertionError):
        kernel._check_parameters({f'BLOCK_SIZE_{d}_VALUE': v for d, v in zip('MKN', (128, 64, 32))})
    # the two gradients of that operator have tcgen05 tiles too: dsd with B stored [K, N], dds with A stored [K, M]
    bwd = op.get_kernel_placeholders(True)['backward:A'].possible_kernels['sparta']
    assert bwd.tile_shapes(torch.float16)[(128, 32, 32)] == _lib.IMPL_TCGEN05
    bwd = op.get_kernel_placeholders(True)['backward:B'].possible_kernels['sparta']
    assert bwd.tile_shapes(torch.float16)[(32, 64, 32)] == _lib.IMPL_TCGEN05
    # sdd: against a dense B stored [N, K], and (through a transposed copy made by the launch closure) [K, N]
    from sparta_b200.specializer.kernels import SparTASparseMatMulKernel
    sdd = lambda tb: SparTASparseMatMulKernel(mode='sdd', biased=False, transpose_A=False, transpose_B=tb)
    assert sdd(True).tile_shapes(torch.float16)[(32, 32, 128)] == _lib.IMPL_TCGEN05
    assert sdd(False).tile_shapes(torch.float16)[(32, 32, 128)] == _lib.IMPL_TCGEN05
    assert all(impl == _lib.IMPL_SIMT for impl in sdd(False).tile_shapes(torch.float32).values())


def test_grid_and_random_walkers():
    space = {'a': TunableItemCfg('choice', [1, 2, 3]), 'b': TunableItemCfg('choice', [10, 20])}
    seen = []
    t = GridSearchTuner(space, lambda i, c: seen.append((c['a'], c['b'])) or c['a'] * c['b'])
    t.tune()
    assert seen == [(1, 10), (1, 20), (2, 10), (2, 20), (3, 10), (3, 20)]
    assert t.best_config == {'a': 1, 'b': 10}
    calls = []
    RandomSearchTuner(space, lambda i, c: calls.append(c) or 0.0, max_trials=4).tune()
    assert len(calls) == 4
    empty = []
    GridSearchTuner({}, lambda i, c: empty.append(c) or 0.0).tune()
    assert empty == [{}]


def test_operator_argument_errors():
    dense = torch.nn.Linear(64, 64)
    m = torch.ones((64, 64), dtype=torch.uint8)
    with pytest.raises(ValueError):
        SparseLinear(dense)
    with pytest.raises(ValueError):
        SparseLinear(torch.nn.Bilinear(4, 4, 4), weight_mask=m)
    op = SparseLinear(dense, weight_mask=m)
    with pytest.raises(ValueError):
        op.update_mask(input_mask=m, weight_mask=m)
    with pytest.raises(AssertionError):
        op.update_mask(weight_mask=torch.ones((32, 64), dtype=torch.uint8))
    with pytest.raises(ValueError):
        SparseBatchMatMul()
    with pytest.warns(UserWarning):
        y = op(torch.zeros((8, 64)))  # not built: dense path with a warning
    assert y.shape == (8, 64)


def test_tunable_item_cfg():
    cfg = TunableItemCfg('choice', _is_nested=True, _value={
        'openai': {}, 'sparta': {'BM': TunableItemCfg('choice', [32, 64])}})
    assert cfg.to_nni_search_space() == {'_type': 'choice', '_value': [
        {'_name': 'openai'}, {'_name': 'sparta', 'BM': {'_type': 'choice', '_value': [32, 64]}}]}
    assert TunableItemCfg('choice', [1, 2]).includes(2) and not cfg.includes(2)
