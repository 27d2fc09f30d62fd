"""``sparta.nn.tune`` / ``sparta.nn.build`` (host-side mirror of sparta/nn/module_tuner.py:105-413).

The search has the reference's two levels -- an upper space over the block sizes that connected
kernels must share, and a lower space per kernel slot and implementation -- and the same grid /
random walkers, so trial counts and the returned ``{module_path: {kernel: {param: value}}}``
dictionaries match.  What differs is the cost of a trial: a configuration names a prebuilt tile
shape, so ``kernel.build`` is a table lookup instead of an nvcc run.
"""
import logging
import random
import sys
import warnings
from typing import Any, Callable, Dict, Iterator, List, Optional

import numpy as np
import torch

from sparta_b200.common.tuning import TunableItemCfg
from sparta_b200.specializer import OperatorBase

_logger = logging.Logger(__name__)
_logger.addHandler(logging.StreamHandler())


class Tuner(object):
    """Walks ``search_space`` and keeps the configuration with the smallest ``eval_func`` value."""

    def __init__(self, search_space: Dict[Any, TunableItemCfg],
                 eval_func: Callable[[int, Dict[Any, Any]], float], max_trials: int = sys.maxsize):
        self._search_space = search_space
        self._eval_func = eval_func
        space_size = int(np.prod([len(space._value) for space in search_space.values()]))
        self._max_trials = min(max_trials, space_size)
        self.best_result = np.inf
        self.best_config = None

    def next_config(self) -> Iterator[Dict[str, Any]]:
        raise NotImplementedError

    def tune(self):
        for i, config in zip(range(self._max_trials), self.next_config()):
            result = self._eval_func(i, config)
            if result < self.best_result:
                self.best_result = result
                self.best_config = config


class RandomSearchTuner(Tuner):

    def next_config(self):
        while True:
            yield {name: random.choice(space._value) for name, space in self._search_space.items()}


class GridSearchTuner(Tuner):

    def next_config(self):
        names = list(self._search_space.keys())
        sizes = [len(self._search_space[n]._value) for n in names]
        total = int(np.prod(sizes)) if names else 1
        for flat in range(total):
            config, rest = {}, flat
            for name, size in zip(reversed(names), reversed(sizes)):  # last parameter varies fastest
                config[name] = self._search_space[name]._value[rest % size]
                rest //= size
            yield {name: config[name] for name in names}


def tune_sparse_module(module: OperatorBase, name: str, sample_inputs: List[torch.Tensor],
                       sample_grads: Optional[List[torch.Tensor]] = None, algo: str = 'grid',
                       max_trials: int = sys.maxsize, backward_weight: float = 0,
                       debug_func: Optional[Callable[[int, Dict[Any, Any]], float]] = None):
    if algo.startswith('grid'):
        tuner_type = GridSearchTuner
    elif algo.startswith('rand'):
        tuner_type = RandomSearchTuner
    else:
        raise ValueError(f'unsupported tuner algorithm "{algo}"')

    with_backward = backward_weight > 0
    module.set_sample_inputs(sample_inputs, sample_grads)
    search_space = module.get_search_space(with_backward)
    connections = module.get_connections(with_backward)

    # upper space: for every connection, the values all connected kernels can take
    upper_choices = []
    for connection in connections:
        per_kernel = []
        for kernel_name, param_name in connection.items():
            values = set()
            for impl_space in search_space[kernel_name].values():
                values |= set(impl_space[param_name]._value)
            per_kernel.append(values)
        upper_choices.append(set.intersection(*per_kernel))
    upper_size = int(np.prod([len(c) for c in upper_choices]))
    upper_space = {i: TunableItemCfg('choice', list(c)) for i, c in enumerate(upper_choices)}

    lower_cache = {}

    def lower_search(upper_idx: int, upper_params: Dict[Any, Any]):
        _logger.info(f'[{name}][Upper Search Space] #{upper_idx}: {list(upper_params.values())}')
        chosen, total_latency = {}, 0
        for kernel_name, kernel in module.get_kernel_placeholders(with_backward).items():
            _logger.info(f'[{name}][Kernel: {kernel_name}]')
            trials = int(np.ceil(max_trials / upper_size))
            best_params, best_latency = None, np.inf
            weight = backward_weight if kernel_name.startswith('backward') else 1
            fixed = {connections[i][kernel_name]: val for i, val in upper_params.items()}
            for impl, space in kernel.get_search_space(fixed).items():
                kernel.select_impl(impl)

                def try_params(lower_idx: int, params: Dict[Any, Any]):
                    try:
                        kernel.build(params)
                        latency = kernel.test()
                    except AssertionError:
                        latency = np.inf
                    _logger.info(f'{impl} #{lower_idx}: {list(params.values())} => {latency} ms')
                    return latency

                walker = tuner_type(space, try_params if debug_func is None else debug_func, trials)
                walker.tune()
                if walker.best_result < best_latency:
                    best_params = dict(_impl=impl, **walker.best_config)
                    best_latency = walker.best_result
            chosen[kernel_name] = best_params
            total_latency += best_latency * weight
        lower_cache[str(upper_params)] = chosen
        return total_latency

    tuner = tuner_type(upper_space, lower_search, upper_size)
    tuner.tune()
    _logger.info(f'[{name}] Tuning completed.')
    if debug_func is None:
        if tuner.best_config is None:
            _logger.warning(f'[{name}] All trials failed.')
            return None
        best_config = lower_cache[str(tuner.best_config)]
        _logger.info(f'[{name}] Best config:\n{best_config}')
        module.build(best_config, sample_inputs)
        return best_config


def tune_combined_module(module: torch.nn.Module, sample_inputs: List[torch.Tensor],
                         sample_grads: Optional[List[torch.Tensor]] = None, algo: str = 'grid',
                         max_trials: int = sys.maxsize, backward_weight: float = 0,
                         verbose: bool = False, debug_func: Optional[Callable] = None):
    """Tune and build every sparse operator found in ``module`` (which may itself be one).

    Inputs (and gradients when ``backward_weight > 0``) of each sparse child are captured with
    hooks during one dense pass; each child is then tuned on its own.  Returns the best configuration
    per operator, keyed ``'root'`` or ``'root/<child>/...'``.
    """
    captured_inputs = {'root': sample_inputs}
    captured_grads = {'root': sample_grads}
    handles = []

    def hook(op: OperatorBase, name: str):
        handles.append(op.register_forward_hook(get_input_hook(captured_inputs, name)))
        handles.append(op.register_full_backward_hook(get_grad_hook(captured_grads, name)))

    iter_sparse_modules(module, 'root', hook)
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        if backward_weight > 0:
            for x in sample_inputs:
                x.requires_grad = True
        outputs = module.forward(*sample_inputs)
        if backward_weight > 0:
            if type(outputs) is not tuple:
                outputs = (outputs, )
            for output, grad in zip(outputs, sample_grads):
                if type(output) is torch.Tensor:
                    output.backward(grad)
            for x in sample_inputs:
                x.requires_grad = False
    for h in handles:
        h.remove()

    _logger.setLevel(logging.DEBUG if verbose else logging.WARNING)
    best_configs = {}

    def tune_one(op: OperatorBase, name: str):
        best_configs[name] = tune_sparse_module(
            module=op, name=name, sample_inputs=captured_inputs[name],
            sample_grads=captured_grads.get(name), algo=algo, max_trials=max_trials,
            backward_weight=backward_weight, debug_func=debug_func,
        )

    iter_sparse_modules(module, 'root', tune_one)
    return best_configs


def build_combined_module(module: torch.nn.Module, sample_inputs: List[torch.Tensor],
                          configs: Dict[str, Dict[str, Any]]):
    """Build every sparse operator in ``module`` with the configuration stored under its path."""
    captured_inputs = {'root': sample_inputs}
    handles = []
    iter_sparse_modules(module, 'root', lambda op, name: handles.append(
        op.register_forward_hook(get_input_hook(captured_inputs, name))))
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        module.forward(*sample_inputs)
    for h in handles:
        h.remove()
    iter_sparse_modules(module, 'root', lambda op, name: op.build(configs[name], sample_inputs=captured_inputs[name]))


def iter_sparse_modules(module: torch.nn.Module, module_name: str,
                        func: Callable[[OperatorBase, str], None]):
    if isinstance(module, OperatorBase):
        func(module, module_name)
        return
    for child_name, child in module.named_children():
        iter_sparse_modules(child, f'{module_name}/{child_name}', func)


def get_input_hook(input_dict: Dict[str, List], module_name: str):
    def input_hook(module, fea_in, fea_out):
        input_dict[module_name] = list(fea_in)
    return input_hook


def get_grad_hook(grad_dict: Dict[str, List], module_name: str):
    def grad_hook(module, grad_input, grad_output):
        grad_dict[module_name] = list(grad_output)
    return grad_hook
