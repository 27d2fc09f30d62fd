"""Kernel objects: a parameter table, a search space and a launch closure over prebuilt CUDA kernels.

Host-side mirror of ``sparta/specializer/kernels/kernel_base.py`` (``PortConfig`` :37-80,
``KernelBase`` :83-220).  ``compile()`` renders no template and runs no nvcc: it validates the
parameters against the prebuilt tile table and binds a closure that calls the C-ABI library.
"""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, Callable, Dict, List, Optional

import torch

from sparta_b200.common.tuning import TunableItemCfg
from sparta_b200.tesa import get_bcs_function, BCSIndexes
from sparta_b200.testing import profile


@dataclasses.dataclass
class _Parameter:
    name: str
    value: Optional[Any] = None
    is_tunable: bool = False
    is_dynamic: bool = False
    search_space: Optional[TunableItemCfg] = None

    def __post_init__(self):
        if self.search_space is not None:
            assert self.is_tunable


@dataclasses.dataclass
class PortConfig(object):
    """One tensor port of a kernel.  A sparse port owns the mask, the block size and the index set
    built from them; ports of several kernels can be merged with ``connect`` so that one index set
    serves all of them."""
    name: str
    is_input: bool
    is_sparse: bool = False
    BCSR: bool = False
    BCSC: bool = False

    def __post_init__(self):
        self.mask: Optional[torch.Tensor] = None
        self._block_H: int = 0
        self._block_W: int = 0
        self.indexes: Optional[BCSIndexes] = None
        self.capacity: Optional[int] = None  # index entries kept per mask (None: every block)

    def set_sparse(self, BCSR: bool, BCSC: bool):
        self.is_sparse = True
        self.BCSR = BCSR
        self.BCSC = BCSC

    def set_block_size(self, block_H: int, block_W: int):
        if self.is_sparse and (block_H != self._block_H or block_W != self._block_W):
            self._block_H = block_H
            self._block_W = block_W
            self._update_indexes()

    def set_mask(self, mask: torch.Tensor):
        if self.is_sparse:
            self.mask = mask
            self._update_indexes()

    def refresh(self):
        """Rebuild the indexes from the current contents of the mask tensor (one kernel launch, no
        host synchronisation): the per-call conversion used for dynamic sparsity."""
        self._update_indexes()

    def _update_indexes(self):
        if self._block_H > 0 and self._block_W > 0 and self.mask is not None:
            self.indexes = get_bcs_function(
                self._block_H, self._block_W, self.BCSR, self.BCSC,
            ).build_indexes(self.mask, self.capacity)

    def connect(self, kernel: 'KernelBase', port_name: str):
        other = kernel.ports[port_name]
        assert self.is_sparse == other.is_sparse
        self.BCSR |= other.BCSR
        self.BCSC |= other.BCSC
        kernel.ports[port_name] = self


class KernelBase(Callable):

    def __init__(self):
        self._parameters: Dict[str, _Parameter] = {}
        self._func: Optional[Callable] = None
        self.ports: Dict[str, PortConfig] = {}
        self.ready = False
        self._add_parameters()
        self._set_ports()

    @abc.abstractmethod
    def _set_ports(self):
        """Create the input / output ports."""

    @abc.abstractmethod
    def _add_parameters(self):
        """Register the kernel's parameters."""

    def _add_parameter(self, name: str, value: Any = None, is_tunable: bool = False,
                       is_dynamic: bool = False, search_space: Optional[TunableItemCfg] = None):
        self._parameters[name] = _Parameter(name, value, is_tunable, is_dynamic, search_space)

    def set_search_space(self, search_space: Dict[str, TunableItemCfg]):
        for name, space in search_space.items():
            self._parameters[name].search_space = space

    def get_search_space(self, fixed_params: Optional[Dict[str, Any]] = None):
        """Tunable parameters and their choices; ``None`` when ``fixed_params`` cannot be met."""
        space = {n: p.search_space for n, p in self._parameters.items() if p.is_tunable}
        for name, value in (fixed_params or {}).items():
            if name not in self._parameters:
                return None
            param = self._parameters[name]
            if param.is_tunable:
                if not param.search_space.includes(value):
                    return None
                space[name] = TunableItemCfg('choice', [value])
            elif param.value is not None and param.value != value:
                return None
        return space

    def set_parameter(self, name: str, value: Any):
        if name not in self._parameters and name in ['_name', '_impl']:
            return
        self._parameters[name].value = value

    def set_parameters(self, params: Dict[str, Any]):
        for name, value in params.items():
            self.set_parameter(name, value)

    def get_parameter(self, name: str):
        return self._parameters[name].value

    def get_parameters(self, names: Optional[List[str]] = None):
        if names is None:
            return {k: v.value for k, v in self._parameters.items()}
        return {k: self._parameters[k].value for k in names}

    @abc.abstractmethod
    def set_shape(self, *args, **kwargs):
        """Set the problem shape."""

    @abc.abstractmethod
    def _check_parameters(self, params: Dict[str, Any]):
        """Raise AssertionError when ``params`` is not a usable configuration."""

    @abc.abstractmethod
    def update_func(self):
        """(Re)bind the launch closure to the current indexes and shape."""

    def compile(self, params: Dict[str, Any]):
        self._check_parameters(params)
        self.set_parameters(params)
        self.update_func()
        self.ready = True

    @abc.abstractmethod
    def reference(self, *args) -> Any:
        """Dense reference; inputs and outputs are dense tensors."""

    @abc.abstractmethod
    def _convert_data(self, inputs: List[torch.Tensor], outputs: List[torch.Tensor]):
        """Mask and, if needed, compress sample inputs / target outputs in place."""

    def test(self, inputs: List[torch.Tensor], num_warmups: int = 10, num_iters: int = 10,
             cuda: bool = True):
        """Check against the dense reference, then time; inputs are dense tensors."""
        sparse_inputs = [x for x in inputs]
        targets = self.reference(*sparse_inputs)
        if type(targets) is not tuple:
            targets = (targets, )
        targets = [y for y in targets]
        self._convert_data(sparse_inputs, targets)
        half = any(isinstance(x, torch.Tensor) and x.dtype in (torch.float16, torch.bfloat16)
                   for x in sparse_inputs)
        tol = dict(atol=2e-2, rtol=2e-2) if half else dict(atol=1e-4, rtol=1e-8)
        return profile(self, sparse_inputs, targets, num_warmups, num_iters, cuda, **tol)

    def __call__(self, *args) -> torch.Tensor:
        if self.ready:
            return self._func(*args)
        raise ValueError('The kernel is not compiled.')
