"""Kernel objects: a parameter table, a search space and a launch closure over prebuilt CUDA kernels.

Host-side mirror of ``sparta/specializer/kernels/kernel_base.py`` (``PortConfig`` :37-80,
``KernelBase`` :83-220).  ``compile()`` renders no template and runs no nvcc: it validates the
parameters against the prebuilt tile table and binds a closure that calls the C-ABI library.
"""
from __future__ import annotations

import abc
from typing import Any, Callable, Dict, List, Optional

import torch

from sparta_b200.common.tuning import TunableItemCfg
from sparta_b200.tesa import get_bcs_function, BCSIndexes
from sparta_b200.testing import profile


class _ParameterTable(object):
    """Name -> value table of a kernel with the choices of the tunable entries.  The names are the
    configuration schema shared with the reference (``BLOCK_SIZE_M_VALUE`` ...): a configuration saved
    by either implementation can be handed to ``compile``."""

    __slots__ = ('_values', '_spaces', '_dynamic')

    def __init__(self):
        self._values: Dict[str, Any] = {}
        self._spaces: Dict[str, TunableItemCfg] = {}  # present <=> the parameter is tunable
        self._dynamic: set = set()

    def add(self, name: str, value: Any = None, space: Optional[TunableItemCfg] = None, dynamic: bool = False):
        self._values[name] = value
        if space is not None:
            self._spaces[name] = space
        if dynamic:
            self._dynamic.add(name)

    def __contains__(self, name: str) -> bool:
        return name in self._values

    def __getitem__(self, name: str) -> '_ParameterView':
        return _ParameterView(self, name)

    def items(self):
        return ((name, _ParameterView(self, name)) for name in self._values)

    def keys(self):
        return self._values.keys()


class _ParameterView(object):
    """One row of the table (``value``, ``is_tunable``, ``search_space``)."""

    __slots__ = ('_table', 'name')

    def __init__(self, table: _ParameterTable, name: str):
        if name not in table._values:
            raise KeyError(name)
        self._table, self.name = table, name

    @property
    def value(self):
        return self._table._values[self.name]

    @value.setter
    def value(self, v):
        self._table._values[self.name] = v

    @property
    def is_tunable(self) -> bool:
        return self.name in self._table._spaces

    @property
    def is_dynamic(self) -> bool:
        return self.name in self._table._dynamic

    @property
    def search_space(self) -> Optional[TunableItemCfg]:
        return self._table._spaces.get(self.name)

    @search_space.setter
    def search_space(self, space: TunableItemCfg):
        self._table._spaces[self.name] = space


class PortConfig(object):
    """One tensor port of a kernel (interface of sparta/specializer/kernels/kernel_base.py:37-80).

    A sparse port owns what defines an index set -- the mask tensor, the block shape, which index forms
    are wanted -- and the ``indexes`` built from them on the GPU.  ``connect`` makes another kernel's port
    an alias of this one, so several kernels (forward and backward, or the three operators of an
    attention layer) read one index set; the wanted forms are OR-ed.
    """

    def __init__(self, name: str, is_input: bool, is_sparse: bool = False, BCSR: bool = False, BCSC: bool = False):
        self.name = name
        self.is_input = is_input
        self.is_sparse = is_sparse
        self.BCSR = BCSR
        self.BCSC = BCSC
        self.mask: Optional[torch.Tensor] = None
        self.indexes: Optional[BCSIndexes] = None
        self.capacity: Optional[int] = None  # index entries kept per mask (None: every block)
        self._block = (0, 0)

    def set_sparse(self, BCSR: bool, BCSC: bool):
        self.is_sparse, self.BCSR, self.BCSC = True, BCSR, BCSC

    def set_block_size(self, block_H: int, block_W: int):
        if self.is_sparse and (block_H, block_W) != self._block:
            self._block = (block_H, block_W)
            self.refresh()

    def set_mask(self, mask: torch.Tensor):
        if self.is_sparse:
            self.mask = mask
            self.refresh()

    def refresh(self):
        """(Re)build the indexes from the current contents of the mask tensor: one kernel launch, no
        host synchronisation.  Operators in dynamic mode call this at the start of every forward."""
        block_H, block_W = self._block
        if self.mask is None or block_H <= 0 or block_W <= 0:
            return
        builder = get_bcs_function(block_H, block_W, self.BCSR, self.BCSC)
        self.indexes = builder.build_indexes(self.mask, self.capacity)

    def connect(self, kernel: 'KernelBase', port_name: str):
        other = kernel.ports[port_name]
        assert self.is_sparse == other.is_sparse
        self.BCSR = self.BCSR or other.BCSR
        self.BCSC = self.BCSC or other.BCSC
        kernel.ports[port_name] = self


class KernelBase(Callable):

    def __init__(self):
        self._parameters = _ParameterTable()
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
        assert search_space is None or is_tunable
        if is_tunable and search_space is None:
            search_space = TunableItemCfg('choice', [] if value is None else [value])
        self._parameters.add(name, value, search_space, is_dynamic)

    def set_search_space(self, search_space: Dict[str, TunableItemCfg]):
        for name, space in search_space.items():
            self._parameters[name].search_space = space

    def get_search_space(self, fixed_params: Optional[Dict[str, Any]] = None):
        """Choices of the tunable parameters, narrowed to ``fixed_params``; ``None`` when this kernel
        cannot honour them (unknown name, value outside the choices, or a conflicting constant)."""
        space = {name: row.search_space for name, row in self._parameters.items() if row.is_tunable}
        for name, wanted in (fixed_params or {}).items():
            if name not in self._parameters:
                return None
            row = self._parameters[name]
            if row.is_tunable:
                if not row.search_space.includes(wanted):
                    return None
                space[name] = TunableItemCfg('choice', [wanted])
            elif row.value is not None and row.value != wanted:
                return None
        return space

    def set_parameter(self, name: str, value: Any):
        if name in ('_name', '_impl') and name not in self._parameters:
            return  # bookkeeping keys of configuration dictionaries
        self._parameters[name].value = value

    def set_parameters(self, params: Dict[str, Any]):
        for name, value in params.items():
            self.set_parameter(name, value)

    def get_parameter(self, name: str):
        return self._parameters[name].value

    def get_parameters(self, names: Optional[List[str]] = None):
        wanted = self._parameters.keys() if names is None else names
        return {name: self._parameters[name].value for name in wanted}

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
