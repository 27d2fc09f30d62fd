"""Sparse contexts own the kernel objects of one operator (forward and backward) and route masks
to their sparse ports (host-side mirror of sparta/specializer/funtional/sparse_ctx_base.py)."""
import abc
from typing import Any, Dict, List, Optional, Type

import torch

from sparta_b200.specializer.kernels import KernelBase, PortConfig


class KernelPlaceholder(object):
    """A slot (e.g. ``forward:C``) that can be filled by one of several kernel implementations."""

    def __init__(self, name: str, impls: Dict[str, Type[KernelBase]], args: Dict[str, Any],
                 port_map: Dict[str, str], connectable: bool):
        self.name = name
        self.possible_kernels = {key: impl(**args) for key, impl in impls.items()}
        self.port_map = port_map
        self.connectable = connectable
        self._active_impl: Optional[str] = None
        self.sample_inputs: List[torch.Tensor] = []
        self.dense_func = next(iter(self.possible_kernels.values())).reference
        self.ready = False

    def set_shape(self, *args, **kwargs):
        kernels = self.possible_kernels.values() if self._active_impl is None else [self.active_kernel()]
        for kernel in kernels:
            kernel.set_shape(*args, **kwargs)

    def select_impl(self, impl: str):
        self._active_impl = impl

    def active_kernel(self) -> Optional[KernelBase]:
        return None if self._active_impl is None else self.possible_kernels[self._active_impl]

    def update_func(self):
        self.active_kernel().update_func()

    def build(self, config: Dict[str, Any]):
        self.active_kernel().compile(config)
        self.ready = True

    def get_search_space(self, fixed_params: Optional[Dict[str, Any]] = None):
        spaces = {}
        for impl, kernel in self.possible_kernels.items():
            space = kernel.get_search_space(fixed_params)
            if space is not None:
                spaces[impl] = space
        return spaces

    def set_sample_inputs(self, sample_inputs: List[torch.Tensor]):
        self.sample_inputs = [x.detach() if type(x) is torch.Tensor else x for x in sample_inputs]
        # the prebuilt tile shapes depend on the element type: tell every candidate kernel
        dtype = next((x.dtype for x in self.sample_inputs if type(x) is torch.Tensor), None)
        for kernel in self.possible_kernels.values():
            if dtype is not None and hasattr(kernel, 'set_sample_dtype'):
                kernel.set_sample_dtype(dtype)

    def test(self, num_warmups: int = 10, num_iters: int = 10, cuda: bool = True):
        return self.active_kernel().test(self.sample_inputs, num_warmups, num_iters, cuda)


class SparseCtxBase(object):

    def __init__(self):
        self._kernels: Dict[str, KernelPlaceholder] = {}
        self.sparse_ports: Dict[str, List[PortConfig]] = {}

    def _init_sparse_ports(self, port_names: List[str]):
        self.sparse_ports = {
            port_name: [
                kernel.ports[placeholder.port_map[port_name]]
                for placeholder in self._kernels.values()
                for kernel in placeholder.possible_kernels.values()
            ]
            for port_name in port_names
        }

    @abc.abstractmethod
    def set_shape(self, *args, **kwargs):
        """Set the problem shape on every kernel."""

    def select_impls(self, impls: Dict[str, str]):
        """Activate one implementation per kernel slot; with compressed tensors the sparse ports of
        the chosen kernels are merged so that forward and backward share one index set."""
        merged: Dict[str, PortConfig] = {}
        self.sparse_ports = {name: [] for name in self.sparse_ports.keys()}
        for kernel_name, impl in impls.items():
            placeholder = self._kernels[kernel_name]
            placeholder.select_impl(impl)
            kernel = placeholder.active_kernel()
            for global_name, local_name in placeholder.port_map.items():
                if placeholder.connectable:
                    if global_name in merged:
                        merged[global_name].connect(kernel, local_name)
                    else:
                        merged[global_name] = kernel.ports[local_name]
                else:
                    self.sparse_ports[global_name].append(kernel.ports[local_name])
        for global_name, port in merged.items():
            self.sparse_ports[global_name].append(port)

    def update_func(self):
        for placeholder in self._kernels.values():
            if placeholder.active_kernel() is not None and placeholder.ready:
                placeholder.update_func()

    def build(self, config: Dict[str, Dict[str, Any]]):
        for kernel_name, kernel_config in config.items():
            self._kernels[kernel_name].build(kernel_config)

    def get_sparse_indexes(self, port_name: str):
        if port_name in self.sparse_ports and len(self.sparse_ports[port_name]) > 0:
            return self.sparse_ports[port_name][0].indexes
        return None

    def get_kernel_placeholders(self, backward: bool = False):
        return {name: k for name, k in self._kernels.items() if backward or name.startswith('forward')}

    @abc.abstractmethod
    def set_sample_inputs(self, sample_inputs: List[torch.Tensor],
                          sample_grads: Optional[List[torch.Tensor]] = None):
        """Distribute sample tensors to the kernel slots (for tuning)."""

    @abc.abstractmethod
    def get_connections(self, backward: bool = False) -> List[Dict[str, str]]:
        """Parameters that must agree across kernels."""

    def get_search_space(self, backward: bool = False):
        return {name: k.get_search_space() for name, k in self._kernels.items()
                if backward or name.startswith('forward')}

    @abc.abstractmethod
    def dense_forward(self, *args) -> Any:
        """Dense computation of the same operator (keeps autograd)."""
