"""Kernel slots and the per-operator context that owns them.

An operator has a few kernel *slots* (``forward:C``, ``backward:A``, ...).  Each slot holds one prebuilt
kernel object per implementation name; ``select_impls`` picks one per slot and decides which sparse
ports share an index set.  The public names and call signatures are those of
sparta/specializer/funtional/sparse_ctx_base.py (``KernelPlaceholder`` :12-67, ``SparseCtxBase`` :70-157),
which the tuner and the operators of this package rely on; there is no JIT step behind them here.
"""
import abc
from typing import Any, Dict, Iterable, List, Optional, Type

import torch

from sparta_b200.specializer.kernels import KernelBase, PortConfig


def _is_forward(slot_name: str) -> bool:
    return slot_name.startswith('forward')


class KernelPlaceholder(object):
    """A slot that one of several kernel implementations can fill.

    ``port_map`` names the slot's sparse tensor twice: by the operator's name for it (key) and by the
    kernel's own port name (value) -- the forward ``B`` of a linear layer sits at port ``A`` or ``C`` of
    its backward kernels.  ``connectable`` says whether that port may share indexes with other slots
    (true for compressed storage, where the value order is defined by the index order).
    """

    def __init__(self, name: str, impls: Dict[str, Type[KernelBase]], args: Dict[str, Any],
                 port_map: Dict[str, str], connectable: bool):
        self.name = name
        self.port_map = dict(port_map)
        self.connectable = connectable
        self.possible_kernels: Dict[str, KernelBase] = {impl: cls(**args) for impl, cls in impls.items()}
        self.sample_inputs: List[Any] = []
        self.ready = False
        self._chosen: Optional[str] = None

    # -- which kernel --------------------------------------------------------------------------
    @property
    def dense_func(self):
        """Dense reference computation of this slot (the same for every implementation)."""
        return next(iter(self.possible_kernels.values())).reference

    def select_impl(self, impl: str):
        self._chosen = impl

    def active_kernel(self) -> Optional[KernelBase]:
        return self.possible_kernels.get(self._chosen) if self._chosen is not None else None

    def _targets(self) -> Iterable[KernelBase]:
        chosen = self.active_kernel()
        return self.possible_kernels.values() if chosen is None else (chosen,)

    # -- forwarding to the kernel(s) -------------------------------------------------------------
    def set_shape(self, *args, **kwargs):
        for kernel in self._targets():
            kernel.set_shape(*args, **kwargs)

    def update_func(self):
        self.active_kernel().update_func()

    def build(self, config: Dict[str, Any]):
        self.active_kernel().compile(config)
        self.ready = True

    def get_search_space(self, fixed_params: Optional[Dict[str, Any]] = None):
        """``{implementation: {parameter: choices}}`` for the implementations that can honour
        ``fixed_params``."""
        found = ((impl, kernel.get_search_space(fixed_params)) for impl, kernel in self.possible_kernels.items())
        return {impl: space for impl, space in found if space is not None}

    def set_sample_inputs(self, sample_inputs: List[torch.Tensor]):
        self.sample_inputs = [t.detach() if type(t) is torch.Tensor else t for t in sample_inputs]
        # the prebuilt tile shapes depend on the element type: tell every candidate kernel
        dtype = next((t.dtype for t in self.sample_inputs if type(t) is torch.Tensor), None)
        if dtype is not None:
            for kernel in self.possible_kernels.values():
                if hasattr(kernel, 'set_sample_dtype'):
                    kernel.set_sample_dtype(dtype)

    def test(self, num_warmups: int = 10, num_iters: int = 10, cuda: bool = True):
        return self.active_kernel().test(self.sample_inputs, num_warmups, num_iters, cuda)


class SparseCtxBase(object):
    """Owns the slots of one operator and the list of sparse ports per operator-level tensor name."""

    def __init__(self):
        self._kernels: Dict[str, KernelPlaceholder] = {}
        self.sparse_ports: Dict[str, List[PortConfig]] = {}

    def _slots(self, backward: bool) -> Dict[str, KernelPlaceholder]:
        return {name: slot for name, slot in self._kernels.items() if backward or _is_forward(name)}

    def _init_sparse_ports(self, port_names: List[str]):
        """Before any implementation is chosen a mask must reach every candidate kernel."""
        self.sparse_ports = {}
        for tensor in port_names:
            self.sparse_ports[tensor] = [kernel.ports[slot.port_map[tensor]]
                                         for slot in self._kernels.values()
                                         for kernel in slot.possible_kernels.values()]

    def select_impls(self, impls: Dict[str, str]):
        """Activate one implementation per slot.  Connectable ports of the chosen kernels that stand for
        the same tensor are merged into one ``PortConfig`` (one mask, one index set, the union of the
        index forms the kernels need); the others stay separate."""
        separate: Dict[str, List[PortConfig]] = {tensor: [] for tensor in self.sparse_ports}
        shared: Dict[str, PortConfig] = {}
        for slot_name, impl in impls.items():
            slot = self._kernels[slot_name]
            slot.select_impl(impl)
            kernel = slot.active_kernel()
            for tensor, local in slot.port_map.items():
                if not slot.connectable:
                    separate[tensor].append(kernel.ports[local])
                elif tensor in shared:
                    shared[tensor].connect(kernel, local)
                else:
                    shared[tensor] = kernel.ports[local]
        for tensor, port in shared.items():
            separate[tensor].append(port)
        self.sparse_ports = separate

    def update_func(self):
        for slot in self._kernels.values():
            if slot.ready and slot.active_kernel() is not None:
                slot.update_func()

    def build(self, config: Dict[str, Dict[str, Any]]):
        for slot_name, params in config.items():
            self._kernels[slot_name].build(params)

    def get_sparse_indexes(self, port_name: str):
        ports = self.sparse_ports.get(port_name) or []
        return ports[0].indexes if ports else None

    def get_kernel_placeholders(self, backward: bool = False):
        return self._slots(backward)

    def get_search_space(self, backward: bool = False):
        return {name: slot.get_search_space() for name, slot in self._slots(backward).items()}

    @abc.abstractmethod
    def set_shape(self, *args, **kwargs):
        """Set the problem shape on every kernel."""

    @abc.abstractmethod
    def set_sample_inputs(self, sample_inputs: List[torch.Tensor],
                          sample_grads: Optional[List[torch.Tensor]] = None):
        """Distribute sample tensors to the kernel slots (for tuning)."""

    @abc.abstractmethod
    def get_connections(self, backward: bool = False) -> List[Dict[str, str]]:
        """Parameters that must agree across kernels."""

    @abc.abstractmethod
    def dense_forward(self, *args) -> Any:
        """Dense computation of the same operator (keeps autograd)."""
