"""Base types of tensor-with-sparsity-attribute indexes (mirrors sparta/tesa/tesa_base.py:12-42)."""
import abc
from typing import Any

import torch


class TeSAIndexes(object):
    """Holds the mask an index set was built from and the context that built it."""

    def __init__(self, function_context: 'TeSAFunctionContext', mask: torch.Tensor):
        self.raw_mask = mask
        self.device = mask.device
        self.function_context = function_context

    @abc.abstractmethod
    def get_mask(self) -> torch.Tensor:
        """The mask actually applied (block coverage of the raw mask)."""


class TeSAFunctionContext(object):

    @abc.abstractmethod
    def build_indexes(self, mask: torch.Tensor, *args) -> TeSAIndexes:
        """Build index tensors from a dense mask."""

    @abc.abstractmethod
    def convert(self, dense: torch.Tensor, *args) -> torch.Tensor:
        """Dense tensor -> compressed values."""

    @abc.abstractmethod
    def inverse(self, sparse_val: torch.Tensor, *args) -> torch.Tensor:
        """Compressed values -> dense tensor."""
