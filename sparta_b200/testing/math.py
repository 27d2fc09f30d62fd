"""Dense reference formulas the sparse operators are checked against
(API of sparta/testing/math.py:8-79); plain torch, any device."""
from typing import Optional

import numpy as np
import torch


def sparse_softmax_forward_reference(x: torch.Tensor, mask: torch.Tensor,
                                     temperature: float = 1.) -> torch.Tensor:
    """Softmax over the last axis that skips masked positions; rows without any unmasked position
    come out as zeros."""
    shifted = x - x.max(dim=-1, keepdim=True).values
    weights = torch.exp(shifted / temperature) * mask
    return weights / (weights.sum(dim=-1, keepdim=True) + 1e-10)


def sparse_softmax_backward_reference(grad: torch.Tensor, output: torch.Tensor, mask: torch.Tensor,
                                      temperature: float = 1.) -> torch.Tensor:
    """Gradient of the masked softmax with respect to its input (zero at masked positions)."""
    y = output * mask
    gy = grad * y
    return (gy - y * gy.sum(dim=-1, keepdim=True)) / temperature


def sparse_multi_head_attention_reference(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                                          mask: torch.Tensor, temperature: Optional[float] = None) -> torch.Tensor:
    """softmax_mask(Q K^T / T) V with T = sqrt(E) unless given.  Shapes (..., N_target, E),
    (..., N_source, E), (..., N_source, E), mask (N_target, N_source)."""
    if temperature is None or np.isnan(temperature):
        temperature = float(np.sqrt(query.shape[-1]))
    scores = torch.matmul(query, key.transpose(-1, -2))
    probs = sparse_softmax_forward_reference(scores, mask, temperature)
    return torch.matmul(probs, value)
