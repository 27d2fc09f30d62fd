"""Mask generators (API of sparta/testing/mask.py:9-60)."""
from typing import Any, Optional, Tuple

import torch


def block_mask(
    shape: Tuple[int, int],
    block: Tuple[int, int] = (1, 1),
    sparsity: float = 0.99,
    algo: str = 'rand',
    device: Any = 'cuda',
    generator: Optional[torch.Generator] = None,
) -> torch.Tensor:
    """Random 2-D uint8 mask whose ``block``-sized tiles are all-one or all-zero.

    ``sparsity`` is the probability that a tile is dropped.  ``generator`` (an addition to the
    reference signature) makes the draw reproducible across devices: with a CPU generator the mask is
    drawn on the CPU and then moved to ``device``.
    """
    assert len(shape) == 2 and len(block) == 2, 'only 2D mask is supported'
    assert shape[0] % block[0] == 0, f'invalid block shape {block}'
    assert shape[1] % block[1] == 0, f'invalid block shape {block}'
    if algo != 'rand':
        raise ValueError(f'unsupported mask generator: {algo}')
    coarse_shape = (shape[0] // block[0], shape[1] // block[1])
    draw_device = generator.device if generator is not None else device
    coarse = (torch.rand(coarse_shape, device=draw_device, generator=generator) > sparsity).to(torch.uint8)
    full = coarse.repeat_interleave(block[0], 0).repeat_interleave(block[1], 1)
    return full.to(device).contiguous()


def band_global_random_mask(n_target: int, n_source: int, block: int = 64, band: int = 8,
                            extra: float = 0.05, seed: int = 0, device: Any = 'cuda') -> torch.Tensor:
    """Attention mask used by the benchmark: ``band`` blocks either side of the diagonal, the first
    block row and block column (global tokens) and a fraction ``extra`` of random blocks."""
    rows, cols = n_target // block, n_source // block
    i = torch.arange(rows).unsqueeze(1)
    j = torch.arange(cols).unsqueeze(0)
    keep = ((i - j).abs() <= band) | (i == 0) | (j == 0)
    g = torch.Generator().manual_seed(seed)
    keep |= torch.rand((rows, cols), generator=g) < extra
    full = keep.to(torch.uint8).repeat_interleave(block, 0).repeat_interleave(block, 1)
    return full.to(device).contiguous()
