"""Sharding of the block-sparse operators across the GPUs of one box.

The path has no exchange step: attention shards by batch x head (the leading dimension of
``[B*H, N, E]`` tensors), SparseLinear by token rows; masks, indexes and weights are replicated, every
rank builds its indexes locally.  The only collective offered is an optional all-gather of the
outputs: as a separate pass (NCCL over NVLink through ``torch.distributed``; gloo works for CPU tests), or,
for the fused attention kernel, folded into the kernel itself: ``GatheredHeads`` holds the full output in
symmetric memory and the kernel stores every tile into the peers' buffers as it finishes it.  The
reference has no multi-GPU code; this module is an extension.
"""
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total: int, world_size: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous ``[begin, end)`` of ``total`` units owned by ``rank``.

    Units are dealt out in groups of ``multiple`` (e.g. the block height for token rows, so that a
    shard never cuts a block row); earlier ranks take the remainder groups.  Raises ``ValueError`` when
    ``total`` is not a multiple of ``multiple`` or a rank would be left without work.
    """
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f'bad rank {rank} for world size {world_size}')
    if multiple < 1 or total % multiple:
        raise ValueError(f'{total} units cannot be split in groups of {multiple}')
    groups = total // multiple
    if groups < world_size:
        raise ValueError(f'{groups} groups of {multiple} units cannot feed {world_size} ranks')
    base, extra = divmod(groups, world_size)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * multiple, end * multiple


def shard_heads(*tensors: torch.Tensor, world_size: int, rank: int):
    """Slices of ``[B*H, N, E]`` tensors along the batch x head dimension for this rank."""
    lo, hi = shard_bounds(tensors[0].shape[0], world_size, rank)
    out = tuple(t[lo:hi] for t in tensors)
    return out if len(out) > 1 else out[0]


def shard_rows(x: torch.Tensor, world_size: int, rank: int, block_rows: int = 1) -> torch.Tensor:
    """Token-row slice of a ``[tokens, features]`` activation; ``block_rows`` keeps shards aligned to
    the row tile of the kernel (and to the block height of an output mask)."""
    lo, hi = shard_bounds(x.shape[0], world_size, rank, block_rows)
    return x[lo:hi]


def shard_row_mask(mask: torch.Tensor, world_size: int, rank: int, block_rows: int) -> torch.Tensor:
    """The rows of an input / output mask ``[tokens, features]`` that belong to this rank's tokens."""
    lo, hi = shard_bounds(mask.shape[0], world_size, rank, block_rows)
    return mask[lo:hi].contiguous()


def all_gather_outputs(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Concatenate the ranks' outputs along dimension 0 (every rank gets the full tensor).

    Shards may differ in size along dimension 0 by one group; equal shards use a single
    ``all_gather_into_tensor``, into ``out`` when the caller provides the full-size buffer (no allocation
    per call).
    """
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    local = local.contiguous()
    sizes = torch.zeros(world, dtype=torch.int64, device=local.device)
    sizes[dist.get_rank(group)] = local.shape[0]
    dist.all_reduce(sizes, group=group)
    sizes = sizes.tolist()
    if len(set(sizes)) == 1:
        shape = (world * sizes[0],) + local.shape[1:]
        if out is None:
            out = torch.empty(shape, dtype=local.dtype, device=local.device)
        assert tuple(out.shape) == shape and out.dtype == local.dtype and out.is_contiguous()
        dist.all_gather_into_tensor(out, local, group=group)
        return out
    # uneven shards: pad to the largest, gather once, drop the padding
    most = max(sizes)
    padded = torch.zeros((most,) + local.shape[1:], dtype=local.dtype, device=local.device)
    padded[:local.shape[0]] = local
    out = torch.empty((world * most,) + local.shape[1:], dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[r * most:r * most + n] for r, n in enumerate(sizes)], dim=0)


class GatheredHeads(object):
    """The all-gathered output ``[world * heads, N, E]`` of head-sharded attention, one copy per rank in
    symmetric memory (``torch.distributed._symmetric_memory``: every rank's buffer is mapped into every
    other rank's address space, NVLink peer access).

    ``local`` is this rank's slice of its own buffer (pass it as the kernel's output); ``peer_addresses`` are
    the device addresses of the same slice in every other rank's buffer (pass them as the kernel's copies:
    ``SparseAttention.forward_gathered``).  ``wait()`` completes the exchange: this rank's stores are done
    when its kernel is, and a barrier tells every rank that all the others are done too; after it ``full``
    holds all heads on every rank.  Equal shards only.
    """

    def __init__(self, heads_per_rank: int, n: int, e: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = dist.group.WORLD if group is None else group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.shape = (self.world * heads_per_rank, n, e)
        self.full = symm_mem.empty(self.shape, dtype=dtype, device=device)
        self._handle = symm_mem.rendezvous(self.full, self.group)
        lo, hi = self.rank * heads_per_rank, (self.rank + 1) * heads_per_rank
        self.local = self.full[lo:hi]
        offset = lo * n * e * self.full.element_size()
        self.peer_addresses: List[int] = [int(self._handle.buffer_ptrs[r]) + offset
                                          for r in range(self.world) if r != self.rank]

    def wait(self):
        torch.cuda.current_stream(self.full.device).synchronize()
        dist.barrier(group=self.group)
        return self.full
