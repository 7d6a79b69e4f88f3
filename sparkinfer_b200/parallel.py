"""Tensor-parallel sharding of the block-scaled linears across the GPUs of one node.

The reference's GEMM is single-GPU; sharding is the serving stack's job. Two modes exist and
both keep the per-GPU work a plain call into the ops of this package:

* column-parallel: the weight and its scales are split along N (whole 128-row blocks), every
  rank holds the full activation and writes its ``[M, N/g]`` slab. No communication.
* row-parallel: K is split (whole 128-column blocks); each rank quantizes its slice of the
  activation with the *same* caller-supplied global scale, multiplies, and the BF16 partial
  outputs are summed with one all-reduce (NCCL over NVLink on GPUs, gloo in CPU tests).

One process per GPU, ``torch.distributed`` for the plumbing.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    """Half-open range ``[begin, end)`` of one rank along the sharded dimension."""

    rank: int
    world_size: int
    begin: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.begin


def shard_range(total: int, world_size: int, rank: int, *, multiple: int = 128) -> Shard:
    """Contiguous, ``multiple``-aligned split of ``total``; earlier ranks take the remainder
    blocks. Raises when ``total`` is not a multiple of ``multiple`` or a rank would be empty."""
    if total % multiple != 0:
        raise ValueError(f"sharded dimension {total} must be a multiple of {multiple}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    blocks = total // multiple
    if blocks < world_size:
        raise ValueError(f"cannot split {blocks} blocks of {multiple} over {world_size} ranks")
    base, extra = divmod(blocks, world_size)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return Shard(rank=rank, world_size=world_size, begin=begin * multiple, end=end * multiple)


def column_parallel_weight(weight: torch.Tensor, block_scale: torch.Tensor | None,
                           shard: Shard) -> tuple[torch.Tensor, torch.Tensor | None]:
    """Rows ``[begin, end)`` of ``weight [N, K]`` and the matching rows of its 128x128 block
    scales ``[N/128, K/128]``."""
    w = weight[shard.begin:shard.end].contiguous()
    s = None if block_scale is None else block_scale[shard.begin // 128:shard.end // 128].contiguous()
    return w, s


def row_parallel_slices(activation: torch.Tensor, weight: torch.Tensor,
                        shard: Shard) -> tuple[torch.Tensor, torch.Tensor]:
    """Columns ``[begin, end)`` of both ``activation [M, K]`` and ``weight [N, K]``."""
    return (activation[:, shard.begin:shard.end].contiguous(),
            weight[:, shard.begin:shard.end].contiguous())


def all_reduce_partials(partial: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the per-rank partial outputs in place (BF16 on the wire, as the path specifies)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def gather_columns(slab: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate the ``[M, N/g]`` slabs of a column-parallel linear along N (not on the timed
    path; equal slab widths)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return slab
    parts = [torch.empty_like(slab) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, slab.contiguous(), group=group)
    return torch.cat(parts, dim=1)


__all__ = ["Shard", "shard_range", "column_parallel_weight", "row_parallel_slices",
           "all_reduce_partials", "gather_columns"]
