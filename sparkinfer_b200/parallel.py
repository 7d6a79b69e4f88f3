"""Tensor-parallel sharding of the block-scaled linears across the GPUs of one node.

The reference's GEMM is single-GPU; sharding is the serving stack's job. Two modes exist and
both keep the per-GPU work a plain call into the ops of this package:

* column-parallel: the weight and its scales are split along N (whole 128-row blocks), every
  rank holds the full activation and writes its ``[M, N/g]`` slab. No communication.
* row-parallel: K is split (whole 128-column blocks); each rank quantizes its slice of the
  activation with the *same* caller-supplied global scale, multiplies, and the BF16 partial
  outputs are summed with one all-reduce: :class:`PeerAllReduce` (this package's own kernel
  over NVLink peer memory) on GPUs, or ``torch.distributed`` (NCCL; gloo in CPU tests).

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


def slab_rows(rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Rows ``[begin, end)`` of the output that ``rank`` sums and broadcasts in
    :class:`PeerAllReduce` (the split the kernel uses: ``rows * rank // world_size``)."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return rows * rank // world_size, rows * (rank + 1) // world_size


class PeerAllReduce:
    """All-reduce of the row-parallel partial outputs by this package's own kernels over peer
    memory, in two forms.

    *Plain* (``scatter=False``): the GEMM writes its whole ``[rows, cols]`` partial into
    :attr:`partial`; calling the object sums all ranks' partials in place
    (``b12x_b200_allreduce_peer``: pull the own slab from every rank, add, push to every rank),
    and :attr:`result` is :attr:`partial`.

    *Fused with the GEMM* (``scatter=True``, ``rows % (256 * world) == 0``): :meth:`gemm` runs the
    CTA-pair GEMM with its output tiles scattered to the owners of their row slabs while the
    main loop runs (``b12x_b200_gemm_blockscaled_scatter``), so that the call only adds the
    local slots and pushes the result slab (``b12x_b200_allreduce_peer_scattered``) into
    :attr:`result`, a second buffer.

    Buffers live in symmetric memory (every rank of the node maps every other rank's). When the
    call's kernel has finished on this rank's stream, :attr:`result` holds the full sum,
    bit-identical on every rank. Collective: every rank constructs it and calls it the same
    number of times. One rank per GPU."""

    def __init__(self, rows: int, cols: int, dtype: torch.dtype = torch.bfloat16, group=None,
                 device: torch.device | None = None, scatter: bool = False):
        import torch.distributed._symmetric_memory as symm_mem

        from ._lib import launch

        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("PeerAllReduce needs an initialised process group")
        if dtype not in (torch.bfloat16, torch.float16):
            raise ValueError(f"partials must be bf16/fp16, got {dtype}")
        if cols % 8 != 0:
            raise ValueError(f"cols={cols} must be a multiple of 8")
        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world_size > 8:
            raise ValueError("at most 8 ranks (one NVLink node)")
        if scatter and rows % (256 * self.world_size) != 0:
            raise ValueError(f"scatter needs rows={rows} to be a multiple of 256 * world")
        self.scatter = bool(scatter)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.rows, self.cols, self.dtype = int(rows), int(cols), dtype
        self.partial = symm_mem.empty((self.rows, self.cols), dtype=dtype, device=self.device)
        self._signal = symm_mem.empty((launch.allreduce_peer_signal_bytes() // 4,),
                                      dtype=torch.int32, device=self.device)
        self._signal.zero_()
        self._handles = [symm_mem.rendezvous(self.partial, group),
                         symm_mem.rendezvous(self._signal, group)]
        self.buffer_ptrs = [int(p) for p in self._handles[0].buffer_ptrs]
        self.signal_ptrs = [int(p) for p in self._handles[1].buffer_ptrs]
        self.result = self.partial
        self.output_ptrs = None
        if self.scatter:
            self.result = symm_mem.empty((self.rows, self.cols), dtype=dtype, device=self.device)
            self._handles.append(symm_mem.rendezvous(self.result, group))
            self.output_ptrs = [int(p) for p in self._handles[2].buffer_ptrs]
        # Every rank's signal block is zero before any rank can send a flag into it.
        torch.cuda.synchronize(self.device)
        dist.barrier(group)

    def gemm(self, kind: int, a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor,
             sfb: torch.Tensor, alpha: torch.Tensor | None, k: int,
             stream: object | None = None) -> None:
        """This rank's partial GEMM ``[rows, K_local] x [cols, K_local]^T`` with the output
        scattered to the slab owners (``scatter=True`` only)."""
        from ._lib import launch

        if not self.scatter:
            raise RuntimeError("gemm() belongs to the scatter form; write into .partial instead")
        launch.gemm_blockscaled_scatter(kind, a, sfa, b, sfb, self.buffer_ptrs, self.rank,
                                        self.dtype, alpha, self.rows, self.cols, k,
                                        stream_int=launch.cuda_stream_to_int(stream))

    def __call__(self, stream: object | None = None) -> torch.Tensor:
        from ._lib import launch

        launch.allreduce_peer(self.buffer_ptrs, self.signal_ptrs, self.rank, self.dtype, self.rows,
                              self.cols, self.cols, self.device, output_ptrs=self.output_ptrs,
                              stream_int=launch.cuda_stream_to_int(stream))
        return self.result


def gather_columns(slab: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenate the ``[M, N/g]`` slabs of a column-parallel linear along N (not on the timed
    path; equal slab widths)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return slab
    parts = [torch.empty_like(slab) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, slab.contiguous(), group=group)
    return torch.cat(parts, dim=1)


__all__ = ["Shard", "shard_range", "column_parallel_weight", "row_parallel_slices",
           "all_reduce_partials", "gather_columns", "slab_rows", "PeerAllReduce"]
