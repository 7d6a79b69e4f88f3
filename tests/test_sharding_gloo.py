"""The N > 1 path on CPU: two gloo ranks run the column-parallel and row-parallel sharding of
sparkinfer_b200.parallel with the oracle standing in for the device GEMM (the collective
plumbing and the shard arithmetic are what is under test here)."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import blockscaled_oracle as O
from sparkinfer_b200.parallel import (
    Shard,
    all_reduce_partials,
    column_parallel_weight,
    gather_columns,
    row_parallel_slices,
    shard_range,
)


def test_shard_range_is_a_partition_in_whole_blocks():
    for total, world in [(18432, 8), (18432, 4), (7168, 8), (2304, 2), (640, 3)]:
        shards = [shard_range(total, world, r) for r in range(world)]
        assert shards[0].begin == 0 and shards[-1].end == total
        for a, b in zip(shards, shards[1:]):
            assert a.end == b.begin
        assert all(s.size % 128 == 0 and s.size > 0 for s in shards)
        assert max(s.size for s in shards) - min(s.size for s in shards) <= 128
    assert shard_range(18432, 8, 3) == Shard(rank=3, world_size=8, begin=6912, end=9216)
    with pytest.raises(ValueError):
        shard_range(1000, 2, 0)
    with pytest.raises(ValueError):
        shard_range(256, 4, 0)
    with pytest.raises(ValueError):
        shard_range(256, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _seeded(seed, shape, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen) * scale).to(torch.bfloat16)


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 32, 512, 1024
        x = _seeded(4042, (m, k))
        w = _seeded(4043, (n, k), 0.02)

        # ---- column-parallel block-FP8 (configuration 3): N split, no collective on the path
        a_codes, a_scale = O.quantize_block_fp8(x.float().numpy(), 1)
        b_codes, b_scale = O.quantize_block_fp8(w.float().numpy(), 128)
        shard = shard_range(n, world, rank)
        wb, sb = column_parallel_weight(torch.from_numpy(b_codes), torch.from_numpy(b_scale), shard)
        assert wb.shape == (n // world, k) and sb.shape == (n // world // 128, k // 128)
        slab = O.gemm_block_fp8(a_codes, a_scale, wb.numpy(), sb.numpy())
        full = gather_columns(torch.from_numpy(slab))
        want = O.gemm_block_fp8(a_codes, a_scale, b_codes, b_scale)
        col_ok = bool(np.array_equal(full.numpy(), want))

        # ---- row-parallel NVFP4 (configuration 4): K split, same global scale on every rank,
        # BF16 partials summed by one all-reduce
        gsx, gsw = O.nvfp4_global_scale(x.float().numpy()), O.nvfp4_global_scale(w.float().numpy())
        kshard = shard_range(k, world, rank)
        xs, ws = row_parallel_slices(x, w, kshard)
        px, sx = O.quantize_nvfp4_rows(xs.float().numpy(), gsx)
        pw, sw = O.quantize_nvfp4_rows(ws.float().numpy(), gsw)
        # The bytes of a K-slice do not depend on the number of ranks.
        px_full, sx_full = O.quantize_nvfp4_rows(x.float().numpy(), gsx)
        slice_ok = bool(
            np.array_equal(px, px_full[:, kshard.begin // 2:kshard.end // 2])
            and np.array_equal(sx, sx_full[:, kshard.begin // 16:kshard.end // 16]))
        partial = torch.from_numpy(O.gemm_nvfp4(px, sx, gsx, pw, sw, gsw)).to(torch.bfloat16)
        reduced = all_reduce_partials(partial.float()).numpy()  # gloo sums FP32 copies of BF16
        pw_full, sw_full = O.quantize_nvfp4_rows(w.float().numpy(), gsw)
        ref = O.gemm_nvfp4(px_full, sx_full, gsx, pw_full, sw_full, gsw)
        err = float(np.abs(reduced - ref).max())
        row_ok = err <= 1e-2 * float(np.abs(ref).max())
        results[rank] = (col_ok, slice_ok, row_ok, err)
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_on_two_gloo_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    for rank in range(world):
        col_ok, slice_ok, row_ok, err = results[rank]
        assert col_ok, "gathered column-parallel slabs differ from the unsharded product"
        assert slice_ok, "a K-slice quantized differently from the same columns of the full tensor"
        assert row_ok, f"row-parallel sum off by {err}"


def test_slab_rows_partition_the_output_like_the_kernel():
    """`slab_rows` mirrors the kernel's split (rows * rank // world): contiguous, complete,
    non-overlapping, also when the world does not divide the rows."""
    from sparkinfer_b200.parallel import slab_rows

    for rows, world in [(4096, 2), (4096, 8), (203, 3), (5, 8), (0, 4)]:
        edges = [slab_rows(rows, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert all(b <= e for b, e in edges)
    import pytest

    with pytest.raises(ValueError):
        slab_rows(16, 2, 2)
