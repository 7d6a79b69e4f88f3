"""The all-reduce kernel of the row-parallel (K-split) step, rehearsed on one GPU.

On hardware every rank runs the kernel on its own GPU and the ranks wait for each other's flags
over NVLink. Kernels that wait on each other must not be separate launches on one GPU, so these
tests use the entry point's rehearsal mode (rank = -1): all ranks run inside one cooperative
grid, every "peer" buffer is an ordinary local allocation, and the flag protocol, the slab split
and the arithmetic are exactly those of the multi-GPU call. `bench.py --gpus N` checks the real
thing (each rank compares the summed output with the oracle of the unsharded problem).

The reference leaves this step to `torch.distributed.all_reduce`; the expected value here is the
same sum: FP32 accumulation of the 2-byte partials in rank order, rounded once.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda", 0)


def _signals(world):
    from sparkinfer_b200._lib import launch

    words = launch.allreduce_peer_signal_bytes() // 4
    return [torch.zeros(words, dtype=torch.int32, device=DEV) for _ in range(world)]


def _expected(partials, cols):
    acc = torch.zeros(partials[0][:, :cols].shape, dtype=torch.float32, device=DEV)
    for p in partials:
        acc += p[:, :cols].float()
    return acc.to(partials[0].dtype)


def _rehearse(bufs, sigs, rows, cols, ld, blocks=0):
    from sparkinfer_b200._lib import launch

    launch.allreduce_peer([b.data_ptr() for b in bufs], [s.data_ptr() for s in sigs], -1,
                          bufs[0].dtype, rows, cols, ld, DEV, blocks=blocks)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_every_rank_ends_with_the_rank_ordered_sum(world, dtype):
    from sparkinfer_b200._lib import launch

    rows, cols = 203, 1032       # rows not divisible by the world: slabs of unequal height
    gen = torch.Generator(device=DEV).manual_seed(100 + world)
    sigs = _signals(world)
    for call in range(3):        # the flags carry a call number: nothing is reset in between
        bufs = [(torch.randn((rows, cols), device=DEV, generator=gen) * (r + 1)).to(dtype)
                for r in range(world)]
        want = _expected(bufs, cols)
        _rehearse(bufs, sigs, rows, cols, cols, blocks=2 + call)
        torch.cuda.synchronize()
        launch.check_kernel_status(DEV)
        for r in range(world):
            assert torch.equal(bufs[r].view(torch.int16), want.view(torch.int16)), (call, r)
        assert all(int(s[0].item()) == call + 1 for s in sigs)      # completed calls
        assert all(int(s[1].item()) == 0 for s in sigs)             # block counter back at zero


def test_padded_rows_keep_their_padding():
    from sparkinfer_b200._lib import launch

    world, rows, cols, ld = 4, 96, 520, 528
    gen = torch.Generator(device=DEV).manual_seed(7)
    bufs = [torch.randn((rows, ld), device=DEV, generator=gen).to(torch.bfloat16) for _ in range(world)]
    pads = [b[:, cols:].clone() for b in bufs]
    want = _expected(bufs, cols)
    _rehearse(bufs, _signals(world), rows, cols, ld)
    torch.cuda.synchronize()
    launch.check_kernel_status(DEV)
    for b, pad in zip(bufs, pads):
        assert torch.equal(b[:, :cols].view(torch.int16), want.view(torch.int16))
        assert torch.equal(b[:, cols:], pad)


def test_full_size_partial_of_config_4_on_two_ranks():
    """4096 x 7168 BF16 (58.7 MB per rank), the output of BASELINE configuration 4."""
    from sparkinfer_b200._lib import launch

    world, rows, cols = 2, 4096, 7168
    gen = torch.Generator(device=DEV).manual_seed(11)
    bufs = [torch.randn((rows, cols), device=DEV, generator=gen).to(torch.bfloat16) for _ in range(world)]
    want = _expected(bufs, cols)
    _rehearse(bufs, _signals(world), rows, cols, cols)
    torch.cuda.synchronize()
    launch.check_kernel_status(DEV)
    for b in bufs:
        assert torch.equal(b.view(torch.int16), want.view(torch.int16))


def test_one_rank_is_a_no_op_and_bad_arguments_are_refused():
    from sparkinfer_b200._lib import launch

    buf = torch.ones((8, 64), dtype=torch.bfloat16, device=DEV)
    sig = _signals(1)
    launch.allreduce_peer([buf.data_ptr()], [sig[0].data_ptr()], 0, buf.dtype, 8, 64, 64, DEV)
    torch.cuda.synchronize()
    assert bool((buf == 1).all())
    with pytest.raises(RuntimeError, match="multiples of 8"):
        launch.allreduce_peer([buf.data_ptr()] * 2, [sig[0].data_ptr()] * 2, -1, buf.dtype, 8, 60, 64, DEV)
    with pytest.raises(RuntimeError, match="rank outside"):
        launch.allreduce_peer([buf.data_ptr()] * 2, [sig[0].data_ptr()] * 2, 2, buf.dtype, 8, 64, 64, DEV)
    with pytest.raises(RuntimeError, match="resident"):
        launch.allreduce_peer([buf.data_ptr()] * 2, [sig[0].data_ptr()] * 2, -1, buf.dtype, 8, 64, 64,
                              DEV, blocks=4096)


def test_a_peer_that_never_arrives_ends_in_a_status_word_not_a_hang():
    """Rank 0 of a world of two, alone: nobody sets its peer's start flag. The wait is bounded
    (64 polls here), the kernel raises the status word, skips the data phase and returns."""
    from sparkinfer_b200._lib import launch

    launch.check_kernel_status(DEV)
    bufs = [torch.full((16, 64), float(r + 1), dtype=torch.bfloat16, device=DEV) for r in range(2)]
    sigs = _signals(2)
    launch.allreduce_peer([b.data_ptr() for b in bufs], [s.data_ptr() for s in sigs], 0,
                          torch.bfloat16, 16, 64, 64, DEV, blocks=2, max_polls=64)
    torch.cuda.synchronize()
    assert int(launch.status_buffer(DEV)[0].item()) == 6
    with pytest.raises(RuntimeError, match="timed out waiting for another rank"):
        launch.check_kernel_status(DEV)
    assert bool((bufs[0] == 1).all()) and bool((bufs[1] == 2).all())   # nothing was summed
    launch.check_kernel_status(DEV)


# --------------------------------------------------------------------------------------
# The fused form: GEMM output scattered to the slab owners, then the scattered reduction
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind,world,m,n,k_local", [
    ("nvfp4", 2, 512, 512, 512), ("mxfp8", 2, 1024, 768, 256), ("nvfp4", 4, 1024, 520, 384),
    ("mxfp8", 8, 2048, 256, 128),
    ("nvfp4", 2, 2048, 2560, 2048),      # 80 pair tiles on 74 pairs: the split leftover tiles scatter too
])
def test_scattered_gemm_then_reduction_equals_the_sum_of_plain_partials(kind, world, m, n, k_local):
    """Each "rank" multiplies its K slice (separate launches that do not wait on each other:
    every receive buffer is local here). Slot r of receive buffer s must equal rows of slab s of
    rank r's plain partial bit for bit, the reduced output must equal the rank-ordered FP32 sum
    rounded once, and that sum must meet the GEMM's error bound against the FP32
    dequantize-matmul over the whole K."""
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import BLOCK_N_PAIR, KIND_MXFP8, KIND_NVFP4
    from test_gemm_fuzz_gpu import _operand

    code = KIND_MXFP8 if kind == "mxfp8" else KIND_NVFP4
    gen = torch.Generator(device=DEV).manual_seed(500 + world + m)
    alpha = torch.tensor([0.5], dtype=torch.float32, device=DEV)
    slab = m // world
    recv = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    outs = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    partials, ref = [], torch.zeros((m, n), dtype=torch.float32, device=DEV)
    for r in range(world):
        a, sfa, a_deq = _operand(kind, m, k_local, gen, DEV)
        b, sfb, b_deq = _operand(kind, n, k_local, gen, DEV)
        ref += 0.5 * (a_deq @ b_deq.T)
        plain = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        launch.gemm_blockscaled(code, a, sfa, b, sfb, plain, alpha, m, n, k_local, block_n=BLOCK_N_PAIR)
        launch.gemm_blockscaled_scatter(code, a, sfa, b, sfb, [t.data_ptr() for t in recv], r,
                                        torch.bfloat16, alpha, m, n, k_local)
        partials.append(plain)
    torch.cuda.synchronize()
    launch.check_kernel_status(DEV)
    for s in range(world):
        for r in range(world):
            got = recv[s][r * slab:(r + 1) * slab]
            want = partials[r][s * slab:(s + 1) * slab]
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (s, r)
    launch.allreduce_peer([t.data_ptr() for t in recv], [t.data_ptr() for t in _signals(world)], -1,
                          torch.bfloat16, m, n, n, DEV, output_ptrs=[t.data_ptr() for t in outs])
    torch.cuda.synchronize()
    launch.check_kernel_status(DEV)
    want = _expected(partials, n)
    for t in outs:
        assert torch.equal(t.view(torch.int16), want.view(torch.int16))
    scale = float(ref.abs().max())
    err = float((outs[0].float() - ref).abs().max())
    assert err <= (world * 2.0 ** -8 + 2.0 ** -16) * scale, (err, scale)


def test_scatter_refuses_shapes_it_cannot_cut_into_whole_tiles():
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import KIND_MXFP8

    z = torch.zeros(1 << 20, dtype=torch.uint8, device=DEV)
    dst = [z.data_ptr(), z.data_ptr()]
    with pytest.raises(RuntimeError, match="multiple of 256"):
        launch.gemm_blockscaled_scatter(KIND_MXFP8, z, z, z, z, dst, 0, torch.bfloat16, None, 384, 256, 128)
    with pytest.raises(RuntimeError, match="BF16 or FP16"):
        launch.gemm_blockscaled_scatter(KIND_MXFP8, z, z, z, z, dst, 0, torch.float32, None, 512, 256, 128)
