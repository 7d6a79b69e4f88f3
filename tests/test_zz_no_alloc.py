"""The allocation-free decode GEMM entry point, called through the C ABI.

Some hosts of this library cannot allocate device memory at the point where they need the
decode GEMM (all memory already handed to their own pool, or the calling thread is inside a
stream capture), so ``b12x_b200_gemm_blockscaled_smallm_noalloc`` carries its partial-sum
scratch inside the library. This test checks that it produces the same bytes as the
caller-workspace entry point, twice in a row on different inputs (the built-in scratch keeps
the previous call's contents), that its results match the CPU oracle when a call that splits
many tiles is followed by one that splits few, and that a shape beyond the built-in capacity
is refused with a readable message and leaves nothing on the stream. The file name sorts last
so a run that stops at the first failure has already run every other test.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(seed, m, n, k, dev):
    """Random NVFP4 codes with benign scale bytes (0x30..0x3F = 0.5 .. 1.875)."""
    gen = torch.Generator(device=dev).manual_seed(seed)
    katoms = k // 64
    x = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=dev, generator=gen)
    w = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=gen)
    sfx = torch.randint(0x30, 0x40, (katoms * 512,), dtype=torch.uint8, device=dev, generator=gen)
    sfw = torch.randint(0x30, 0x40, ((n // 128) * katoms * 512,), dtype=torch.uint8, device=dev,
                        generator=gen)
    return x, sfx, w, sfw


def test_noalloc_entry_point_matches_workspace_entry_point_twice():
    from sparkinfer_b200 import _native

    lib = _native.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    kind = _native.KIND_NVFP4
    m, n, k = 8, 1024, 2048           # 8 tiles x 8 k-tiles: every tile is split over 8 CTAs
    need = lib.b12x_b200_gemm_smallm_workspace_bytes(kind, m, n, k, 0)
    assert 0 < need <= lib.b12x_b200_gemm_smallm_noalloc_capacity_bytes()
    workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
    alpha = torch.tensor([0.125], dtype=torch.float32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, seed in enumerate((11, 12)):
        x, sfx, w, sfw = _operands(seed, m, n, k, dev)
        want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        rc = lib.b12x_b200_gemm_blockscaled_smallm(
            kind, x.data_ptr(), sfx.data_ptr(), w.data_ptr(), sfw.data_ptr(), want.data_ptr(),
            _native.DT_BF16, alpha.data_ptr(), m, n, k, n, workspace.data_ptr(), need, 0,
            status.data_ptr(), stream)
        _native.check(rc, "smallm")
        rc = lib.b12x_b200_gemm_blockscaled_smallm_noalloc(
            kind, x.data_ptr(), sfx.data_ptr(), w.data_ptr(), sfw.data_ptr(), got.data_ptr(),
            _native.DT_BF16, alpha.data_ptr(), m, n, k, n, 0, status.data_ptr(), stream)
        _native.check(rc, "smallm_noalloc")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        assert not torch.isnan(got.float()).any(), f"call {call}: output not fully written"
        assert float(got.float().abs().max()) > 0
        # Same kernel, same deterministic reduction order: equal bytes (tolerance zero).
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call} differs"


def test_noalloc_entry_point_matches_the_oracle_after_a_larger_problem():
    """A call with 32 split tiles, then one with 4: the second must not be disturbed by what the
    first left in the shared scratch (counters or partial sums). Both against the oracle's
    dequantize-to-FP32 matmul of the same random codes and scale bytes."""
    from gpu_util import assert_gemm_close
    from oracle import blockscaled_oracle as O
    from sparkinfer_b200 import _native

    lib = _native.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    kind = _native.KIND_NVFP4
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rng = np.random.default_rng(99)
    for m, n, k in ((16, 4096, 2048), (3, 512, 4096)):
        assert (lib.b12x_b200_gemm_smallm_workspace_bytes(kind, m, n, k, 0)
                <= lib.b12x_b200_gemm_smallm_noalloc_capacity_bytes())
        ops = []
        for rows in (m, n):
            packed = rng.integers(0, 256, (rows, k // 2), dtype=np.uint8)
            scales = rng.integers(0x30, 0x40, (rows, k // 16), dtype=np.uint8)
            ops.append((torch.from_numpy(packed).to(dev),
                        torch.from_numpy(O.swizzle_scales(scales, 0)).to(dev),
                        O.dequantize_nvfp4(packed, scales, np.float32(1.0))))
        (x, sfx, x_deq), (w, sfw, w_deq) = ops
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        rc = lib.b12x_b200_gemm_blockscaled_smallm_noalloc(
            kind, x.data_ptr(), sfx.data_ptr(), w.data_ptr(), sfw.data_ptr(), got.data_ptr(),
            _native.DT_BF16, None, m, n, k, n, 0, status.data_ptr(), stream)
        _native.check(rc, "smallm_noalloc")
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        assert_gemm_close(got, x_deq @ w_deq.T)


def test_noalloc_entry_point_refuses_shapes_beyond_its_scratch():
    from sparkinfer_b200 import _native

    lib = _native.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    m, n, k = 128, 8192, 4096         # 64 tiles x 2 CTAs x 64 KiB partials > 4 MiB
    need = lib.b12x_b200_gemm_smallm_workspace_bytes(_native.KIND_NVFP4, m, n, k, 0)
    assert need > lib.b12x_b200_gemm_smallm_noalloc_capacity_bytes()
    x, sfx, w, sfw = _operands(5, m, n, k, dev)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
    rc = lib.b12x_b200_gemm_blockscaled_smallm_noalloc(
        _native.KIND_NVFP4, x.data_ptr(), sfx.data_ptr(), w.data_ptr(), sfw.data_ptr(),
        out.data_ptr(), _native.DT_BF16, None, m, n, k, n, 0, None,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -3
    assert "built-in scratch" in _native.last_error()
    torch.cuda.synchronize()
    assert int(out.count_nonzero()) == 0
