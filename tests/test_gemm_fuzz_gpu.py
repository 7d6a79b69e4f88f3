"""Seeded shape fuzz of the block-scaled GEMM against a plain PyTorch FP32 reference of the same
op (operands dequantized on the GPU, FP32 matmul). Random codes and random scale bytes, random
M / N / K including ragged edges, every kernel family (decode, tiled with each tile width, CTA
pair), BF16 / FP16 / FP32 outputs. Complements the oracle-based parity tests, which use fewer
and smaller shapes because the CPU oracle quantizes real data."""

from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def _atoms(scale_rows: torch.Tensor, pad: int) -> torch.Tensor:
    """[rows, cols] scale bytes -> flat 512-byte atoms [row_tile][col_tile][32][4][4]."""
    rows, cols = scale_rows.shape
    rp, cp = -(-rows // 128) * 128, -(-cols // 4) * 4
    padded = torch.full((rp, cp), pad, dtype=torch.uint8, device=scale_rows.device)
    padded[:rows, :cols] = scale_rows
    return padded.view(rp // 128, 4, 32, cp // 4, 4).permute(0, 3, 2, 1, 4).contiguous().view(-1)


def _operand(kind: str, rows: int, k: int, gen, dev):
    """Random operand: (codes, scale atoms, dequantized FP32 [rows, k])."""
    if kind == "mxfp8":
        codes = torch.randint(0, 256, (rows, k), dtype=torch.uint8, device=dev, generator=gen)
        codes = codes & 0xBF  # |value| < 2, no NaN pattern
        scales = torch.randint(121, 129, (rows, k // 32), dtype=torch.uint8, device=dev, generator=gen)
        deq = codes.view(torch.float8_e4m3fn).float() * torch.exp2(
            scales.float() - 127.0).repeat_interleave(32, dim=1)
        return codes, _atoms(scales, 127), deq
    packed = torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, device=dev, generator=gen)
    lut = torch.tensor(E2M1, dtype=torch.float32, device=dev)
    vals = torch.stack((lut[(packed & 0xF).long()], lut[(packed >> 4).long()]), dim=-1).view(rows, k)
    if kind == "mxfp4":
        scales = torch.randint(121, 129, (rows, k // 32), dtype=torch.uint8, device=dev, generator=gen)
        deq = vals * torch.exp2(scales.float() - 127.0).repeat_interleave(32, dim=1)
        return packed, _atoms(scales, 127), deq
    scales = torch.randint(0x18, 0x31, (rows, k // 16), dtype=torch.uint8, device=dev, generator=gen)
    deq = vals * scales.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=1)
    return packed, _atoms(scales, 0), deq


def _cases():
    rng = np.random.default_rng(20261125)
    cases = []
    for i in range(48):
        kind = "mxfp8" if rng.random() < 0.5 else "nvfp4"
        m = int(rng.choice([1, 3, 8, 17, 33, 64, 65, 127, 128, 129, 200, 256, 300, 511, 640]))
        n = int(rng.choice([8, 24, 64, 72, 128, 136, 192, 200, 256, 264, 320, 504, 512, 776, 1024, 1288]))
        k_unit = 32 if kind == "mxfp8" else 64
        k = k_unit * int(rng.integers(1, 24))
        route = str(rng.choice(["auto", "auto", "bn64", "bn128", "bn192", "bn256", "pair", "decode"]))
        if route == "decode" and m > 128:
            route = "auto"
        dtype = [torch.bfloat16, torch.bfloat16, torch.float16, torch.float32][int(rng.integers(0, 4))]
        cases.append((i, kind, m, n, k, route, dtype))
    return cases


@pytest.mark.parametrize("index,kind,m,n,k,route,dtype", _cases())
def test_gemm_matches_fp32_reference_on_random_shapes(index, kind, m, n, k, route, dtype):
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import BLOCK_N_PAIR, KIND_MXFP8, KIND_NVFP4

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(1000 + index)
    a, sfa, a_deq = _operand(kind, m, k, gen, dev)
    b, sfb, b_deq = _operand(kind, n, k, gen, dev)
    alpha = torch.tensor([0.75], dtype=torch.float32, device=dev)
    ldc = n + (8 if index % 3 == 0 else 0)  # sometimes a padded output pitch
    out = torch.full((m, ldc), float("nan"), dtype=dtype, device=dev)
    kwargs = {}
    if route.startswith("bn"):
        kwargs["block_n"] = int(route[2:])
    elif route == "pair":
        kwargs["block_n"] = BLOCK_N_PAIR
    elif route == "decode":
        kwargs["small_m"] = True
    launch.gemm_blockscaled(KIND_MXFP8 if kind == "mxfp8" else KIND_NVFP4, a, sfa, b, sfb, out,
                            alpha, m, n, k, ldc=ldc, **kwargs)
    torch.cuda.synchronize()
    launch.check_kernel_status(dev)
    ref = 0.75 * (a_deq @ b_deq.T)
    got = out[:, :n].float()
    assert not torch.isnan(got).any()
    if ldc > n:
        assert torch.isnan(out[:, n:].float()).all(), "wrote past column N"
    scale = float(ref.abs().max())
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -20}[dtype]
    err = float((got - ref).abs().max())
    assert err <= (eps + 2.0 ** -16) * scale + 1e-30, (err, scale)


def _block_fp8_cases():
    rng = np.random.default_rng(77)
    cases = []
    for i in range(16):
        m = int(rng.choice([1, 5, 64, 128, 129, 255, 256, 300, 513]))
        n = int(rng.choice([128, 256, 384, 640, 1152]))
        k = 128 * int(rng.integers(1, 10))
        dtype = [torch.bfloat16, torch.float16, torch.float32][int(rng.integers(0, 3))]
        cases.append((i, m, n, k, dtype))
    return cases


@pytest.mark.parametrize("index,m,n,k,dtype", _block_fp8_cases())
def test_block_fp8_gemm_matches_fp32_reference_on_random_shapes(index, m, n, k, dtype):
    from sparkinfer_b200._lib import launch

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(5000 + index)
    a = torch.randint(0, 256, (m, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    b = torch.randint(0, 256, (n, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    sa = torch.rand((m, k // 128), device=dev, generator=gen) + 0.25
    sb = torch.rand((n // 128, k // 128), device=dev, generator=gen) + 0.25
    out = torch.full((m, n), float("nan"), dtype=dtype, device=dev)
    launch.gemm_block_fp8(a, sa, b, sb, out, None, m, n, k)
    torch.cuda.synchronize()
    launch.check_kernel_status(dev)
    a_deq = a.view(torch.float8_e4m3fn).float() * sa.repeat_interleave(128, dim=1)
    b_deq = b.view(torch.float8_e4m3fn).float() * sb.repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
    ref = a_deq @ b_deq.T
    got = out.float()
    assert not torch.isnan(got).any()
    scale = float(ref.abs().max())
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -20}[dtype]
    assert float((got - ref).abs().max()) <= (eps + 2.0 ** -16) * scale + 1e-30


@pytest.mark.parametrize("kind,m,n,k,dtype", [
    ("nvfp4", 2048, 2560, 2048, torch.bfloat16),   # 80 pair tiles on 74 pairs: 6 left, 4 segments
    ("mxfp8", 1536, 3328, 1024, torch.bfloat16),   # 78 tiles: 4 left
    ("nvfp4", 2000, 2500, 1536, torch.float32),    # ragged edges inside the leftover tiles
    ("mxfp8", 1792, 2816, 1024, torch.float16),    # 7 x 11 = 77 tiles: 3 left
    ("nvfp4", 256, 19200, 1024, torch.bfloat16),   # one tile row: 75 tiles, 1 left, 2 k-tiles each
])
def test_cta_pair_split_tail_matches_fp32_reference(kind, m, n, k, dtype):
    """The CTA-pair kernel cuts the tiles of its last partial round along K over all SM pairs
    and adds the FP32 partials up through the per-stream workspace. Every output element against
    the FP32 reference, twice in a row with identical bytes (the reduction order is fixed and
    the counters return to zero), and against the unsplit kernel (no workspace passed)."""
    import ctypes

    from sparkinfer_b200 import _native
    from sparkinfer_b200._lib import launch

    dev = torch.device("cuda:0")
    code = _native.KIND_MXFP8 if kind == "mxfp8" else _native.KIND_NVFP4
    need = _native.load().b12x_b200_gemm_blockscaled_workspace_bytes(code, m, n, k, 0, 0)
    assert need > 0, "shape chosen to have a split tail"
    gen = torch.Generator(device=dev).manual_seed(4242 + m + n)
    a, sfa, a_deq = _operand(kind, m, k, gen, dev)
    b, sfb, b_deq = _operand(kind, n, k, gen, dev)
    alpha = torch.tensor([0.5], dtype=torch.float32, device=dev)
    ref = 0.5 * (a_deq @ b_deq.T)
    scale = float(ref.abs().max())
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -20}[dtype]
    outs = []
    for _ in range(2):
        out = torch.full((m, n), float("nan"), dtype=dtype, device=dev)
        launch.gemm_blockscaled(code, a, sfa, b, sfb, out, alpha, m, n, k)
        torch.cuda.synchronize()
        launch.check_kernel_status(dev)
        assert not torch.isnan(out.float()).any()
        assert float((out.float() - ref).abs().max()) <= (eps + 2.0 ** -16) * scale
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    work = launch.stream_workspace(need, dev)
    assert int(work[:65536].count_nonzero()) == 0, "counters must return to zero"
    unsplit = torch.full((m, n), float("nan"), dtype=dtype, device=dev)
    rc = _native.load().b12x_b200_gemm_blockscaled(
        code, a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), unsplit.data_ptr(),
        {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[dtype], alpha.data_ptr(), m, n, k, n,
        0, 0, launch.status_buffer(dev).data_ptr(),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _native.check(rc, "b12x_b200_gemm_blockscaled")
    torch.cuda.synchronize()
    assert float((unsplit.float() - ref).abs().max()) <= (eps + 2.0 ** -16) * scale
    assert float((unsplit.float() - outs[0].float()).abs().max()) <= 2 * eps * scale + 1e-30


# --------------------------------------------------------------------------------------
# The unscaled FP8 recipe (dense_gemm(plain_fp8=True) on the tiled kernels): E4M3 x E4M3,
# alpha the only scale, no scale tensors at all
# --------------------------------------------------------------------------------------
def _plain_fp8_cases():
    rng = np.random.default_rng(4242)
    cases = []
    for i in range(20):
        m = int(rng.choice([65, 128, 129, 255, 256, 300, 512, 777, 1024]))
        n = int(rng.choice([64, 128, 200, 256, 384, 640, 1152, 2048]))
        k = 32 * int(rng.integers(1, 40))
        if k % 16:
            k += 16
        route = str(rng.choice(["auto", "bn64", "bn128", "bn192", "bn256", "pair"]))
        dtype = [torch.bfloat16, torch.float16, torch.float32][int(rng.integers(0, 3))]
        cases.append((i, m, n, k, route, dtype, bool(rng.integers(0, 2))))
    cases.append((20, 2048, 2560, 2048, "auto", torch.bfloat16, False))   # pair kernel, split leftover tiles
    cases.append((21, 4096, 4096, 4096, "auto", torch.bfloat16, True))    # several rounds, two accumulators
    return cases


@pytest.mark.parametrize("index,m,n,k,route,dtype,with_bias", _plain_fp8_cases())
def test_plain_fp8_matches_fp32_reference(index, m, n, k, route, dtype, with_bias):
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import BLOCK_N_PAIR, KIND_FP8

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(9000 + index)
    a = torch.randint(0, 256, (m, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    b = torch.randint(0, 256, (n, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    a_deq, b_deq = a.view(torch.float8_e4m3fn).float(), b.view(torch.float8_e4m3fn).float()
    alpha = torch.tensor([0.375], dtype=torch.float32, device=dev)
    bias = None
    if with_bias and dtype != torch.float32:
        bias = torch.randn(n, device=dev, generator=gen).to(dtype)
    out = torch.full((m, n), float("nan"), dtype=dtype, device=dev)
    kwargs = {}
    if route.startswith("bn"):
        kwargs["block_n"] = int(route[2:])
    elif route == "pair":
        kwargs["block_n"] = BLOCK_N_PAIR
    launch.gemm_blockscaled(KIND_FP8, a, None, b, None, out, alpha, m, n, k, bias=bias, **kwargs)
    torch.cuda.synchronize()
    launch.check_kernel_status(dev)
    ref = 0.375 * (a_deq @ b_deq.T)
    if bias is not None:
        ref = (ref.to(dtype).float() + bias.float())
    got = out.float()
    assert not torch.isnan(got).any()
    scale = float(ref.abs().max())
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -20}[dtype]
    err = float((got - ref).abs().max())
    assert err <= ((2 if bias is not None else 1) * eps + 2.0 ** -16) * scale + 1e-30, (err, scale)


def test_plain_fp8_refuses_the_decode_kernel():
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import KIND_FP8

    dev = torch.device("cuda:0")
    z = torch.zeros((64, 128), dtype=torch.uint8, device=dev)
    out = torch.empty((8, 64), dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError, match="tiled kernels only"):
        launch.gemm_blockscaled(KIND_FP8, z, None, z, None, out, None, 8, 64, 128, small_m=True)


def _mxfp4_cases():
    rng = np.random.default_rng(4321)
    cases = []
    for i in range(20):
        m = int(rng.choice([1, 17, 64, 128, 129, 200, 256, 300, 511, 640, 1024]))
        n = int(rng.choice([8, 64, 72, 128, 192, 200, 256, 264, 512, 776, 1024, 1288]))
        k = 64 * int(rng.integers(1, 40))
        route = str(rng.choice(["auto", "bn64", "bn128", "bn192", "bn256", "pair", "pair", "decode",
                                "decode"]))
        if route == "decode" and m > 128:
            m = int(rng.choice([1, 4, 16, 33, 64, 100]))
        dtype = [torch.bfloat16, torch.float16, torch.float32][int(rng.integers(0, 3))]
        cases.append((i, m, n, k, route, dtype))
    cases.append((20, 2048, 4608, 2048, "auto", torch.bfloat16))
    cases.append((21, 4096, 2304, 1600, "pair", torch.bfloat16))   # leftover tiles split along K
    cases.append((22, 16, 14336, 4096, "decode", torch.bfloat16))  # decode shape, stream-K
    cases.append((23, 64, 4096, 1984, "decode", torch.float32))    # two issuers, half-filled atom
    cases.append((24, 128, 1032, 320, "decode", torch.bfloat16))
    return cases


@pytest.mark.parametrize("index,m,n,k,route,dtype", _mxfp4_cases())
def test_mxfp4_matches_fp32_reference(index, m, n, k, route, dtype):
    """E2M1 codes with UE8M0 scales per 32 elements (scale_vec::2X of the FP4 MMA): every tile
    width of the tiled kernel and the CTA-pair kernel, K with a half-filled scale atom."""
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import BLOCK_N_PAIR, KIND_MXFP4
    from tests.gpu_util import assert_whole_output_close

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(7000 + index)
    a, sfa, a_deq = _operand("mxfp4", m, k, gen, dev)
    b, sfb, b_deq = _operand("mxfp4", n, k, gen, dev)
    alpha = torch.tensor([0.5], dtype=torch.float32, device=dev)
    out = torch.full((m, n), float("nan"), dtype=dtype, device=dev)
    kwargs = {}
    if route.startswith("bn"):
        kwargs["block_n"] = int(route[2:])
    elif route == "pair":
        kwargs["block_n"] = BLOCK_N_PAIR
    elif route == "decode":
        kwargs["small_m"] = True
    launch.gemm_blockscaled(KIND_MXFP4, a, sfa, b, sfb, out, alpha, m, n, k, **kwargs)
    torch.cuda.synchronize()
    launch.check_kernel_status(dev)
    assert_whole_output_close(out, a_deq, b_deq, 0.5, out_dtype=dtype)


def test_mxfp4_runs_through_mm_and_has_no_fused_activation_quantizer():
    """The public ``blockscaled.mm`` accepts float4_e2m1fn with float8_e8m0fnu / 32 scales (the
    reference's MXF4 mode, b12x/_lib/dense_gemm.py:580-582); a decode shape goes to the decode
    kernel like the other recipes. The fused-quantization entry refuses the kind."""
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._lib.layout import convert_sf_to_mma_layout as mma_view
    from sparkinfer_b200._native import KIND_MXFP4
    from sparkinfer_b200.gemm import blockscaled
    from tests.gpu_util import assert_whole_output_close

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(99)
    m, n, k = 16, 4096, 1024        # a decode shape for the other recipes
    a, sfa, a_deq = _operand("mxfp4", m, k, gen, dev)
    b, sfb, b_deq = _operand("mxfp4", n, k, gen, dev)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    from sparkinfer_b200 import _native

    x = torch.zeros((m, k), dtype=torch.bfloat16, device=dev)
    with pytest.raises(_native.NativeLibraryError, match="MXFP4"):
        launch.gemm_smallm_fused_quant(KIND_MXFP4, x, None, b, sfb, out, None, m, n, k)
    got = blockscaled.mm(
        (a.view(m, k // 2, 1), mma_view(sfa.view(torch.float8_e8m0fnu), m, k, 1, 32)),
        (b.view(n, k // 2, 1), mma_view(sfb.view(torch.float8_e8m0fnu), n, k, 1, 32)),
        ab_dtype="float4_e2m1fn", sf_dtype="float8_e8m0fnu", c_dtype="bfloat16", sf_vec_size=32)
    torch.cuda.synchronize()
    assert_whole_output_close(got[:, :, 0], a_deq, b_deq, 1.0)
