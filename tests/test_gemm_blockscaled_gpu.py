"""Block-scaled GEMM on the GPU against the CPU oracle (dequantize to FP32, matmul).

Modelled on the reference's tests/gemm/test_blockscaled.py:90-220, test_gemm_stack.py:210-312
and test_cute_migration_gemm_corpus.py:78-139: NVFP4 and MXFP8 operands built by the (oracle)
reference quantizers, BF16/FP16/FP32 outputs, grouped batches with their own scales,
caller-owned outputs, CUDA-graph replay, a device alpha read at run time; plus decode shapes,
ragged edges, every tile width, and full-size configurations checked on sampled rows and
through linearity in alpha.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN, bf16_bits_to_f32, seeded_bf16
from oracle import blockscaled_oracle as O

pytestmark = pytest.mark.gpu

NVFP4 = dict(ab_dtype="float4_e2m1fn", sf_dtype="float8_e4m3fn", sf_vec_size=16)
MXFP8 = dict(ab_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu", sf_vec_size=32)


def _alpha(gsa, gsb):
    from gpu_util import DEV

    return torch.tensor([1.0 / (float(gsa) * float(gsb))], dtype=torch.float32, device=DEV)


@pytest.mark.parametrize("m,n,k,c_dtype,tile_n", [
    (128, 128, 128, "bfloat16", None), (256, 512, 128, "bfloat16", None),
    (512, 256, 256, "bfloat16", None), (128, 128, 128, "float16", None),
    (32, 128, 128, "bfloat16", None), (1, 512, 512, "bfloat16", None),
    (4, 512, 512, "bfloat16", 64), (16, 512, 1024, "bfloat16", 128),
    (64, 768, 512, "bfloat16", 192), (130, 72, 384, "bfloat16", None),
    (300, 504, 640, "float32", 192), (256, 1024, 2048, "bfloat16", 256),
    (128, 200, 192, "bfloat16", 64),
])
def test_mm_nvfp4_matches_oracle(m, n, k, c_dtype, tile_n):
    from gpu_util import assert_gemm_close, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled

    lhs, gsa, a_deq = nvfp4_operand(seeded_bf16(m * 7 + k, (m, k), 0.25))
    rhs, gsb, b_deq = nvfp4_operand(seeded_bf16(n * 11 + k, (n, k), 0.02))
    out = blockscaled.mm(lhs, rhs, alpha=_alpha(gsa, gsb), c_dtype=c_dtype,
                         mma_tiler_mn=(128, tile_n) if tile_n else None, **NVFP4)
    torch.cuda.synchronize()
    assert out.shape == (m, n, 1)
    assert_gemm_close(out[:, :, 0], a_deq @ b_deq.T, out_dtype=out.dtype)


@pytest.mark.parametrize("m,n,k,c_dtype,tile_n", [
    (128, 128, 128, "bfloat16", None), (7, 32, 128, "bfloat16", None),
    (3, 40, 256, "bfloat16", None), (64, 1024, 512, "bfloat16", 128),
    (256, 512, 384, "float16", 64), (129, 256, 256, "bfloat16", None),
    (8, 4096, 4096, "bfloat16", None), (300, 504, 640, "float32", 192),
    (512, 1024, 1024, "bfloat16", 256),
])
def test_mm_mxfp8_matches_oracle(m, n, k, c_dtype, tile_n):
    from gpu_util import assert_gemm_close, mxfp8_operand
    from sparkinfer_b200.gemm import blockscaled

    lhs, a_deq = mxfp8_operand(seeded_bf16(m * 5 + k, (m, k), 0.25))
    rhs, b_deq = mxfp8_operand(seeded_bf16(n * 13 + k, (n, k), 1.0 / 32))
    out = blockscaled.mm(lhs, rhs, c_dtype=c_dtype,
                         mma_tiler_mn=(128, tile_n) if tile_n else None, expected_m=m, **MXFP8)
    torch.cuda.synchronize()
    assert_gemm_close(out[:, :, 0], a_deq @ b_deq.T, out_dtype=out.dtype)


@pytest.mark.parametrize("m,n,k,tile", [
    (16, 512, 512, None),           # decode kernel, unit block scales
    (256, 512, 384, None),          # tiled kernel, unscaled E4M3 MMA
    (300, 504, 640, (128, 192)), (1024, 2048, 1024, (256, 256)),
    (2048, 2560, 2048, None),       # CTA-pair kernel
])
def test_mm_plain_fp8_ignores_the_scale_tensors(m, n, k, tile):
    """dense_gemm(plain_fp8=True): E4M3 codes times alpha, whatever the scale storage holds
    (here: bytes that would scale by 2^-127 if they were read)."""
    from gpu_util import DEV
    from sparkinfer_b200._lib import layout
    from sparkinfer_b200.gemm import blockscaled

    gen = torch.Generator(device=DEV).manual_seed(m + n + k)
    a = (torch.randint(0, 256, (m, k), dtype=torch.uint8, device=DEV, generator=gen) & 0xBF)
    b = (torch.randint(0, 256, (n, k), dtype=torch.uint8, device=DEV, generator=gen) & 0xBF)
    zeros_a = torch.zeros((-(-m // 128)) * (-(-k // 128)) * 512, dtype=torch.uint8, device=DEV)
    zeros_b = torch.zeros((-(-n // 128)) * (-(-k // 128)) * 512, dtype=torch.uint8, device=DEV)
    sfa = layout.convert_sf_to_mma_layout(zeros_a, m, k, 1, 32).view(torch.float8_e8m0fnu)
    sfb = layout.convert_sf_to_mma_layout(zeros_b, n, k, 1, 32).view(torch.float8_e8m0fnu)
    alpha = torch.tensor([0.25], dtype=torch.float32, device=DEV)
    out = blockscaled.mm((a.view(torch.float8_e4m3fn).view(m, k, 1), sfa),
                         (b.view(torch.float8_e4m3fn).view(n, k, 1), sfb), alpha=alpha,
                         c_dtype="bfloat16", plain_fp8=True, mma_tiler_mn=tile, **MXFP8)
    torch.cuda.synchronize()
    ref = 0.25 * (a.view(torch.float8_e4m3fn).float() @ b.view(torch.float8_e4m3fn).float().T)
    err = float((out[:, :, 0].float() - ref).abs().max())
    assert err <= (2.0 ** -8 + 2.0 ** -16) * float(ref.abs().max()), err


def test_mm_nvfp4_matches_reference_fixture():
    """Operands and FP32 result produced by the reference's own torch code."""
    from gpu_util import assert_gemm_close, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled

    g = np.load(GOLDEN / "gemm_ref.npz")
    a = torch.from_numpy(g["nv_a"].view(np.int16)).view(torch.bfloat16)
    b = torch.from_numpy(g["nv_b"].view(np.int16)).view(torch.bfloat16)
    lhs, gsa, _ = nvfp4_operand(a, g["nv_gsa"][0])
    rhs, gsb, _ = nvfp4_operand(b, g["nv_gsb"][0])
    out = blockscaled.mm(lhs, rhs, alpha=_alpha(gsa, gsb), c_dtype="float32", **NVFP4)
    assert_gemm_close(out[:, :, 0], g["nv_out"], out_dtype=torch.float32)


def test_mm_equals_bf16_of_dequantized_matmul_on_tiny_shape():
    """tests/gemm/test_cute_migration_gemm_corpus.py:78-139: M=32, N=128, K=128, the kernel
    output equals the BF16 rounding of the dequantized product up to the accumulation order."""
    from gpu_util import nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 32, 128, 128
    lhs, gsa, a_deq = nvfp4_operand(seeded_bf16(1, (m, k), 0.25))
    rhs, gsb, b_deq = nvfp4_operand(seeded_bf16(2, (n, k), 0.25))
    out = blockscaled.mm(lhs, rhs, alpha=_alpha(gsa, gsb), c_dtype="bfloat16", **NVFP4)
    ref = O.bf16_round(a_deq @ b_deq.T)
    got = out[:, :, 0].float().cpu().numpy()
    ulp = np.abs(ref) * 2.0 ** -7 + 1e-30
    assert (np.abs(got - ref) <= ulp).all()
    assert (got == ref).mean() > 0.98


def test_mm_grouped_batches_use_their_own_scales():
    """L = 3 MXFP8 groups, each scaled differently (tests/gemm/test_blockscaled.py:128-175)."""
    from gpu_util import DEV, assert_gemm_close, to_dev
    from sparkinfer_b200._lib import layout
    from sparkinfer_b200.gemm import blockscaled

    m, n, k, groups = 64, 256, 256, 3
    mult = [1.0, 4.0, 0.5]
    a_vals, a_sw, b_vals, b_sw, refs = [], [], [], [], []
    for g in range(groups):
        a = seeded_bf16(50 + g, (m, k), 0.25 * mult[g]).float().numpy()
        b = seeded_bf16(60 + g, (n, k), 0.03 / mult[g]).float().numpy()
        av, asr = O.quantize_mxfp8_rows(a)
        bv, bsr = O.quantize_mxfp8_rows(b)
        a_vals.append(av); b_vals.append(bv)
        a_sw.append(O.swizzle_scales(asr, 127)); b_sw.append(O.swizzle_scales(bsr, 127))
        refs.append(O.dequantize_mxfp8(av, asr) @ O.dequantize_mxfp8(bv, bsr).T)
    a_t = to_dev(np.stack(a_vals)).view(torch.float8_e4m3fn).as_strided((m, k, groups), (k, 1, m * k))
    b_t = to_dev(np.stack(b_vals)).view(torch.float8_e4m3fn).as_strided((n, k, groups), (k, 1, n * k))
    sfa = layout.convert_sf_to_mma_layout(to_dev(np.concatenate(a_sw)), m, k, groups, 32)
    sfb = layout.convert_sf_to_mma_layout(to_dev(np.concatenate(b_sw)), n, k, groups, 32)
    out = blockscaled.mm((a_t, sfa), (b_t, sfb), c_dtype="bfloat16", **MXFP8)
    assert out.shape == (m, n, groups) and out.stride() == (n, 1, m * n)
    for g in range(groups):
        assert_gemm_close(out[:, :, g], refs[g])


def test_mm_writes_caller_output_and_replays_under_cuda_graph():
    """out= given: no allocation, capture after warm-up, three bit-identical replays, and a
    device alpha changed between replays is honoured (tests/gemm/test_blockscaled.py:178-220,
    tests/gemm/test_gemm_stack.py:167-190)."""
    from gpu_util import DEV, assert_gemm_close, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 128, 256, 256
    lhs, gsa, a_deq = nvfp4_operand(seeded_bf16(5, (m, k), 0.25))
    rhs, gsb, b_deq = nvfp4_operand(seeded_bf16(6, (n, k), 0.02))
    alpha = _alpha(gsa, gsb)
    out = torch.zeros((m, n, 1), dtype=torch.bfloat16, device=DEV)
    ret = blockscaled.mm(lhs, rhs, out, alpha=alpha, c_dtype="bfloat16", **NVFP4)
    torch.cuda.synchronize()
    assert ret.data_ptr() == out.data_ptr()
    eager = out.clone()
    ref = a_deq @ b_deq.T
    assert_gemm_close(eager[:, :, 0], ref)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        blockscaled.mm(lhs, rhs, out, alpha=alpha, c_dtype="bfloat16", **NVFP4)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    alpha.mul_(2.0)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out.float(), eager.float() * 2.0)  # power-of-two alpha: exact


def test_mm_row_strided_output_view():
    from gpu_util import DEV, assert_gemm_close, mxfp8_operand
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 128, 128, 256
    lhs, a_deq = mxfp8_operand(seeded_bf16(8, (m, k), 0.25))
    rhs, b_deq = mxfp8_operand(seeded_bf16(9, (n, k), 0.03))
    wide = torch.full((m, 2 * n), 7.0, dtype=torch.bfloat16, device=DEV)
    out = wide[:, :n].unsqueeze(-1)
    blockscaled.mm(lhs, rhs, out, c_dtype="bfloat16", **MXFP8)
    torch.cuda.synchronize()
    assert_gemm_close(wide[:, :n], a_deq @ b_deq.T)
    assert (wide[:, n:] == 7.0).all()


def test_mm_fused_quant_a_equals_quantize_then_mm():
    from gpu_util import assert_gemm_close, mxfp8_operand
    from gpu_util import DEV
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 5, 512, 512
    x = seeded_bf16(15, (m, k), 0.25)
    rhs, b_deq = mxfp8_operand(seeded_bf16(16, (n, k), 0.03))
    _, a_deq = mxfp8_operand(x)
    out = blockscaled.mm_fused_quant_a(x.to(DEV), rhs[0], rhs[1])
    torch.cuda.synchronize()
    assert out.shape == (m, n, 1) and out.dtype == torch.bfloat16
    assert_gemm_close(out[:, :, 0], a_deq @ b_deq.T)
    with pytest.raises(ValueError, match="1<=M<=8"):
        blockscaled.mm_fused_quant_a(seeded_bf16(1, (9, k)).to(DEV), rhs[0], rhs[1])


@pytest.mark.parametrize("recipe", ["mxfp8_prefill", "nvfp4_row_parallel_shard",
                                    "nvfp4_row_parallel_unsharded"])
def test_full_size_configurations_on_sampled_rows(recipe):
    """Full-size operands (the MXFP8 prefill GEMM 8192 x 7168 x 7168; the row-parallel NVFP4
    GEMM 4096 x 7168 x 18432 on one GPU; one 1/8 K-shard of it, K = 2304): quantized on the GPU
    by the row quantizers and multiplied by the GEMM into a NaN-prefilled output. Checked three
    ways: a sample of rows and columns against the CPU oracle, EVERY output element against an
    FP32 matmul of the operands dequantized with torch ops on the GPU, and linearity in alpha."""
    from gpu_util import (DEV, assert_whole_output_close, torch_dequant_mxfp8,
                          torch_dequant_nvfp4)
    from sparkinfer_b200._lib import layout
    from sparkinfer_b200._lib.mxfp8_rows import empty_mxfp8_rows_for_dense_gemm, quantize_mxfp8_rows
    from sparkinfer_b200.gemm import blockscaled
    from sparkinfer_b200.quantization import nvfp4

    if recipe == "mxfp8_prefill":
        m, n, k = 8192, 7168, 7168
    elif recipe == "nvfp4_row_parallel_unsharded":
        m, n, k = 4096, 7168, 18432
    else:
        m, n, k = 4096, 7168, 2304
    x = seeded_bf16(42 + 2000, (m, k)).to(DEV)
    w = seeded_bf16(42 + 2001, (n, k), 0.02).to(DEV)
    rows = np.r_[0:16, m // 2:m // 2 + 16, m - 16:m]
    cols = np.r_[0:64, n - 64:n]
    if recipe == "mxfp8_prefill":
        xq = empty_mxfp8_rows_for_dense_gemm(m, k, device=DEV)
        wq = empty_mxfp8_rows_for_dense_gemm(n, k, device=DEV)
        quantize_mxfp8_rows(x, xq.values, xq.scale_rows, xq.scale_mma)
        quantize_mxfp8_rows(w, wq.values, wq.scale_rows, wq.scale_mma)
        lhs = (xq.values.view(m, k, 1), xq.scale_mma)
        rhs = (wq.values.view(n, k, 1), wq.scale_mma)
        alpha = torch.ones(1, device=DEV)
        kw = MXFP8
        a_deq = O.dequantize_mxfp8(*O.quantize_mxfp8_rows(x[rows].float().cpu().numpy()))
        b_deq = O.dequantize_mxfp8(*O.quantize_mxfp8_rows(w[cols].float().cpu().numpy()))
        a_all = torch_dequant_mxfp8(xq.values, xq.scale_rows, m, k)
        b_all = torch_dequant_mxfp8(wq.values, wq.scale_rows, n, k)
    else:
        gsx = O.nvfp4_global_scale(x.float().cpu().numpy())
        gsw = O.nvfp4_global_scale(w.float().cpu().numpy())
        ops, deqs = [], []
        for t, gs, r in ((x, gsx, m), (w, gsw, n)):
            plan = nvfp4.plan(r, k)
            outs = nvfp4.allocate_outputs(plan, device=DEV)
            nvfp4.run(plan=plan, x=t, global_scale=torch.tensor([gs], device=DEV), outputs=outs)
            ops.append((outs.packed_a_view, outs.scale_mma_view(r, k)))
            deqs.append(torch_dequant_nvfp4(outs.packed_a_storage, outs.scale_flat, r, k))
        lhs, rhs = ops
        a_all, b_all = deqs
        alpha = _alpha(gsx, gsw)
        kw = NVFP4
        pa, sa = O.quantize_nvfp4_rows(x[rows].float().cpu().numpy(), gsx)
        pb, sb = O.quantize_nvfp4_rows(w[cols].float().cpu().numpy(), gsw)
        a_deq, b_deq = O.dequantize_nvfp4(pa, sa, gsx), O.dequantize_nvfp4(pb, sb, gsw)
    del x, w
    out = torch.full((m, n, 1), float("nan"), dtype=torch.bfloat16, device=DEV)
    blockscaled.mm(lhs, rhs, out, alpha=alpha, c_dtype="bfloat16", **kw)
    torch.cuda.synchronize()
    got = out[:, :, 0][torch.from_numpy(rows).to(DEV)][:, torch.from_numpy(cols).to(DEV)]
    ref = a_deq @ b_deq.T
    err = np.abs(got.float().cpu().numpy() - ref).max()
    assert err <= 1e-2 * np.abs(ref).max()
    assert err <= (2.0 ** -8 + 2.0 ** -16) * np.abs(ref).max()
    assert_whole_output_close(out[:, :, 0], a_all, b_all, float(alpha.item()))
    del a_all, b_all
    torch.cuda.empty_cache()
    alpha2 = alpha * 4.0
    out2 = blockscaled.mm(lhs, rhs, alpha=alpha2, c_dtype="bfloat16", **kw)
    torch.cuda.synchronize()
    assert torch.equal(out2.float(), out.float() * 4.0)
    assert not torch.isnan(out.float()).any()


def test_no_kernel_reported_a_timed_out_wait():
    from gpu_util import DEV
    from sparkinfer_b200._lib.launch import check_kernel_status

    check_kernel_status(DEV)


# --------------------------------------------------------------------------------------
# block_fp8=True: E4M3 operands with compact FP32 scales (1x128 activations, 128x128 weights)
# --------------------------------------------------------------------------------------
BLOCK_FP8 = dict(ab_dtype="float8_e4m3fn", sf_dtype="float32", sf_vec_size=128, block_fp8=True)


def _block_fp8_operands(seed, m, n, k):
    from gpu_util import to_dev

    a = seeded_bf16(seed, (m, k)).float().numpy()
    b = seeded_bf16(seed + 1, (n, k)).float().numpy()
    a_codes, a_scale = O.quantize_block_fp8(a, 1)
    b_codes, b_scale = O.quantize_block_fp8(b, 128)
    lhs = (to_dev(a_codes).view(torch.float8_e4m3fn).view(m, k, 1), to_dev(a_scale))
    rhs = (to_dev(b_codes).view(torch.float8_e4m3fn).view(n, k, 1), to_dev(b_scale))
    return lhs, rhs, O.gemm_block_fp8(a_codes, a_scale, b_codes, b_scale)


@pytest.mark.parametrize("m,n,k,c_dtype", [
    (1, 128, 256, "bfloat16"), (8, 256, 256, "bfloat16"), (64, 128, 512, "bfloat16"),
    (129, 256, 256, "bfloat16"), (2, 4096, 4096, "bfloat16"), (300, 384, 1024, "float32"),
    (512, 1152, 768, "float16"),
])
def test_mm_block_fp8_matches_oracle(m, n, k, c_dtype):
    """tests/gemm/test_gemm_stack.py:139-165: rtol 2e-2 / atol 2e-3 and cosine >= 0.9999
    against the dequantized FP32 product; the tighter bound of assert_gemm_close holds too."""
    from gpu_util import assert_gemm_close
    from sparkinfer_b200.gemm import blockscaled

    lhs, rhs, ref = _block_fp8_operands(m + n + k, m, n, k)
    out = blockscaled.mm(lhs, rhs, c_dtype=c_dtype, **BLOCK_FP8)
    torch.cuda.synchronize()
    got = out[:, :, 0].float().cpu().numpy()
    assert np.allclose(got, ref, rtol=2e-2, atol=2e-3 * np.abs(ref).max())
    cos = float((got * ref).sum() / np.sqrt((got * got).sum() * (ref * ref).sum()))
    assert cos >= 0.9999
    assert_gemm_close(out[:, :, 0], ref, out_dtype=out.dtype)


def test_mm_block_fp8_matches_reference_fixture_and_rereads_live_scales():
    """Operands and result from the reference's _block_fp8_reference restated with torch ops;
    then a CUDA-graph replay after changing a scale in place
    (tests/gemm/test_gemm_stack.py:167-190)."""
    from gpu_util import DEV, assert_gemm_close, to_dev
    from sparkinfer_b200.gemm import blockscaled

    g = np.load(GOLDEN / "gemm_ref.npz")
    m, k = g["bf8_a"].shape
    n = g["bf8_b"].shape[0]
    sa, sb = to_dev(g["bf8_sa"]), to_dev(g["bf8_sb"])
    lhs = (to_dev(g["bf8_a"]).view(torch.float8_e4m3fn).view(m, k, 1), sa)
    rhs = (to_dev(g["bf8_b"]).view(torch.float8_e4m3fn).view(n, k, 1), sb)
    out = torch.empty((m, n, 1), dtype=torch.float32, device=DEV)
    blockscaled.mm(lhs, rhs, out, c_dtype="float32", **BLOCK_FP8)
    torch.cuda.synchronize()
    assert_gemm_close(out[:, :, 0], g["bf8_out"], out_dtype=torch.float32)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        blockscaled.mm(lhs, rhs, out, c_dtype="float32", **BLOCK_FP8)
    sb[0, :] *= 2.0
    graph.replay()
    torch.cuda.synchronize()
    ref = O.gemm_block_fp8(g["bf8_a"], g["bf8_sa"], g["bf8_b"], sb.cpu().numpy())
    assert_gemm_close(out[:, :, 0], ref, out_dtype=torch.float32)


def test_mm_block_fp8_rejects_bad_scales():
    from gpu_util import DEV
    from sparkinfer_b200.gemm import blockscaled

    a = torch.zeros((4, 256, 1), dtype=torch.float8_e4m3fn, device=DEV)
    b = torch.zeros((128, 256, 1), dtype=torch.float8_e4m3fn, device=DEV)
    sa = torch.ones((4, 2), device=DEV)
    sb = torch.ones((1, 2), device=DEV)
    with pytest.raises(ValueError, match="block_fp8 requires"):
        blockscaled.mm((a, sa[:, :1]), (b, sb), c_dtype="bfloat16", **BLOCK_FP8)
    with pytest.raises(ValueError, match="block_fp8 requires"):
        blockscaled.mm((a, sa), (b, sb), c_dtype="bfloat16", ab_dtype="float8_e4m3fn",
                       sf_dtype="float8_e8m0fnu", sf_vec_size=128, block_fp8=True)
    with pytest.raises(ValueError, match="unswapped"):
        blockscaled.mm((a, sa), (b, sb), c_dtype="bfloat16", swap_ab=True, **BLOCK_FP8)


@pytest.mark.parametrize("kind,m,n,k", [
    ("nvfp4", 256, 256, 128), ("nvfp4", 300, 504, 640), ("nvfp4", 1024, 2048, 1024),
    ("mxfp8", 256, 512, 256), ("mxfp8", 130, 264, 384), ("mxfp8", 768, 1280, 2048),
])
def test_cta_pair_kernel_matches_oracle(kind, m, n, k):
    """The cta_group::2 kernel (two CTAs per 256 x 256 tile) is chosen automatically only for
    problems with at least two thirds of a wave of pair tiles; ask for its tile here on small and
    ragged shapes, including ones whose second CTA lies entirely below the matrix."""
    from gpu_util import assert_gemm_close, mxfp8_operand, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled

    if kind == "nvfp4":
        lhs, gsa, a_deq = nvfp4_operand(seeded_bf16(m + 3 * k, (m, k), 0.25))
        rhs, gsb, b_deq = nvfp4_operand(seeded_bf16(n + 5 * k, (n, k), 0.02))
        out = blockscaled.mm(lhs, rhs, alpha=_alpha(gsa, gsb), c_dtype="bfloat16",
                             mma_tiler_mn=(256, 256), **NVFP4)
    else:
        lhs, a_deq = mxfp8_operand(seeded_bf16(m + 3 * k, (m, k), 0.25))
        rhs, b_deq = mxfp8_operand(seeded_bf16(n + 5 * k, (n, k), 0.03))
        out = blockscaled.mm(lhs, rhs, c_dtype="bfloat16", mma_tiler_mn=(256, 256), **MXFP8)
    torch.cuda.synchronize()
    assert_gemm_close(out[:, :, 0], a_deq @ b_deq.T)


@pytest.mark.parametrize("m,n,k", [(8, 4096, 2048), (16, 14336, 1024), (40, 2048, 4096)])
def test_decode_gemm_chain_back_to_back_matches_separate_launches(m, n, k):
    """Decode GEMMs launched back to back overlap on the device (each starts beside its
    predecessor, shares the SMs' shared and tensor memory with it, and all share one scratch
    buffer). A chain of six with different weights, eagerly and as a CUDA graph, must give bit
    for bit what six synchronised launches give; the first of those is checked against the
    oracle. Shapes cover whole tiles per CTA, split tiles (partial sums through scratch) and
    the single-issuer layout (M > 32)."""
    from gpu_util import assert_gemm_close, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled

    lhs, gsa, a_deq = nvfp4_operand(seeded_bf16(m + k, (m, k), 0.25))
    weights = [nvfp4_operand(seeded_bf16(100 * r + n, (n, k), 0.02)) for r in range(6)]
    alphas = [_alpha(gsa, w[1]) for w in weights]
    separate = []
    for (rhs, _, _), alpha in zip(weights, alphas):
        separate.append(blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="bfloat16", **NVFP4))
        torch.cuda.synchronize()
    assert_gemm_close(separate[0][:, :, 0], a_deq @ weights[0][2].T)

    outs = [torch.empty_like(s) for s in separate]

    def chain():
        for (rhs, _, _), alpha, out in zip(weights, alphas, outs):
            blockscaled.mm(lhs, rhs, out, alpha=alpha, c_dtype="bfloat16", **NVFP4)

    for _ in range(3):
        for out in outs:
            out.zero_()
        chain()
        torch.cuda.synchronize()
        for got, want in zip(outs, separate):
            assert torch.equal(got, want)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain()
    for _ in range(3):
        for out in outs:
            out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for got, want in zip(outs, separate):
            assert torch.equal(got, want)
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(torch.device("cuda:0"))


@pytest.mark.parametrize("kind,m,n,k", [
    ("nvfp4", 65, 384, 512), ("nvfp4", 128, 640, 1024), ("mxfp8", 100, 256, 768),
    ("mxfp8", 48, 1152, 512), ("nvfp4", 33, 2048, 2048),
])
def test_decode_kernel_on_request_up_to_128_rows(kind, m, n, k):
    """M in 65..128 goes to the tiled kernel by default; the decode kernel still accepts it
    through the C ABI (128 padded rows, one issuing warp, all 512 TMEM columns). Call the
    launcher with ``small_m=True`` on the operands of the facade and compare with the oracle."""
    from gpu_util import assert_gemm_close, mxfp8_operand, nvfp4_operand
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import KIND_MXFP8, KIND_NVFP4

    if kind == "nvfp4":
        (a, sfa), gsa, a_deq = nvfp4_operand(seeded_bf16(m + k, (m, k), 0.25))
        (b, sfb), gsb, b_deq = nvfp4_operand(seeded_bf16(n + k, (n, k), 0.02))
        alpha, code = _alpha(gsa, gsb), KIND_NVFP4
    else:
        (a, sfa), a_deq = mxfp8_operand(seeded_bf16(m + k, (m, k), 0.25))
        (b, sfb), b_deq = mxfp8_operand(seeded_bf16(n + k, (n, k), 0.03))
        alpha, code = None, KIND_MXFP8
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    # The 6-D scale views alias contiguous atom storage whose first byte is element 0.
    launch.gemm_blockscaled(code, a, sfa, b, sfb, out, alpha, m, n, k, small_m=True)
    torch.cuda.synchronize()
    launch.check_kernel_status(a.device)
    assert_gemm_close(out, a_deq @ b_deq.T)


def test_full_size_block_fp8_column_parallel_shape_on_sampled_rows():
    """Config 3 at full size (4096 x 18432 x 7168, E4M3 with FP32 scales per 1x128 / 128x128
    block = amax/448 of seeded data): sampled rows and columns against the oracle, linearity
    in alpha over the whole output, and the two halves of N computed as separate column-parallel
    shards must reproduce the unsharded output bit for bit."""
    from gpu_util import DEV, to_dev
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 4096, 18432, 7168
    rows = np.r_[0:8, m // 2:m // 2 + 8, m - 8:m]
    col_blocks = [0, 71, 143]  # 128-column blocks of the weight that are checked
    gen = torch.Generator().manual_seed(42 + 3000)
    a = torch.randn((m, k), generator=gen).to(torch.bfloat16).float()
    b = (torch.randn((n, k), generator=gen) * 0.02).to(torch.bfloat16).float()
    sa = (a.view(m, k // 128, 128).abs().amax(dim=2) / 448.0).clamp_min(1e-12)
    sb = (b.view(n // 128, 128, k // 128, 128).abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
    a8 = (a.view(m, k // 128, 128) / sa[:, :, None]).reshape(m, k).to(torch.float8_e4m3fn)
    b8 = (b.view(n // 128, 128, k // 128, 128) / sb[:, None, :, None]).reshape(n, k).to(
        torch.float8_e4m3fn)
    lhs = (a8.to(DEV).view(m, k, 1), sa.to(DEV).contiguous())
    rhs = (b8.to(DEV).view(n, k, 1), sb.to(DEV).contiguous())
    out = torch.full((m, n, 1), float("nan"), dtype=torch.bfloat16, device=DEV)
    blockscaled.mm(lhs, rhs, out, c_dtype="bfloat16", **BLOCK_FP8)
    torch.cuda.synchronize()
    # Every output element against an FP32 matmul of the operands dequantized on the GPU.
    from gpu_util import assert_whole_output_close
    a_all = lhs[0][:, :, 0].float() * lhs[1].repeat_interleave(128, dim=1)
    b_all = rhs[0][:, :, 0].float() * rhs[1].repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
    assert_whole_output_close(out[:, :, 0], a_all, b_all)
    del a_all, b_all
    torch.cuda.empty_cache()
    a_codes = a8.view(torch.uint8).numpy()[rows]
    for cb in col_blocks:
        b_codes = b8.view(torch.uint8).numpy()[cb * 128:(cb + 1) * 128]
        ref = O.gemm_block_fp8(a_codes, sa.numpy()[rows], b_codes, sb.numpy()[cb:cb + 1])
        got = out[:, cb * 128:(cb + 1) * 128, 0][torch.from_numpy(rows).to(DEV)]
        err = np.abs(got.float().cpu().numpy() - ref).max()
        assert err <= 1e-2 * np.abs(ref).max()
        assert err <= (2.0 ** -8 + 2.0 ** -16) * np.abs(ref).max()
    alpha = torch.tensor([0.25], device=DEV)
    out_q = blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="bfloat16", **BLOCK_FP8)
    assert torch.equal(out_q.float() * 4.0, out.float())
    half = n // 2
    for lo in (0, half):
        shard = blockscaled.mm(lhs, (rhs[0][lo:lo + half], rhs[1][lo // 128:(lo + half) // 128]),
                               c_dtype="bfloat16", **BLOCK_FP8)
        assert torch.equal(shard, out[:, lo:lo + half])
    torch.cuda.synchronize()


@pytest.fixture(scope="module")
def decode_weight():
    """Config-1 weight (14336 x 4096, randn * 0.02) quantized once by the oracle."""
    from gpu_util import to_dev
    from sparkinfer_b200._lib import layout

    n, k = 14336, 4096
    w = seeded_bf16(42 + 1001, (n, k), 0.02).float().numpy()
    gsw = O.nvfp4_global_scale(w)
    wp, ws = O.quantize_nvfp4_rows(w, gsw)
    sf = layout.convert_sf_to_mma_layout(to_dev(O.swizzle_scales(ws, 0)), n, k, 1, 16)
    return (to_dev(wp).reshape(n, k // 2, 1), sf), gsw, wp, ws


@pytest.mark.parametrize("m", [1, 4, 16, 64])
def test_full_size_decode_sweep_on_sampled_columns(m, decode_weight):
    """Config 1 at full size (N = 14336, K = 4096, M in {1, 4, 16, 64}): activations
    row-quantized on the GPU per call, weights quantized by the oracle, sampled output columns
    against the oracle."""
    from gpu_util import DEV
    from sparkinfer_b200.gemm import blockscaled
    from sparkinfer_b200.quantization import nvfp4

    n, k = 14336, 4096
    rhs, gsw, wp, ws = decode_weight
    x = seeded_bf16(42 + 1000, (m, k)).to(DEV)
    gsx = O.nvfp4_global_scale(x.float().cpu().numpy())
    plan = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(plan, device=DEV)
    nvfp4.run(plan=plan, x=x, global_scale=torch.tensor([gsx], device=DEV), outputs=outs)
    lhs = (outs.packed_a_view, outs.scale_mma_view(m, k))
    out = blockscaled.mm(lhs, rhs, alpha=_alpha(gsx, gsw), c_dtype="bfloat16", **NVFP4)
    torch.cuda.synchronize()
    cols = np.r_[0:64, n // 2:n // 2 + 64, n - 64:n]
    pa, sa = O.quantize_nvfp4_rows(x.float().cpu().numpy(), gsx)
    ref = O.dequantize_nvfp4(pa, sa, gsx) @ O.dequantize_nvfp4(wp[cols], ws[cols], gsw).T
    got = out[:, :, 0][:, torch.from_numpy(cols).to(DEV)].float().cpu().numpy()
    err = np.abs(got - ref).max()
    assert err <= 1e-2 * np.abs(ref).max()
    assert err <= (2.0 ** -8 + 2.0 ** -16) * np.abs(ref).max()
    assert not torch.isnan(out.float()).any()


@pytest.mark.parametrize("tile", [None, (128, 64), (128, 128), (256, 256)])
def test_config0_nvfp4_128x4096x4096_whole_output_against_oracle(tile):
    """Configuration 0 at its stated size: A = randn, B = randn * 0.02 (seeds 42 and 43),
    both quantized to NVFP4 by the oracle with gs = 448 * 6 / amax, alpha = 1 / (gsA * gsB),
    BF16 out; every output element against the oracle's dequantize-to-FP32 matmul. Runs through
    the automatic route and through each tiled kernel."""
    from gpu_util import DEV, assert_gemm_close, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 128, 4096, 4096
    lhs, gsa, a_deq = nvfp4_operand(seeded_bf16(42, (m, k)))
    rhs, gsb, b_deq = nvfp4_operand(seeded_bf16(43, (n, k), 0.02))
    out = torch.full((m, n, 1), float("nan"), dtype=torch.bfloat16, device=DEV)
    blockscaled.mm(lhs, rhs, out, alpha=_alpha(gsa, gsb), c_dtype="bfloat16", mma_tiler_mn=tile,
                   **NVFP4)
    torch.cuda.synchronize()
    assert_gemm_close(out[:, :, 0], a_deq @ b_deq.T)
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(DEV)


# --------------------------------------------------------------------------------------
# Activation quantizer fused into the decode GEMM
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (5, 512, 512), (8, 4096, 4096), (8, 640, 7168),
                                   (3, 24064, 1024), (7, 200, 384)])
def test_mm_fused_quant_a_mxfp8_equals_quantize_then_mm_bit_for_bit(m, n, k):
    """The in-kernel quantizer must reproduce quantize_rows + mm exactly (same codes, same scale
    bytes, same accumulation order), and both must match the oracle. Shapes cover one CTA per
    tile, tiles split along K over several CTAs, several tiles per CTA (the rows are
    re-quantized per tile) and a ragged N."""
    from gpu_util import DEV, assert_gemm_close, mxfp8_operand
    from sparkinfer_b200._lib.mxfp8_rows import empty_mxfp8_rows_for_dense_gemm, quantize_mxfp8_rows
    from sparkinfer_b200.gemm import blockscaled

    x = seeded_bf16(15 + m, (m, k), 0.25)
    x[0, :32] = 0  # an all-zero block: scale byte 127
    rhs, b_deq = mxfp8_operand(seeded_bf16(16 + n, (n, k), 0.03))
    _, a_deq = mxfp8_operand(x)
    xd = x.to(DEV)
    fused = torch.full((m, n, 1), float("nan"), dtype=torch.bfloat16, device=DEV)
    blockscaled.mm_fused_quant_a(xd, rhs[0], rhs[1], out=fused)
    xq = empty_mxfp8_rows_for_dense_gemm(m, k, device=DEV)
    quantize_mxfp8_rows(xd, xq.values, xq.scale_rows, xq.scale_mma)
    unfused = blockscaled.mm((xq.values.view(m, k, 1), xq.scale_mma), rhs, c_dtype="bfloat16", **MXFP8)
    torch.cuda.synchronize()
    assert_gemm_close(fused[:, :, 0], a_deq @ b_deq.T)
    assert torch.equal(fused.view(torch.int16), unfused.view(torch.int16))
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(DEV)


@pytest.mark.parametrize("m,n,k,groups,row_pad", [
    (1, 128, 256, 2, 0), (4, 512, 512, 5, 0), (8, 1536, 1024, 3, 64), (3, 200, 384, 4, 8),
    (8, 4096, 512, 16, 0),      # 512 weight tiles in one work list (more than SMs: stream-K)
])
def test_mm_fused_quant_a_grouped_equals_the_groups_one_by_one(m, n, k, groups, row_pad):
    """``source [M, groups, K]`` (rows strided when ``row_pad`` > 0), weights ``[N, K, groups]``:
    one launch for all groups must give, per group, what ``mm_fused_quant_a`` gives for that
    group alone, and meet the oracle."""
    from gpu_util import DEV, assert_gemm_close, to_dev
    from sparkinfer_b200._lib import layout
    from sparkinfer_b200.gemm import blockscaled

    backing = torch.zeros((m, groups * k + row_pad), dtype=torch.bfloat16)
    source = backing[:, :groups * k].view(m, groups, k)
    b_vals, b_sw, refs = [], [], []
    for g in range(groups):
        source[:, g] = seeded_bf16(700 + g + m, (m, k), 0.25 * (1 + g))
        b = seeded_bf16(800 + g + n, (n, k), 0.03 / (1 + g)).float().numpy()
        bv, bsr = O.quantize_mxfp8_rows(b)
        b_vals.append(bv); b_sw.append(O.swizzle_scales(bsr, 127))
        av, asr = O.quantize_mxfp8_rows(source[:, g].float().numpy())
        refs.append(O.dequantize_mxfp8(av, asr) @ O.dequantize_mxfp8(bv, bsr).T)
    src_dev = backing.to(DEV)[:, :groups * k].view(m, groups, k)
    b_t = to_dev(np.stack(b_vals)).view(torch.float8_e4m3fn).as_strided((n, k, groups), (k, 1, n * k))
    sfb = layout.convert_sf_to_mma_layout(to_dev(np.concatenate(b_sw)), n, k, groups, 32)
    out = torch.full((groups, m, n), float("nan"), dtype=torch.bfloat16, device=DEV).permute(1, 2, 0)
    got = blockscaled.mm_fused_quant_a_grouped(src_dev, b_t, sfb, groups=groups, out=out)
    torch.cuda.synchronize()
    assert got is out
    for g in range(groups):
        assert_gemm_close(out[:, :, g], refs[g])
        one_sfb = layout.convert_sf_to_mma_layout(to_dev(b_sw[g]), n, k, 1, 32)
        alone = blockscaled.mm_fused_quant_a(
            src_dev[:, g].contiguous(), to_dev(b_vals[g]).view(torch.float8_e4m3fn).view(n, k, 1), one_sfb)
        # Same codes and scales; the two launches may cut K into different numbers of segments
        # (the split depends on how many tiles share the SMs), so FP32 partial sums can
        # associate differently: equal to within one rounding of the output.
        diff = float((alone[:, :, 0].float() - out[:, :, g].float()).abs().max())
        assert diff <= 2.0 ** -8 * float(np.abs(refs[g]).max()), (g, diff)
    with pytest.raises(ValueError, match="both positions and cos_sin_cache"):
        blockscaled.mm_fused_quant_a_grouped(src_dev, b_t, sfb, groups=groups,
                                             positions=torch.zeros(m, dtype=torch.int64, device=DEV))
    with pytest.raises(ValueError, match="source groups"):
        blockscaled.mm_fused_quant_a_grouped(src_dev, b_t, sfb, groups=groups + 1)
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(DEV)


@pytest.mark.parametrize("m,n,k,groups,head,nope,rope,cache_dtype,pos_dtype", [
    (3, 128, 512, 2, 128, 96, 32, torch.float32, torch.int64),
    (3, 128, 512, 2, 128, 96, 32, torch.bfloat16, torch.int64),
    (8, 1024, 2048, 4, 512, 448, 64, torch.float32, torch.int32),
    (1, 256, 1024, 1, 256, 192, 64, torch.bfloat16, torch.int32),
])
def test_mm_fused_quant_a_grouped_inverse_rope(m, n, k, groups, head, nope, rope, cache_dtype, pos_dtype):
    """The inverse-RoPE prologue of the grouped fused quantizer, as the reference tests it
    (tests/gemm/test_gemm_wo_projection.py:340-372, 983-1040): an identity rotation reproduces
    the plain fused call bit for bit; a real rotation equals rotating (oracle, FP32), quantizing
    (oracle) and multiplying the codes with the ordinary grouped GEMM."""
    from gpu_util import DEV, assert_gemm_close, to_dev
    from sparkinfer_b200._lib import layout
    from sparkinfer_b200.gemm import blockscaled

    source = torch.stack([seeded_bf16(900 + g + m, (m, k), 0.125) for g in range(groups)], dim=1).contiguous()
    b_vals, b_sw, b_deq = [], [], []
    for g in range(groups):
        bv, bsr = O.quantize_mxfp8_rows(seeded_bf16(950 + g + n, (n, k), 0.03).float().numpy())
        b_vals.append(bv); b_sw.append(O.swizzle_scales(bsr, 127)); b_deq.append(O.dequantize_mxfp8(bv, bsr))
    src_dev = source.to(DEV)
    b_t = to_dev(np.stack(b_vals)).view(torch.float8_e4m3fn).as_strided((n, k, groups), (k, 1, n * k))
    sfb = layout.convert_sf_to_mma_layout(to_dev(np.concatenate(b_sw)), n, k, groups, 32)
    max_pos = 64
    positions = (torch.arange(7, 7 + m) % max_pos).to(pos_dtype)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rope, 2, dtype=torch.float32) / rope))
    freqs = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv_freq)
    cache = torch.cat([freqs.cos(), freqs.sin()], dim=-1).to(cache_dtype)
    kw = dict(groups=groups, head_dim=head, nope_dim=nope, rope_dim=rope)

    identity = torch.zeros((max_pos, rope), dtype=cache_dtype)
    identity[:, : rope // 2] = 1
    plain = blockscaled.mm_fused_quant_a_grouped(src_dev, b_t, sfb, groups=groups)
    same = blockscaled.mm_fused_quant_a_grouped(src_dev, b_t, sfb, positions=positions.to(DEV),
                                                cos_sin_cache=identity.to(DEV), **kw)
    torch.cuda.synchronize()
    assert torch.equal(plain, same)

    got = blockscaled.mm_fused_quant_a_grouped(src_dev, b_t, sfb, positions=positions.to(DEV),
                                               cos_sin_cache=cache.to(DEV), **kw)
    torch.cuda.synchronize()
    assert not torch.equal(got, plain)
    a_vals, a_sw = [], []
    for g in range(groups):
        rotated = O.inverse_rope_rows(source[:, g].float().numpy(), positions.numpy(),
                                      cache.float().numpy(), head, nope, rope)
        av, asr = O.quantize_mxfp8_rows(rotated)
        a_vals.append(av); a_sw.append(O.swizzle_scales(asr, 127))
        assert_gemm_close(got[:, :, g], O.dequantize_mxfp8(av, asr) @ b_deq[g].T)
    a_t = to_dev(np.stack(a_vals)).view(torch.float8_e4m3fn).as_strided((m, k, groups), (k, 1, m * k))
    sfa = layout.convert_sf_to_mma_layout(to_dev(np.concatenate(a_sw)), m, k, groups, 32)
    unfused = blockscaled.mm((a_t, sfa), (b_t, sfb), ab_dtype="float8_e4m3fn",
                             sf_dtype="float8_e8m0fnu", sf_vec_size=32, c_dtype="bfloat16")
    torch.cuda.synchronize()
    # Same codes and scales (the kernel's rotation and the oracle's agree to the bit); the two
    # launches may split K differently, so equal to within one rounding of the output.
    diff = float((unfused.float() - got.float()).abs().max())
    assert diff <= 2.0 ** -8 * float(got.float().abs().max()), diff
    with pytest.raises(ValueError, match="32-aligned head_dim"):
        blockscaled.mm_fused_quant_a_grouped(src_dev, b_t, sfb, positions=positions.to(DEV),
                                             cos_sin_cache=cache.to(DEV), groups=groups,
                                             head_dim=head, nope_dim=nope - 16, rope_dim=rope)
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(DEV)


@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (4, 512, 512), (16, 14336, 4096), (13, 1024, 2048),
                                   (9, 24064, 1024), (16, 200, 320), (2, 4096, 7168)])
def test_mm_fused_quant_a_nvfp4_equals_quantize_then_mm_bit_for_bit(m, n, k):
    """NVFP4 variant of the fused activation quantizer (M <= 16), against quantization.nvfp4 +
    mm (bit for bit) and the oracle. K = 320 ends in a half-filled unit; zero rows and a zero
    block exercise the zero-scale path."""
    from gpu_util import DEV, assert_gemm_close, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled
    from sparkinfer_b200.quantization import nvfp4

    x = seeded_bf16(25 + m, (m, k))
    x[m - 1, 16:48] = 0
    rhs, gsw, b_deq = nvfp4_operand(seeded_bf16(26 + n, (n, k), 0.02))
    _, gsx, a_deq = nvfp4_operand(x)
    xd = x.to(DEV)
    gs = torch.tensor([gsx], dtype=torch.float32, device=DEV)
    alpha = _alpha(gsx, gsw)
    fused = torch.full((m, n, 1), float("nan"), dtype=torch.bfloat16, device=DEV)
    blockscaled.mm_fused_quant_a_nvfp4(xd, gs, rhs[0], rhs[1], alpha=alpha, out=fused)
    plan = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(plan, device=DEV)
    nvfp4.run(plan=plan, x=xd, global_scale=gs, outputs=outs)
    unfused = blockscaled.mm((outs.packed_a_view, outs.scale_mma_view(m, k)), rhs, alpha=alpha,
                             c_dtype="bfloat16", **NVFP4)
    torch.cuda.synchronize()
    assert_gemm_close(fused[:, :, 0], a_deq @ b_deq.T)
    assert torch.equal(fused.view(torch.int16), unfused.view(torch.int16))
    # A live global scale: CUDA-graph replays read it (and alpha) at run time.
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        blockscaled.mm_fused_quant_a_nvfp4(xd, gs, rhs[0], rhs[1], alpha=alpha, out=fused)
    gs.mul_(0.5)
    alpha.mul_(2.0)
    graph.replay()
    nvfp4.run(plan=plan, x=xd, global_scale=gs, outputs=outs)
    unfused2 = blockscaled.mm((outs.packed_a_view, outs.scale_mma_view(m, k)), rhs, alpha=alpha,
                              c_dtype="bfloat16", **NVFP4)
    torch.cuda.synchronize()
    assert torch.equal(fused.view(torch.int16), unfused2.view(torch.int16))
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(DEV)


def test_mm_fused_quant_a_nvfp4_rejects_what_the_kernel_cannot_do():
    from gpu_util import DEV
    from sparkinfer_b200.gemm import blockscaled

    b = torch.zeros((128, 128, 1), dtype=torch.uint8, device=DEV)
    sfb = torch.zeros((512 * 4,), dtype=torch.uint8, device=DEV)
    gs = torch.ones(1, device=DEV)
    with pytest.raises(ValueError, match="1<=M<=16"):
        blockscaled.mm_fused_quant_a_nvfp4(torch.zeros((17, 256), dtype=torch.bfloat16, device=DEV),
                                           gs, b, sfb)
    with pytest.raises(ValueError, match="contiguous BF16"):
        blockscaled.mm_fused_quant_a_nvfp4(torch.zeros((4, 256), dtype=torch.float16, device=DEV),
                                           gs, b, sfb)
    with pytest.raises(ValueError, match="global_scale"):
        blockscaled.mm_fused_quant_a_nvfp4(torch.zeros((4, 256), dtype=torch.bfloat16, device=DEV),
                                           torch.ones(2, device=DEV), b, sfb)


# --------------------------------------------------------------------------------------
# Stream ordering of the kernels that start before their predecessor has finished
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [128, 256])
def test_decode_gemm_right_after_the_quantization_of_its_own_weight(n):
    """The row quantizers release the next kernel early only for matrices of at most 128 rows,
    and the decode GEMM waits for its predecessor before streaming a weight of at most 128
    rows, so a weight quantized by the kernel launched immediately before the GEMM is never
    read half-written. Both sides of the 128-row rule, repeated to give a race a chance."""
    from gpu_util import DEV, assert_gemm_close, nvfp4_operand
    from sparkinfer_b200.gemm import blockscaled
    from sparkinfer_b200.quantization import nvfp4

    m, k = 4, 8192
    w = seeded_bf16(70 + n, (n, k), 0.02)
    lhs, gsx, a_deq = nvfp4_operand(seeded_bf16(71, (m, k)))
    _, gsw, b_deq = nvfp4_operand(w)
    wd = w.to(DEV)
    gs = torch.tensor([gsw], dtype=torch.float32, device=DEV)
    plan = nvfp4.plan(n, k)
    outs = nvfp4.allocate_outputs(plan, device=DEV)
    alpha = _alpha(gsx, gsw)
    ref = a_deq @ b_deq.T
    for _ in range(5):
        outs.packed_a_storage.zero_()
        outs.scale_storage.zero_()
        nvfp4.run(plan=plan, x=wd, global_scale=gs, outputs=outs)
        out = blockscaled.mm(lhs, (outs.packed_a_view, outs.scale_mma_view(n, k)), alpha=alpha,
                             c_dtype="bfloat16", **NVFP4)
        torch.cuda.synchronize()
        assert_gemm_close(out[:, :, 0], ref)


def test_decode_gemms_on_two_streams_use_separate_workspaces():
    """Every stream gets its own partial-sum workspace, so decode GEMMs whose tiles are split
    over several CTAs may run on two streams at once."""
    from gpu_util import DEV, nvfp4_operand
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 8, 1024, 8192   # 8 tiles, 18 CTAs each: every tile goes through the workspace
    lhs, gsa, _ = nvfp4_operand(seeded_bf16(81, (m, k)))
    weights = [nvfp4_operand(seeded_bf16(82 + i, (n, k), 0.02)) for i in range(2)]
    alphas = [_alpha(gsa, w[1]) for w in weights]
    want = []
    for (rhs, _, _), alpha in zip(weights, alphas):
        want.append(blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="bfloat16", **NVFP4))
        torch.cuda.synchronize()
    streams = [torch.cuda.Stream(device=DEV) for _ in range(2)]
    outs = [torch.empty_like(w) for w in want]
    for _ in range(3):
        for o in outs:
            o.zero_()
        torch.cuda.synchronize()
        for rep in range(20):
            for s, (rhs, _, _), alpha, o in zip(streams, weights, alphas, outs):
                blockscaled.mm(lhs, rhs, o, alpha=alpha, c_dtype="bfloat16", stream=s, **NVFP4)
        torch.cuda.synchronize()
        for o, w_ in zip(outs, want):
            assert torch.equal(o, w_)
    keys = {key for key in launch._WORKSPACES if key[0] == 0}
    assert len({k_[1] for k_ in keys}) >= 3  # the default stream and the two side streams
    launch.check_kernel_status(DEV)


def test_a_timed_out_wait_is_reported_and_the_next_gemm_is_correct():
    """Every device wait in the library is bounded and reports through a status word. The
    library's self-test kernel waits (4096 polls) on a barrier nothing completes, with no copy
    in flight, and raises the word exactly as a GEMM kernel would; the host must turn that into
    an exception, clear the word and the decode counters, and keep working."""
    from gpu_util import DEV, assert_gemm_close, nvfp4_operand
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 8, 1024, 4096
    lhs, gsa, a_deq = nvfp4_operand(seeded_bf16(91, (m, k)))
    rhs, gsb, b_deq = nvfp4_operand(seeded_bf16(92, (n, k), 0.02))
    alpha = _alpha(gsa, gsb)
    blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="bfloat16", **NVFP4)  # creates the workspace
    launch.check_kernel_status(DEV)
    launch.selftest_wait_timeout(DEV, 4096)
    torch.cuda.synchronize()
    assert int(launch.status_buffer(DEV)[0].item()) == 2
    # Pretend the kernel that gave up had left a tile counter behind.
    work = launch.smallm_workspace(1, m, n, k, DEV)
    work[:4].fill_(1)
    with pytest.raises(RuntimeError, match="MMA issuer timed out"):
        launch.check_kernel_status(DEV)
    assert int(launch.status_buffer(DEV)[0].item()) == 0
    assert int(work[:65536].count_nonzero()) == 0
    launch.check_kernel_status(DEV)  # cleared: does not raise again
    out = blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="bfloat16", **NVFP4)
    torch.cuda.synchronize()
    assert_gemm_close(out[:, :, 0], a_deq @ b_deq.T)
    launch.check_kernel_status(DEV)


# --------------------------------------------------------------------------------------
# Epilogues: bias and MXFP8 re-quantization of the output
# --------------------------------------------------------------------------------------
@pytest.mark.parametrize("route,m,n,k,dtype", [
    ("decode", 8, 512, 512, torch.bfloat16), ("decode", 33, 2048, 1024, torch.float16),
    ("decode", 5, 200, 384, torch.float32), ("bn64", 130, 264, 384, torch.bfloat16),
    ("bn128", 256, 512, 256, torch.float32), ("bn256", 300, 504, 640, torch.float16),
    ("pair", 768, 1280, 1024, torch.bfloat16), ("pair", 300, 504, 640, torch.float32),
    ("auto", 2048, 2560, 2048, torch.bfloat16),    # CTA-pair kernel with split leftover tiles
])
def test_fused_bias_equals_a_bias_add_on_the_stored_output(route, m, n, k, dtype):
    """The bias epilogue of every GEMM kernel must give, bit for bit, what adding the bias
    tensor to the kernel's own stored output gives (for BF16 / FP16 outputs that means two
    roundings: the product is rounded to the output type, the sum again)."""
    from gpu_util import DEV, mxfp8_operand
    from sparkinfer_b200._lib import launch
    from sparkinfer_b200._native import BLOCK_N_PAIR, KIND_MXFP8

    (a, sfa), _ = mxfp8_operand(seeded_bf16(m + 2 * k, (m, k), 0.25))
    (b, sfb), _ = mxfp8_operand(seeded_bf16(n + 3 * k, (n, k), 0.03))
    bias = (seeded_bf16(n, (n,), 2.0).float() if dtype == torch.float32 else seeded_bf16(n, (n,), 2.0)
            ).to(dtype).to(DEV)
    kwargs = {"decode": dict(small_m=True), "pair": dict(block_n=BLOCK_N_PAIR), "auto": {}}.get(
        route, dict(block_n=int(route[2:])) if route.startswith("bn") else {})
    alpha = torch.tensor([0.5], dtype=torch.float32, device=DEV)
    plain = torch.empty((m, n), dtype=dtype, device=DEV)
    fused = torch.full((m, n), float("nan"), dtype=dtype, device=DEV)
    launch.gemm_blockscaled(KIND_MXFP8, a, sfa, b, sfb, plain, alpha, m, n, k, **kwargs)
    launch.gemm_blockscaled(KIND_MXFP8, a, sfa, b, sfb, fused, alpha, m, n, k, bias=bias, **kwargs)
    torch.cuda.synchronize()
    launch.check_kernel_status(DEV)
    assert torch.equal(fused, plain + bias)


def test_fused_bias_in_the_block_fp8_gemm_and_its_argument_checks():
    from gpu_util import DEV
    from sparkinfer_b200._lib import launch

    for (m, n, k, dtype) in ((129, 256, 256, torch.bfloat16), (300, 384, 1024, torch.float32),
                             (8, 128, 512, torch.float16)):
        lhs, rhs, _ = _block_fp8_operands(m + n, m, n, k)
        bias = seeded_bf16(n, (n,), 2.0).float().to(dtype).to(DEV)
        plain = torch.empty((m, n), dtype=dtype, device=DEV)
        fused = torch.full((m, n), float("nan"), dtype=dtype, device=DEV)
        launch.gemm_block_fp8(lhs[0][:, :, 0], lhs[1], rhs[0][:, :, 0], rhs[1], plain, None, m, n, k)
        launch.gemm_block_fp8(lhs[0][:, :, 0], lhs[1], rhs[0][:, :, 0], rhs[1], fused, None, m, n, k,
                              bias=bias)
        torch.cuda.synchronize()
        assert torch.equal(fused, plain + bias)
    with pytest.raises(ValueError, match="fused bias"):
        launch.gemm_block_fp8(lhs[0][:, :, 0], lhs[1], rhs[0][:, :, 0], rhs[1], fused, None, m, n, k,
                              bias=bias.float())


@pytest.mark.parametrize("kind,m,n,k,groups", [
    ("mxfp8", 5, 512, 512, 1), ("mxfp8", 16, 1024, 2048, 1), ("nvfp4", 1, 256, 512, 1),
    ("nvfp4", 8, 14336, 1024, 1), ("mxfp8", 4, 64, 256, 2), ("mxfp8", 7, 96, 384, 4),
])
def test_quantized_c_equals_row_quantization_of_the_bf16_output(kind, m, n, k, groups):
    """``mm(..., _quantized_c=...)`` (the reference's small-M quantized-C GEMM,
    b12x/_lib/dense_gemm.py:7497-7588): besides the BF16 output the kernel writes its MXFP8
    re-quantization along N. Codes, row-major scale bytes and scale atoms must equal, bit for
    bit, ``quantization.mxfp8.quantize_rows`` applied to the BF16 output (groups side by side)."""
    from gpu_util import DEV, mxfp8_operand, nvfp4_operand, to_dev
    from sparkinfer_b200._lib import layout
    from sparkinfer_b200._lib.mxfp8_rows import empty_mxfp8_rows_for_dense_gemm, quantize_mxfp8_rows
    from sparkinfer_b200.gemm import blockscaled

    if groups == 1:
        if kind == "mxfp8":
            lhs, _ = mxfp8_operand(seeded_bf16(m + k, (m, k), 0.25))
            rhs, _ = mxfp8_operand(seeded_bf16(n + k, (n, k), 0.05))
            kw, alpha = MXFP8, None
        else:
            lhs, gsa, _ = nvfp4_operand(seeded_bf16(m + k, (m, k), 0.25))
            rhs, gsb, _ = nvfp4_operand(seeded_bf16(n + k, (n, k), 0.05))
            kw, alpha = NVFP4, _alpha(gsa, gsb)
    else:
        av, asw, bv, bsw = [], [], [], []
        for g in range(groups):
            a_q = O.quantize_mxfp8_rows(seeded_bf16(50 + g, (m, k), 0.25 * (g + 1)).float().numpy())
            b_q = O.quantize_mxfp8_rows(seeded_bf16(60 + g, (n, k), 0.05).float().numpy())
            av.append(a_q[0]); bv.append(b_q[0])
            asw.append(O.swizzle_scales(a_q[1], 127)); bsw.append(O.swizzle_scales(b_q[1], 127))
        lhs = (to_dev(np.stack(av)).view(torch.float8_e4m3fn).as_strided((m, k, groups), (k, 1, m * k)),
               layout.convert_sf_to_mma_layout(to_dev(np.concatenate(asw)), m, k, groups, 32))
        rhs = (to_dev(np.stack(bv)).view(torch.float8_e4m3fn).as_strided((n, k, groups), (k, 1, n * k)),
               layout.convert_sf_to_mma_layout(to_dev(np.concatenate(bsw)), n, k, groups, 32))
        kw, alpha = MXFP8, None
    width = n * groups
    q = empty_mxfp8_rows_for_dense_gemm(m, width, device=DEV)
    q.values.view(torch.uint8).fill_(0xEE)
    out = blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="bfloat16",
                         _quantized_c=(q.values, q.scale_rows[0], q.scale_mma), **kw)
    plain = blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="bfloat16", **kw)
    torch.cuda.synchronize()
    assert torch.equal(out, plain), "the BF16 output must not change"
    flat = out.permute(0, 2, 1).reshape(m, width).contiguous()      # [M, L * N], groups side by side
    want = empty_mxfp8_rows_for_dense_gemm(m, width, device=DEV)
    quantize_mxfp8_rows(flat, want.values, want.scale_rows, want.scale_mma)
    torch.cuda.synchronize()
    assert torch.equal(q.values.view(torch.uint8), want.values.view(torch.uint8))
    assert torch.equal(q.scale_rows.view(torch.uint8), want.scale_rows.view(torch.uint8))
    got_atoms = q.scale_mma.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8)
    want_atoms = want.scale_mma.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8)
    assert torch.equal(got_atoms, want_atoms)   # rows >= M keep the pre-filled 127 in both
    with pytest.raises(ValueError, match="quantized C is restricted"):
        blockscaled.mm(lhs, rhs, alpha=alpha, c_dtype="float16",
                       _quantized_c=(q.values, q.scale_rows[0], q.scale_mma), **kw)
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(DEV)


@pytest.mark.parametrize("m,n,k,groups,tile", [
    (4, 384, 512, 5, None),          # decode kernel: 15 weight tiles of 5 groups in one work list
    (33, 200, 256, 3, None),         # decode kernel, ragged N, K split over CTAs
    (130, 264, 384, 2, (128, 64)),   # single-CTA tiled kernel, ragged edges inside each group
    (256, 512, 256, 3, (128, 128)),
    (300, 504, 640, 2, (256, 256)),  # CTA-pair kernel, rows of a group end inside a pair tile
    (512, 1024, 512, 4, None),       # automatic choice
])
def test_mm_grouped_batches_run_in_one_launch(m, n, k, groups, tile):
    """``L`` problems stacked as ``[M, K, L]`` / ``[N, K, L]`` go through ONE kernel launch (the
    tiles of all groups form one work list); every group against the oracle, and group edges
    must not leak: the operands of group g + 1 follow those of group g directly in memory."""
    from gpu_util import DEV, assert_gemm_close, to_dev
    from sparkinfer_b200._lib import layout
    from sparkinfer_b200.gemm import blockscaled

    a_vals, a_sw, b_vals, b_sw, refs = [], [], [], [], []
    for g in range(groups):
        a = seeded_bf16(500 + g, (m, k), 0.25 * (1 + g)).float().numpy()
        b = seeded_bf16(600 + g, (n, k), 0.03 / (1 + g)).float().numpy()
        av, asr = O.quantize_mxfp8_rows(a)
        bv, bsr = O.quantize_mxfp8_rows(b)
        a_vals.append(av); b_vals.append(bv)
        a_sw.append(O.swizzle_scales(asr, 127)); b_sw.append(O.swizzle_scales(bsr, 127))
        refs.append(O.dequantize_mxfp8(av, asr) @ O.dequantize_mxfp8(bv, bsr).T)
    a_t = to_dev(np.stack(a_vals)).view(torch.float8_e4m3fn).as_strided((m, k, groups), (k, 1, m * k))
    b_t = to_dev(np.stack(b_vals)).view(torch.float8_e4m3fn).as_strided((n, k, groups), (k, 1, n * k))
    sfa = layout.convert_sf_to_mma_layout(to_dev(np.concatenate(a_sw)), m, k, groups, 32)
    sfb = layout.convert_sf_to_mma_layout(to_dev(np.concatenate(b_sw)), n, k, groups, 32)
    out = torch.full((groups, m, n), float("nan"), dtype=torch.bfloat16, device=DEV).permute(1, 2, 0)
    blockscaled.mm((a_t, sfa), (b_t, sfb), out, c_dtype="bfloat16", mma_tiler_mn=tile, **MXFP8)
    torch.cuda.synchronize()
    for g in range(groups):
        assert_gemm_close(out[:, :, g], refs[g])
    from sparkinfer_b200._lib.launch import check_kernel_status
    check_kernel_status(DEV)


def test_mm_through_the_custom_ops_equals_the_direct_launch(monkeypatch):
    """A plain eager call launches directly; tracing goes through b12x::dense_gemm_launch and
    b12x::dense_gemm_launch_functional. Both routes must run the same kernel on the same
    arguments: identical bytes, with and without a caller-owned output."""
    from gpu_util import DEV, mxfp8_operand
    from sparkinfer_b200._lib import dense_gemm as dg
    from sparkinfer_b200.gemm import blockscaled

    m, n, k = 48, 384, 512
    lhs, _ = mxfp8_operand(seeded_bf16(901, (m, k), 0.25))
    rhs, _ = mxfp8_operand(seeded_bf16(902, (n, k), 0.03))
    direct = blockscaled.mm(lhs, rhs, c_dtype="bfloat16", **MXFP8)
    direct_out = torch.full((m, n, 1), float("nan"), dtype=torch.bfloat16, device=DEV)
    blockscaled.mm(lhs, rhs, direct_out, c_dtype="bfloat16", **MXFP8)
    monkeypatch.setattr(dg, "_DIRECT_LAUNCH", False)
    via_functional = blockscaled.mm(lhs, rhs, c_dtype="bfloat16", **MXFP8)
    via_op = torch.full((m, n, 1), float("nan"), dtype=torch.bfloat16, device=DEV)
    blockscaled.mm(lhs, rhs, via_op, c_dtype="bfloat16", **MXFP8)
    torch.cuda.synchronize()
    for t in (direct_out, via_functional, via_op):
        assert torch.equal(t.view(torch.int16), direct.view(torch.int16))
