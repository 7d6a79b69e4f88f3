"""The CPU oracle against the fixtures generated from the reference's torch functions
(tests/golden/make_golden.py) and against the reference tests' known-answer vectors."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN, bf16_bits_to_f32
from oracle import blockscaled_oracle as O


@pytest.fixture(scope="module")
def nv():
    return np.load(GOLDEN / "nvfp4_quant.npz")


@pytest.fixture(scope="module")
def mx():
    return np.load(GOLDEN / "mxfp8_quant.npz")


@pytest.mark.parametrize("idx", range(5))
def test_nvfp4_quantizer_matches_reference(nv, idx):
    x = bf16_bits_to_f32(nv[f"x{idx}"])
    gs = nv[f"gs{idx}"][0]
    assert O.nvfp4_global_scale(x) == gs
    packed, scales = O.quantize_nvfp4_rows(x, gs)
    assert np.array_equal(packed, nv[f"packed{idx}"])
    assert np.array_equal(scales, nv[f"scales{idx}"])
    assert np.array_equal(O.swizzle_scales(scales), nv[f"swizzled{idx}"])
    assert np.array_equal(O.unswizzle_scales(nv[f"swizzled{idx}"], *scales.shape), scales)


def test_nvfp4_dequantize_matches_reference(nv):
    got = O.dequantize_nvfp4(nv["packed0"], nv["scales0"], nv["gs0"][0])
    assert np.array_equal(got, nv["dequant0"])


def test_nvfp4_scale_boundary_known_answers(nv):
    """tests/quantization/test_bf16_to_fp4_tma.py:485-560: scale codes 0,1,3,8,7,8,8,9 for the
    hand-built row; a block below half the smallest E4M3 subnormal gets scale 0, payload 0."""
    x = bf16_bits_to_f32(nv["ka_x"])
    packed, scales = O.quantize_nvfp4_rows(x, 1.0)
    assert scales[0].tolist() == [0, 1, 3, 8, 7, 8, 8, 9]
    assert scales[1, 0] == 0 and not packed[1, :8].any()
    assert np.array_equal(packed, nv["ka_packed"])
    assert np.array_equal(scales, nv["ka_scales"])
    assert not ((packed & 0x0F) == 0x08).any() and not ((packed >> 4) == 0x08).any()  # no -0
    assert scales.max() <= 0x7E


def test_nvfp4_zero_global_scale_gives_zero_outputs(nv):
    packed, scales = O.quantize_nvfp4_rows(bf16_bits_to_f32(nv["ka_x"]), 0.0)
    assert not packed.any() and not scales.any()


def test_fp4_tie_breaks():
    """tests/quantization/test_fp4_quantization.py:8-12 (+-3.5 -> +-4) and the full tie table."""
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -3.5], dtype=np.float32)
    want = np.array([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, -4.0], dtype=np.float32)
    assert np.array_equal(O.e2m1_quantize_values(ties), want)


@pytest.mark.parametrize("idx", range(5))
def test_mxfp8_quantizer_matches_reference(mx, idx):
    x = bf16_bits_to_f32(mx[f"x{idx}"])
    values, scale_rows = O.quantize_mxfp8_rows(x)
    assert np.array_equal(values, mx[f"values{idx}"])
    assert np.array_equal(scale_rows, mx[f"scale_rows{idx}"])
    assert np.array_equal(O.swizzle_scales(scale_rows), mx[f"swizzled{idx}"])


def test_mxfp8_zero_block_scale_is_127(mx):
    x = bf16_bits_to_f32(mx["x1"])
    _, scale_rows = O.quantize_mxfp8_rows(x)
    assert scale_rows[3, 1] == 127


def test_mxfp8_dequantize_matches_reference(mx):
    assert np.array_equal(O.dequantize_mxfp8(mx["values0"], mx["scale_rows0"]), mx["dequant0"])


def test_ue8m0_table_over_every_bf16_amax(mx):
    got = O.ue8m0_from_amax(bf16_bits_to_f32(mx["amax_table_bits"]))
    assert np.array_equal(got, mx["amax_table_byte"])


def test_gemm_references_match_reference():
    g = np.load(GOLDEN / "gemm_ref.npz")
    a, b = bf16_bits_to_f32(g["nv_a"]), bf16_bits_to_f32(g["nv_b"])
    gsa, gsb = g["nv_gsa"][0], g["nv_gsb"][0]
    pa, sa = O.quantize_nvfp4_rows(a, gsa)
    pb, sb = O.quantize_nvfp4_rows(b, gsb)
    assert np.array_equal(O.gemm_nvfp4(pa, sa, gsa, pb, sb, gsb), g["nv_out"])
    out = O.gemm_block_fp8(g["bf8_a"], g["bf8_sa"], g["bf8_b"], g["bf8_sb"])
    assert np.array_equal(out, g["bf8_out"])
    # the reference's own _block_fp8_reference (tests/gemm/test_gemm_stack.py:98-113), BF16 out
    assert np.array_equal(O.bf16_round(out), bf16_bits_to_f32(g["bf8_out_bf16_bits"]))


def test_e4m3_codec_matches_torch_in_domain():
    rng = np.random.RandomState(0)
    xs = np.concatenate([
        np.linspace(-464, 464, 100001, dtype=np.float32),
        (rng.randn(100000) * np.exp(rng.randn(100000) * 4)).astype(np.float32),
        np.array([2.0 ** -10, np.nextafter(np.float32(2.0 ** -10), np.float32(1)), 464.0, 448.0],
                 dtype=np.float32),
    ])
    xs = xs[np.abs(xs) <= 464]
    want = torch.from_numpy(xs).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(xs), want)
    codes = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(O.e4m3_decode(codes), nan=-1), np.nan_to_num(ref, nan=-1))
    assert O.e4m3_encode(np.float32(1e6)) == 0x7E  # saturates instead of NaN


def test_swizzle_offsets_agree_with_formula():
    rows, cols = 300, 10
    scales = np.arange(rows * cols, dtype=np.uint32).astype(np.uint8).reshape(rows, cols)
    flat = O.swizzle_scales(scales)
    for r, c in [(0, 0), (31, 3), (32, 0), (127, 9), (128, 4), (299, 9)]:
        assert flat[O.scale_atom_offset(r, c, cols)] == scales[r, c]


@pytest.mark.parametrize("idx", [0, 2, 3])
def test_weight_requantization_matches_reference(idx):
    """Checkpoint block-FP8 weight -> MXFP8 rows: the oracle's re-quantization onto UE8M0
    block scales and the expansion to per-row scale bytes against the reference's
    pack_fp8_block_scaled_weight_mxfp8 (single-group cases; case 3 carries power-of-two
    scales, which the reference passes through without touching the codes)."""
    g = np.load(GOLDEN / "weight_pack.npz")
    m, k, groups = (int(v) for v in g[f"shape{idx}"])
    assert groups == 1
    codes, scale = g[f"w{idx}"], g[f"scale{idx}"]
    exact_pow2 = bool(np.all(np.frexp(scale)[0] == 0.5))
    if exact_pow2:
        new_codes = codes
        block_bytes = (np.round(np.log2(scale)) + 127).astype(np.uint8)
    else:
        new_codes, block_bytes = O.requantize_block_fp8_to_ue8m0(codes, scale)
    rows = O.expand_block_scale_bytes(block_bytes, m, k)
    assert np.array_equal(new_codes, g[f"values{idx}"])
    assert np.array_equal(rows, g[f"scale_rows{idx}"].reshape(m, k // 32))
    assert np.array_equal(O.swizzle_scales(rows, 127), g[f"scale_mma{idx}"])


@pytest.mark.parametrize("idx", range(3))
def test_bmm_oracle_matches_the_reference_tests_torch_reference(idx):
    """Dequantization bit for bit (bytes 0, 1 and 254 included) and the FP64 product."""
    g = np.load(GOLDEN / "bmm_ref.npz")
    values, scales = g[f"values{idx}"], g[f"scales{idx}"]
    deq = O.dequantize_rowwise_mxfp8_bf16(values, scales)
    want = bf16_bits_to_f32(g[f"dequant_bits{idx}"])
    assert np.array_equal(deq.view(np.uint32), want.view(np.uint32))
    got = O.bmm_mxfp8(bf16_bits_to_f32(g[f"lhs_bits{idx}"]), values, scales, bool(g[f"major{idx}"][0]))
    assert got.shape == g[f"product{idx}"].shape
    np.testing.assert_allclose(got, g[f"product{idx}"], rtol=1e-12, atol=0)


def test_bmm_oracle_scale_byte_255_is_nan():
    values = np.full((1, 2, 32), 0x38, dtype=np.uint8)       # 1.0
    scales = np.array([[[255], [127]]], dtype=np.uint8)
    deq = O.dequantize_rowwise_mxfp8_bf16(values, scales)
    assert np.isnan(deq[0, 0]).all() and (deq[0, 1] == 1.0).all()


def test_inverse_rope_oracle_identity_and_formula():
    """cos = 1 / sin = 0 leaves the rows untouched (the case the reference's own test pins,
    tests/gemm/test_gemm_wo_projection.py:340-372); a real rotation touches only the rotary part
    of every head and follows even*cos + odd*sin, odd*cos - even*sin."""
    rng = np.random.RandomState(0)
    x = O.bf16_round(rng.randn(3, 512).astype(np.float32))
    identity = np.zeros((8, 32), np.float32)
    identity[:, :16] = 1
    assert np.array_equal(O.inverse_rope_rows(x, [0, 1, 2], identity, 128, 96, 32), x)
    theta = rng.rand(8, 16).astype(np.float32)
    cache = np.concatenate([np.cos(theta), np.sin(theta)], axis=1).astype(np.float32)
    y = O.inverse_rope_rows(x, [3, 4, 5], cache, 128, 96, 32).reshape(3, 4, 128)
    xr = x.reshape(3, 4, 128)
    assert np.array_equal(y[:, :, :96], xr[:, :, :96])
    c, s = cache[[3, 4, 5], :16][:, None, :], cache[[3, 4, 5], 16:][:, None, :]
    e, o = xr[:, :, 96::2], xr[:, :, 97::2]
    np.testing.assert_allclose(y[:, :, 96::2], e * c + o * s, atol=1e-6)
    np.testing.assert_allclose(y[:, :, 97::2], o * c - e * s, atol=1e-6)
