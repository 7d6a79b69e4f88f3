"""mxfp8_linear and block_fp8_linear on the GPU against the oracle composition
"quantize rows -> dequantize -> FP32 matmul" (the reference's tests/gemm/test_mxfp8_linear.py
:77-116 and tests/gemm/test_block_fp8_linear.py:50-114)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import seeded_bf16
from oracle import blockscaled_oracle as O

pytestmark = pytest.mark.gpu


def _modelopt_weight(seed, n, k, scale=1.0 / 8):
    """ModelOpt-style MXFP8 weight built by the oracle quantizer: (values e4m3, scales u8)."""
    from gpu_util import to_dev

    w = seeded_bf16(seed, (n, k), scale).float().numpy()
    values, scale_rows = O.quantize_mxfp8_rows(w)
    return to_dev(values).view(torch.float8_e4m3fn), to_dev(scale_rows), O.dequantize_mxfp8(values, scale_rows)


def _quantized_activation_reference(x: torch.Tensor, padded_k: int) -> np.ndarray:
    xf = np.zeros((x.shape[0], padded_k), dtype=np.float32)
    xf[:, : x.shape[1]] = x.float().numpy()
    return O.dequantize_mxfp8(*O.quantize_mxfp8_rows(xf))


@pytest.mark.parametrize("tokens,k,n", [(7, 128, 32), (3, 160, 40), (129, 256, 256), (16, 4096, 512)])
def test_mxfp8_linear_matches_quantized_reference(tokens, k, n):
    from gpu_util import DEV, assert_gemm_close
    from sparkinfer_b200.gemm import mxfp8_linear

    x = seeded_bf16(tokens + k, (tokens, k), 0.25)
    w_values, w_scale, w_deq = _modelopt_weight(n + k, n, k)
    packed = mxfp8_linear.pack_weight(w_values, w_scale)
    padded_k = -(-k // 128) * 128
    assert packed.in_features == k and packed.padded_in_features == padded_k
    assert packed.weight.values.shape == (n, padded_k)
    assert packed.weight.scale_rows.shape == (1, n, padded_k // 32)
    assert torch.equal(packed.weight.scale_rows.view(torch.uint8)[0, :, : k // 32], w_scale)
    assert (packed.weight.scale_rows.view(torch.uint8)[0, :, k // 32:] == 127).all()
    out = mxfp8_linear.mm(x.to(DEV), packed)
    torch.cuda.synchronize()
    assert out.shape == (tokens, n) and out.dtype == torch.bfloat16
    w_pad = np.zeros((n, padded_k), dtype=np.float32)
    w_pad[:, :k] = w_deq
    assert_gemm_close(out, _quantized_activation_reference(x, padded_k) @ w_pad.T)


def test_mxfp8_linear_bias_leading_dims_and_empty():
    from gpu_util import DEV, assert_gemm_close
    from sparkinfer_b200.gemm import mxfp8_linear

    k, n = 256, 128
    w_values, w_scale, w_deq = _modelopt_weight(3, n, k)
    packed = mxfp8_linear.pack_weight(w_values, w_scale)
    x = seeded_bf16(4, (2, 5, k), 0.25)
    bias = seeded_bf16(5, (n,)).to(DEV)
    out = mxfp8_linear.mm(x.to(DEV), packed, bias=bias)
    assert out.shape == (2, 5, n)
    ref = _quantized_activation_reference(x.reshape(10, k), k) @ w_deq.T
    plain = mxfp8_linear.mm(x.to(DEV), packed)
    assert_gemm_close(plain.reshape(10, n), ref)
    assert torch.equal(out, plain + bias)
    assert mxfp8_linear.mm(torch.empty((0, k), dtype=torch.bfloat16, device=DEV), packed).shape == (0, n)
    with pytest.raises(ValueError, match="does not match"):
        mxfp8_linear.mm(torch.zeros((2, 128), dtype=torch.bfloat16, device=DEV), packed)
    with pytest.raises(TypeError):
        mxfp8_linear.mm(x.to(DEV), object())


def _block_fp8_checkpoint(seed, n, k):
    """DeepSeek-style weight: E4M3 codes + FP32 128x128 scales (amax / 448)."""
    from gpu_util import to_dev

    w = seeded_bf16(seed, (n, k), 0.05).float().numpy()
    codes, scales = O.quantize_block_fp8(w, 128, 128)
    return to_dev(codes).view(torch.float8_e4m3fn), to_dev(scales), codes, scales


@pytest.mark.parametrize("tokens", [1, 8, 9, 200])
def test_block_fp8_linear_plan_bind_run(tokens):
    from gpu_util import DEV, assert_gemm_close
    from sparkinfer_b200._lib.mxfp8_rows import empty_dense_gemm_mnl_view
    from sparkinfer_b200.gemm import block_fp8_linear as bfl

    k, n = 512, 384
    w_codes, w_scales, codes_np, scales_np = _block_fp8_checkpoint(21, n, k)
    weight = bfl.pack_weight(w_codes, w_scales)
    assert weight.in_features == k and weight.out_features == n
    # The packed weight keeps the information of the checkpoint: its dequantized rows are the
    # re-quantization of codes * scale onto power-of-two block scales.
    w_rec = O.e4m3_decode(codes_np).reshape(n // 128, 128, k // 128, 128) * scales_np[:, None, :, None]
    w_deq = O.dequantize_mxfp8(weight.weight.values.view(torch.uint8).cpu().numpy(),
                               weight.weight.scale_rows.view(torch.uint8)[0].cpu().numpy())
    assert np.abs(w_deq - w_rec.reshape(n, k)).max() <= 2.0 ** -4 * np.abs(w_rec).max()
    byte = weight.weight.scale_rows.view(torch.uint8)[0].cpu().numpy()
    assert (byte.reshape(n // 128, 128, k // 128, 4) == byte.reshape(n // 128, 128, k // 128, 4)[:, :1, :, :1]).all()

    x = seeded_bf16(22 + tokens, (tokens, k), 0.25)
    plan = bfl.plan(bfl.Caps(device=DEV, max_tokens=256, in_features=k, out_features=n))
    spec = plan.scratch_specs()[0]
    scratch = torch.empty(spec.shape, dtype=spec.dtype, device=spec.device)
    output = empty_dense_gemm_mnl_view(tokens, n, 1, device=DEV, dtype=torch.bfloat16)
    binding = bfl.bind(plan, scratch=scratch, source=x.to(DEV), packed_weight=weight, output=output)
    y = bfl.run(binding=binding)
    torch.cuda.synchronize()
    assert y.shape == (tokens, n) and y.data_ptr() == output.data_ptr()
    ref = _quantized_activation_reference(x, k) @ w_deq.T
    assert_gemm_close(y, ref)
    # one-shot form gives the same bits
    y2 = bfl.run(x.to(DEV), weight)
    assert torch.equal(y2, y)
    # bound path under CUDA-graph capture (tests/gemm/test_block_fp8_linear.py:70-114)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        binding.run()
    output.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(output[:, :, 0], y2)


def test_block_fp8_quantize_input_and_prewarm():
    from gpu_util import DEV
    from sparkinfer_b200.gemm import block_fp8_linear as bfl

    x = seeded_bf16(31, (20, 256), 0.25)
    xq = bfl.quantize_input(x.to(DEV))
    ref_values, ref_rows = O.quantize_mxfp8_rows(x.float().numpy())
    assert np.array_equal(xq.values.view(torch.uint8).cpu().numpy(), ref_values)
    assert np.array_equal(xq.scale_rows.view(torch.uint8)[0].cpu().numpy(), ref_rows)
    assert xq.scale_mma.shape == (32, 4, 1, 4, 2, 1)
    w_codes, w_scales, _, _ = _block_fp8_checkpoint(32, 128, 256)
    bfl.prewarm(bfl.pack_weight(w_codes, w_scales), [1, 4, 0, 4])


def _tensor_fp8_case(seed, tokens, k, n, output_scale=0.0002):
    """E4M3 source and weight (values clamped to +-4 as in the reference's test) and the FP32
    product they stand for: the E4M3 codes decoded by the oracle, matmul in FP32, one scale."""
    from gpu_util import DEV, to_dev

    def codes(s, shape):
        x = np.clip(seeded_bf16(s, shape).float().numpy(), -4.0, 4.0)
        return O.e4m3_encode(x)

    a, w = codes(seed, (tokens, k)), codes(seed + 1, (n, k))
    ref = (O.e4m3_decode(a) @ O.e4m3_decode(w).T) * np.float32(output_scale)
    scale = torch.tensor([output_scale], dtype=torch.float32, device=DEV)
    return (to_dev(a).view(torch.float8_e4m3fn), to_dev(w).view(torch.float8_e4m3fn), scale, ref)


@pytest.mark.parametrize("tokens,k,n,out_dtype", [
    (7, 128, 64, torch.bfloat16), (3, 160, 40, torch.bfloat16), (130, 512, 384, torch.float16),
    (16, 4096, 1024, torch.bfloat16),
])
def test_tensor_fp8_linear_matches_fp32_product(tokens, k, n, out_dtype):
    """tests/gemm/test_tensor_fp8_linear.py:36-75: rtol 1e-2 / atol 2e-3 against
    (source @ weight^T) * output_scale; K = 160 is padded to 256 with zero codes."""
    from gpu_util import assert_gemm_close
    from sparkinfer_b200.gemm import tensor_fp8_linear

    source, weight, scale, ref = _tensor_fp8_case(tokens + k + n, tokens, k, n)
    packed = tensor_fp8_linear.pack_weight(weight, scale)
    assert packed.in_features == k and packed.padded_in_features == -(-k // 128) * 128
    assert packed.values.shape == (n, packed.padded_in_features)
    assert torch.count_nonzero(packed.values.view(torch.uint8)[:, k:]) == 0
    out = tensor_fp8_linear.mm(source, packed, out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert out.shape == (tokens, n) and out.dtype == out_dtype
    got = out.float().cpu().numpy()
    assert np.allclose(got, ref, rtol=1e-2, atol=2e-3)
    assert_gemm_close(out, ref, out_dtype=out_dtype)


def test_tensor_fp8_linear_ignores_scale_storage_bias_leading_dims_graph_and_errors():
    """tests/gemm/test_tensor_fp8_linear.py:78-170: the block-scale storage of the packed
    weight is not read (plain FP8), bias and leading dimensions, empty input, CUDA-graph
    replay after prewarm, and the host-side argument errors."""
    from dataclasses import replace

    from gpu_util import DEV
    from sparkinfer_b200.gemm import tensor_fp8_linear

    source, weight, scale, ref = _tensor_fp8_case(77, 4, 128, 64)
    packed = tensor_fp8_linear.pack_weight(weight, scale)
    zeroed = replace(packed, scale_mma=torch.zeros_like(packed.scale_mma))
    out = tensor_fp8_linear.mm(source, zeroed)
    torch.cuda.synchronize()
    assert np.allclose(out.float().cpu().numpy(), ref, rtol=1e-2, atol=2e-3)

    bias = torch.linspace(-1, 1, 64, device=DEV).to(torch.bfloat16)
    out3 = tensor_fp8_linear.mm(source.view(2, 2, 128), packed, bias=bias)
    assert out3.shape == (2, 2, 64)
    want = (torch.from_numpy(ref).to(DEV).to(torch.bfloat16) + bias).view(2, 2, 64)
    assert torch.allclose(out3.float(), want.float(), rtol=1e-2, atol=1e-2)
    empty = tensor_fp8_linear.mm(source[:0], packed)
    assert empty.shape == (0, 64)

    assert tensor_fp8_linear.prewarm(packed, [4, 4, 0]) == 1
    eager = tensor_fp8_linear.mm(source, packed).clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = tensor_fp8_linear.mm(source, packed)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, eager)

    with pytest.raises(ValueError, match="float8_e4m3fn"):
        tensor_fp8_linear.mm(source.view(torch.uint8).to(torch.bfloat16), packed)
    with pytest.raises(ValueError, match="does not match"):
        tensor_fp8_linear.mm(source[:, :64], packed)
    with pytest.raises(TypeError):
        tensor_fp8_linear.mm(source, weight)
    with pytest.raises(ValueError, match="bf16/fp16"):
        tensor_fp8_linear.mm(source, packed, out_dtype=torch.float32)
    with pytest.raises(ValueError, match="one float32"):
        tensor_fp8_linear.pack_weight(weight, torch.ones(2, device=DEV))
    with pytest.raises(ValueError, match="multiple of 32"):
        tensor_fp8_linear.pack_weight(weight[:, :48], scale)


# --------------------------------------------------------------------------------------
# Weight packing on the device (one kernel) against the reference's outputs and the torch
# restatement of the same arithmetic
# --------------------------------------------------------------------------------------
def _packed_bytes(rows):
    values = rows.values if rows.values.ndim == 2 else rows.values.permute(2, 0, 1)
    physical = rows.scale_mma.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8)
    return (values.contiguous().view(torch.uint8).cpu().numpy(),
            rows.scale_rows.contiguous().view(torch.uint8).cpu().numpy(),
            physical.cpu().numpy().reshape(-1))


@pytest.mark.parametrize("idx", [0, 1, 2, 3])
def test_device_weight_packer_matches_reference_fixture(idx):
    """Same fixture as the CPU test of the torch restatement: outputs of the reference's own
    pack_fp8_block_scaled_weight_mxfp8 (re-quantized codes, per-row scale bytes, scale atoms;
    one and two groups, ragged row count, power-of-two scales passed through)."""
    from conftest import GOLDEN
    from sparkinfer_b200._lib import mxfp8_rows as mr

    g = np.load(GOLDEN / "weight_pack.npz")
    m, k, groups = (int(v) for v in g[f"shape{idx}"])
    weight = torch.from_numpy(g[f"w{idx}"]).view(torch.float8_e4m3fn).to("cuda:0")
    scale = torch.from_numpy(g[f"scale{idx}"]).to("cuda:0")
    values, scale_rows, atoms = _packed_bytes(
        mr.pack_fp8_block_scaled_weight_mxfp8(weight, scale, m=m, k=k, num_groups=groups))
    assert np.array_equal(values, g[f"values{idx}"])
    assert np.array_equal(scale_rows, g[f"scale_rows{idx}"])
    assert np.array_equal(atoms, g[f"scale_mma{idx}"])


@pytest.mark.parametrize("m,k,groups,spread", [
    (384, 512, 1, 1.0), (200, 256, 3, 1e-3), (1000, 1024, 1, 1e4), (128, 128, 2, 1e-30),
    (77, 384, 1, 1e30),
])
def test_device_weight_packer_equals_torch_restatement(monkeypatch, m, k, groups, spread):
    """Random checkpoint-style weights with scales over a wide range (down to values whose
    blocks land on the smallest UE8M0 bytes, up to the largest), and blocks of zeros."""
    from sparkinfer_b200._lib import mxfp8_rows as mr

    gen = torch.Generator().manual_seed(m * 7 + k)
    w = (torch.randn((groups * m, k), generator=gen) * 60).clamp(-448, 448).to(torch.float8_e4m3fn)
    w[: min(m, 128), :128] = 0                       # one all-zero block
    blocks = (groups * -(-m // 128), k // 128)
    scale = (torch.rand(blocks, generator=gen) + 0.25) * spread * torch.exp2(
        torch.randint(-6, 7, blocks, generator=gen).float())
    got = _packed_bytes(mr.pack_fp8_block_scaled_weight_mxfp8(
        w.to("cuda:0"), scale.to("cuda:0"), m=m, k=k, num_groups=groups))
    monkeypatch.setattr(mr, "_check_gpu_tensor", lambda name, tensor: None)
    want = _packed_bytes(mr.pack_fp8_block_scaled_weight_mxfp8(w, scale, m=m, k=k, num_groups=groups))
    for a, b, what in zip(got, want, ("codes", "scale rows", "scale atoms")):
        assert np.array_equal(a, b), what
    # power-of-two scales: codes pass through untouched
    pow2 = torch.exp2(torch.randint(-20, 20, blocks, generator=gen).float())
    got = _packed_bytes(mr.pack_fp8_block_scaled_weight_mxfp8(
        w.to("cuda:0"), pow2.to("cuda:0"), m=m, k=k, num_groups=groups))
    want = _packed_bytes(mr.pack_fp8_block_scaled_weight_mxfp8(w, pow2, m=m, k=k, num_groups=groups))
    for a, b, what in zip(got, want, ("codes", "scale rows", "scale atoms")):
        assert np.array_equal(a, b), what
