"""Helpers shared by the GPU parity tests: oracle-side operand construction and uploads."""

from __future__ import annotations

import numpy as np
import torch

from oracle import blockscaled_oracle as O
from sparkinfer_b200._lib import layout

DEV = torch.device("cuda:0")


def to_dev(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def nvfp4_operand(x_bf16: torch.Tensor, gs=None):
    """Oracle-quantized NVFP4 operand: (``(codes[M,K/2,1], sf_view)``, gs, dequantized FP32)."""
    xf = x_bf16.float().numpy()
    gs = O.nvfp4_global_scale(xf) if gs is None else np.float32(gs)
    packed, scales = O.quantize_nvfp4_rows(xf, gs)
    m, k = xf.shape
    sf = layout.convert_sf_to_mma_layout(to_dev(O.swizzle_scales(scales, 0)), m, k, 1, 16)
    codes = to_dev(packed).reshape(m, k // 2, 1)
    return (codes, sf), gs, O.dequantize_nvfp4(packed, scales, gs)


def mxfp8_operand(x_bf16: torch.Tensor):
    """Oracle-quantized MXFP8 operand: (``(codes[M,K,1], sf_view)``, dequantized FP32)."""
    xf = x_bf16.float().numpy()
    values, scale_rows = O.quantize_mxfp8_rows(xf)
    m, k = xf.shape
    sf = layout.convert_sf_to_mma_layout(to_dev(O.swizzle_scales(scale_rows, 127)), m, k, 1, 32)
    codes = to_dev(values).view(torch.float8_e4m3fn).reshape(m, k, 1)
    return (codes, sf.view(torch.float8_e8m0fnu)), O.dequantize_mxfp8(values, scale_rows)


def assert_gemm_close(got: torch.Tensor, ref: np.ndarray, *, out_dtype=torch.bfloat16):
    """The path's stated tolerance: max|err| <= 1e-2 * max|ref| (FP32 dequantize-matmul
    reference), plus a much tighter bound that catches a wrong scale or a dropped k-block:
    FP32 accumulation error plus one output rounding."""
    g = got.float().cpu().numpy()
    assert not np.isnan(g).any()
    scale = float(np.abs(ref).max())
    err = float(np.abs(g - ref).max())
    assert err <= 1e-2 * scale, (err, scale)
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -20}[out_dtype]
    assert err <= (eps + 2.0 ** -18) * scale + 1e-30, (err, scale)
