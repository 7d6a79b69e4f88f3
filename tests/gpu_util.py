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


# --------------------------------------------------------------------------------------
# Whole-output reference on the GPU: dequantize with torch ops, FP32 matmul. Used beside the
# oracle sample where the CPU oracle cannot afford the whole problem.
# --------------------------------------------------------------------------------------
E2M1_LUT = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def unswizzle_atoms(atoms: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Flat 512-byte scale atoms [row_tile][col_tile][32][4][4] -> row-major [rows, cols]."""
    rp, cp = -(-rows // 128) * 128, -(-cols // 4) * 4
    flat = atoms.reshape(-1)[: rp * cp].view(torch.uint8)
    t = flat.view(rp // 128, cp // 4, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return t.reshape(rp, cp)[:rows, :cols].contiguous()


def torch_dequant_nvfp4(packed: torch.Tensor, atoms: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """codes x E4M3 block scales (the global scale is left to alpha), FP32 [rows, k]."""
    packed = packed.reshape(rows, k // 2).view(torch.uint8)
    lut = torch.tensor(E2M1_LUT, dtype=torch.float32, device=packed.device)
    vals = torch.stack((lut[(packed & 0xF).long()], lut[(packed >> 4).long()]), dim=-1).view(rows, k)
    scales = unswizzle_atoms(atoms, rows, k // 16).view(torch.float8_e4m3fn).float()
    return (vals.view(rows, k // 16, 16) * scales[:, :, None]).view(rows, k)


def torch_dequant_mxfp8(values: torch.Tensor, scale_rows: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """E4M3 codes x 2^(byte - 127) from the row-major UE8M0 bytes [rows, k / 32]."""
    v = values.reshape(rows, k).view(torch.float8_e4m3fn).float()
    scales = torch.exp2(scale_rows.reshape(rows, k // 32).view(torch.uint8).float() - 127.0)
    return (v.view(rows, k // 32, 32) * scales[:, :, None]).view(rows, k)


def assert_whole_output_close(got: torch.Tensor, a_deq: torch.Tensor, b_deq: torch.Tensor,
                              alpha: float = 1.0, *, out_dtype=torch.bfloat16, chunk: int = 4096):
    """max|got - alpha * a_deq @ b_deq^T| <= (eps_out + 2^-16) * max|ref| over EVERY output
    element, and no NaN left from a NaN-prefilled output (a tile never written)."""
    assert not torch.isnan(got.float()).any(), "part of the output was never written"
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        worst, scale = 0.0, 0.0
        for r0 in range(0, a_deq.shape[0], chunk):
            ref = (a_deq[r0:r0 + chunk] @ b_deq.T) * alpha
            scale = max(scale, float(ref.abs().max()))
            worst = max(worst, float((got[r0:r0 + chunk].float() - ref).abs().max()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -20}[out_dtype]
    assert worst <= 1e-2 * scale, (worst, scale)
    assert worst <= (eps + 2.0 ** -16) * scale + 1e-30, (worst, scale)
    return worst, scale
