"""MXFP8 row operands: storage contracts, the row quantizer entry point and one-time weight
packing.

Mirrors the hot-path parts of b12x/gemm/_shared/wo_mxfp8.py (:51-69 ``MXFP8Rows``, :717-830
storage helpers, :844-987 scale expansion/packing, :990-1187 block-FP8 weight re-quantization)
and b12x/_lib/quant/mxfp8_rows.py:398-434 (``quantize_mxfp8_rows_cute``). The per-call work
(quantizing activation rows) is a CUDA kernel; weight packing is load-time torch code, as in
the reference.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import launch
from .launch import cuda_stream_to_int

FP8_E4M3_MAX = 448.0
MXFP8_SCALE_VEC_SIZE = 32
MXFP8_SCALE_ROW_TILE = 128
MXFP8_SCALE_K_TILE = 4


@dataclass(frozen=True)
class MXFP8Rows:
    """Row-wise MXFP8 operand for ``dense_gemm``.

    ``values``: ``[M, K]`` (or ``[M, K, L]`` over physical ``[L, M, K]``) E4M3;
    ``scale_rows``: ``[L, M, K/32]`` UE8M0; ``scale_mma``: the strided
    ``(32, 4, ceil(M/128), 4, ceil(K/128), L)`` view the GEMM consumes.
    """

    values: torch.Tensor
    scale_rows: torch.Tensor
    scale_mma: torch.Tensor
    values_tiled: torch.Tensor | None = None


def _check_gpu_tensor(name: str, tensor: torch.Tensor) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be on CUDA")


def _check_mxfp8_k(k: int) -> None:
    if k <= 0 or k % 128 != 0:
        raise ValueError(f"MXFP8 dense_gemm K must be a positive multiple of 128, got {k}")


def empty_dense_gemm_mnl_view(m: int, n: int, l: int, *, device, dtype: torch.dtype) -> torch.Tensor:
    """``[M, N, L]`` view backed by physical ``[L, M, N]`` storage."""
    if m <= 0 or n <= 0 or l <= 0:
        raise ValueError("m, n, and l must be positive")
    if l == 1:
        return torch.empty((m, n, 1), device=device, dtype=dtype)
    return torch.empty((l, m, n), device=device, dtype=dtype).as_strided((m, n, l), (n, 1, m * n))


def empty_mxfp8_rows_bases(m: int, k: int, *, num_groups: int, device,
                           initialize_scales: bool = True):
    """The three contiguous buffers behind an :class:`MXFP8Rows`:
    ``(values [M,K] e4m3, scale_rows [L,M,K/32] u8, scale atoms [L,mt,kt,32,4,4] u8)``.
    Scales start at 127 (UE8M0 1.0) unless ``initialize_scales`` is false."""
    if m <= 0 or k <= 0 or num_groups <= 0:
        raise ValueError("m, k, and num_groups must be positive")
    _check_mxfp8_k(k)
    vshape = (m, k) if num_groups == 1 else (num_groups, m, k)
    values_base = torch.empty(vshape, device=device, dtype=torch.float8_e4m3fn)
    make = (lambda s: torch.full(s, 127, dtype=torch.uint8, device=device)) if initialize_scales \
        else (lambda s: torch.empty(s, dtype=torch.uint8, device=device))
    scale_rows_base = make((num_groups, m, k // MXFP8_SCALE_VEC_SIZE))
    m_tiles = math.ceil(m / MXFP8_SCALE_ROW_TILE)
    k_tiles = math.ceil((k // MXFP8_SCALE_VEC_SIZE) / MXFP8_SCALE_K_TILE)
    scale_physical_base = make((num_groups, m_tiles, k_tiles, 32, 4, 4))
    return values_base, scale_rows_base, scale_physical_base


def mxfp8_rows_from_bases(values_base, scale_rows_base, scale_physical_base, m: int, k: int, *,
                          num_groups: int) -> MXFP8Rows:
    """Rebuild the dense-GEMM views over the contiguous bases (views only)."""
    values = values_base if num_groups == 1 else values_base.as_strided(
        (m, k, num_groups), (k, 1, m * k))
    return MXFP8Rows(
        values=values,
        scale_rows=scale_rows_base.view(torch.float8_e8m0fnu),
        scale_mma=scale_physical_base.view(torch.float8_e8m0fnu).permute(3, 4, 1, 5, 2, 0),
    )


def empty_mxfp8_rows_for_dense_gemm(m: int, k: int, *, num_groups: int = 1, device) -> MXFP8Rows:
    bases = empty_mxfp8_rows_bases(m, k, num_groups=num_groups, device=device)
    return mxfp8_rows_from_bases(*bases, m, k, num_groups=num_groups)


def _check_mxfp8_rows_storage(out: MXFP8Rows, *, m: int, k: int, num_groups: int) -> None:
    _check_gpu_tensor("out.values", out.values)
    _check_gpu_tensor("out.scale_rows", out.scale_rows)
    _check_gpu_tensor("out.scale_mma", out.scale_mma)
    if out.values.dtype != torch.float8_e4m3fn:
        raise ValueError(f"out.values must be float8_e4m3fn, got {out.values.dtype}")
    for name, t in (("scale_rows", out.scale_rows), ("scale_mma", out.scale_mma)):
        if t.dtype != torch.float8_e8m0fnu:
            raise ValueError(f"out.{name} must be float8_e8m0fnu, got {t.dtype}")
    want_values = (m, k) if num_groups == 1 else (m, k, num_groups)
    if tuple(out.values.shape) != want_values:
        raise ValueError(f"out.values must have shape {want_values}, got {tuple(out.values.shape)}")
    sf_k = k // MXFP8_SCALE_VEC_SIZE
    if tuple(out.scale_rows.shape) != (num_groups, m, sf_k):
        raise ValueError(
            f"out.scale_rows must have shape {(num_groups, m, sf_k)}, got {tuple(out.scale_rows.shape)}")
    want_mma = (32, 4, math.ceil(m / 128), 4, math.ceil(sf_k / 4), num_groups)
    if tuple(out.scale_mma.shape) != want_mma:
        raise ValueError(
            f"out.scale_mma must have shape {want_mma}, got {tuple(out.scale_mma.shape)}")
    if not out.values.is_contiguous() and num_groups == 1:
        raise ValueError("out.values must be contiguous")
    if not out.scale_rows.is_contiguous():
        raise ValueError("out.scale_rows must be contiguous")


def quantize_mxfp8_rows(source: torch.Tensor, values: torch.Tensor, scale_rows: torch.Tensor,
                        scale_mma: torch.Tensor, *, value_order: str = "linear",
                        stream: object = None) -> None:
    """Quantize contiguous BF16/FP16 ``[M, K]`` rows into caller-owned MXFP8 tensors.

    Same contract as the reference's ``quantize_mxfp8_rows_cute``: ``values [M,K]`` E4M3,
    ``scale_rows [M,K/32]`` (or ``[1,M,K/32]``) UE8M0 and the 6-D ``scale_mma`` view are written
    in place; nothing is allocated. Padding bytes of ``scale_mma`` (rows >= M) end up 127.
    """
    if source.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"MXFP8 quantizer requires BF16 or FP16 input, got {source.dtype}")
    if source.ndim != 2 or not source.is_contiguous():
        raise ValueError("MXFP8 quantizer requires contiguous [M,K] input")
    if value_order != "linear":
        raise NotImplementedError("only value_order='linear' belongs to the dense GEMM path")
    m, k = map(int, source.shape)
    if k % MXFP8_SCALE_VEC_SIZE != 0:
        raise ValueError(f"K must be a multiple of {MXFP8_SCALE_VEC_SIZE}, got {k}")
    if values.numel() != m * k or values.element_size() != 1 or not values.is_contiguous():
        raise ValueError(f"values must be a contiguous one-byte tensor of {m * k} elements")
    if scale_rows is not None and (scale_rows.numel() != m * (k // 32) or not scale_rows.is_contiguous()):
        raise ValueError(f"scale_rows must be contiguous with {m * (k // 32)} elements")
    need = math.ceil(m / 128) * math.ceil(k / 128) * 512
    if scale_mma is not None and scale_mma.numel() < need:
        raise ValueError(f"scale_mma must hold at least {need} bytes, got {scale_mma.numel()}")
    if m == 0:
        return
    launch.quantize_mxfp8_rows(source, values, scale_rows, scale_mma,
                               stream_int=cuda_stream_to_int(stream))


# ----------------------------------------------------------------------------------------
# One-time weight packing (torch; load time, not on the serving path)
# ----------------------------------------------------------------------------------------
def _scale_u8_from_max_abs(max_abs: torch.Tensor) -> torch.Tensor:
    """UE8M0 byte = 127 + clamp(ceil(log2(amax/448)), -127, 127); 127 for zero blocks."""
    safe = torch.where(max_abs > 0, max_abs.to(torch.float32) / FP8_E4M3_MAX,
                       torch.ones_like(max_abs, dtype=torch.float32))
    return (torch.ceil(torch.log2(safe)).clamp(-127, 127) + 127).to(torch.uint8)


def _scale_to_e8m0_u8(scale: torch.Tensor) -> torch.Tensor:
    if scale.dtype == torch.float8_e8m0fnu:
        return scale.view(torch.uint8)
    if scale.dtype == torch.uint8:
        return scale
    if not scale.is_floating_point():
        raise ValueError(f"scale must be e8m0, uint8, or floating-point, got {scale.dtype}")
    safe = torch.where(scale > 0, scale.to(torch.float32), torch.ones_like(scale, dtype=torch.float32))
    return (torch.round(torch.log2(safe)).clamp(-127, 127) + 127).to(torch.uint8)


def _expand_block_scales_to_mxfp8_rows(scale: torch.Tensor, *, m: int, k: int,
                                       num_groups: int) -> torch.Tensor:
    """128x128 block scales -> per-row, per-32-column UE8M0 ``[L, M, K/32]``."""
    _check_mxfp8_k(k)
    m_tiles = math.ceil(m / 128)
    k_tiles = k // 128
    if scale.numel() != num_groups * m_tiles * k_tiles:
        raise ValueError(
            f"block scale must have {num_groups * m_tiles * k_tiles} entries "
            f"([{num_groups}*{m_tiles}, {k_tiles}]); got {tuple(scale.shape)}")
    block_u8 = _scale_to_e8m0_u8(scale).reshape(num_groups, m_tiles, k_tiles)
    rows = block_u8[:, :, None, :, None].expand(num_groups, m_tiles, 128, k_tiles, 4)
    rows = rows.reshape(num_groups, m_tiles * 128, k_tiles * 4)[:, :m, : k // 32].contiguous()
    return rows.view(torch.float8_e8m0fnu)


def pack_mxfp8_scales_for_dense_gemm(scale_rows: torch.Tensor, *, m: int, k: int,
                                     num_groups: int = 1) -> torch.Tensor:
    """Row-major UE8M0 scales -> 6-D MMA view; padding rows/columns are 127 (UE8M0 1.0)."""
    if scale_rows.dtype == torch.uint8:
        scale_rows = scale_rows.view(torch.float8_e8m0fnu)
    if scale_rows.dtype != torch.float8_e8m0fnu:
        raise ValueError(f"scale_rows must be uint8/e8m0, got {scale_rows.dtype}")
    _check_mxfp8_k(k)
    sf_k = k // 32
    if scale_rows.numel() != num_groups * m * sf_k:
        raise ValueError(
            f"scale_rows must have shape {(num_groups, m, sf_k)}, got {tuple(scale_rows.shape)}")
    grouped = scale_rows.reshape(num_groups, m, sf_k).view(torch.uint8)
    m_tiles, k_tiles = math.ceil(m / 128), math.ceil(sf_k / 4)
    padded = torch.full((num_groups, m_tiles * 128, k_tiles * 4), 127, dtype=torch.uint8,
                        device=scale_rows.device)
    padded[:, :m, :sf_k] = grouped
    physical = padded.view(num_groups, m_tiles, 4, 32, k_tiles, 4).permute(0, 1, 4, 3, 2, 5)
    return physical.contiguous().view(torch.float8_e8m0fnu).permute(3, 4, 1, 5, 2, 0)


def _scale_is_exact_ue8m0(scale: torch.Tensor) -> bool:
    if scale.dtype in (torch.uint8, torch.float8_e8m0fnu):
        return True
    if not scale.is_floating_point():
        return False
    f = scale.detach().to(torch.float32)
    mantissa = f.view(torch.int32) & 0x7FFFFF
    return bool(torch.all((f > 0) & (mantissa == 0)).item())


def _requantize_block_fp8_to_ue8m0(weight: torch.Tensor, scale: torch.Tensor, *, m: int, k: int,
                                   num_groups: int):
    """Re-derive E4M3 codes on ceil-power-of-two 128x128 block scales: reconstruct
    ``w * s`` in FP32, take the block amax, ``e = clamp(ceil(log2(amax/448)))``, re-cast
    ``w / 2^e``. One-time, at weight load (b12x/gemm/_shared/wo_mxfp8.py:1010-1095)."""
    m_tiles, k_tiles = math.ceil(m / 128), k // 128
    if num_groups == 1:
        w_g = weight.reshape(1, m, k)
    elif tuple(weight.shape) == (num_groups * m, k):
        w_g = weight.reshape(num_groups, m, k)
    elif tuple(weight.shape) == (m, k, num_groups):
        w_g = weight.permute(2, 0, 1)
    else:
        raise ValueError(f"weight must have shape {(num_groups * m, k)} or {(m, k, num_groups)}, "
                         f"got {tuple(weight.shape)}")
    s = scale.to(torch.float32)
    if s.numel() != num_groups * m_tiles * k_tiles:
        raise ValueError(f"block scale must have shape {(num_groups * m_tiles, k_tiles)}; "
                         f"got {tuple(scale.shape)}")
    s_g = s.reshape(num_groups, m_tiles, k_tiles)
    s_elem = s_g.repeat_interleave(128, dim=1).repeat_interleave(128, dim=2)[:, :m, :k]
    w_rec = w_g.to(torch.float32) * s_elem
    w_pad = w_rec.new_zeros(num_groups, m_tiles * 128, k_tiles * 128)
    w_pad[:, :m, :k] = w_rec
    blocks = w_pad.view(num_groups, m_tiles, 128, k_tiles, 128)
    amax = blocks.abs().amax(dim=(2, 4), keepdim=True)
    safe = torch.where(amax > 0, amax / FP8_E4M3_MAX, torch.ones_like(amax))
    exponent = torch.clamp(torch.ceil(torch.log2(safe)), -127.0, 127.0)
    new_vals = (blocks / torch.exp2(exponent)).to(torch.float8_e4m3fn)
    new_vals = new_vals.view(num_groups, m_tiles * 128, k_tiles * 128)[:, :m, :k].contiguous()
    new_scale = (exponent.view(num_groups, m_tiles, k_tiles) + 127).to(torch.uint8)
    return new_vals.reshape(m, k) if num_groups == 1 else new_vals.reshape(num_groups * m, k), new_scale


def pack_fp8_block_scaled_weight_mxfp8(weight: torch.Tensor, scale: torch.Tensor, *, m: int,
                                       k: int, num_groups: int = 1) -> MXFP8Rows:
    """Checkpoint E4M3 weight + 128x128 block scale -> MXFP8 rows for the GEMM.

    Arbitrary FP32 block scales (``weight_scale_inv`` style) trigger the re-quantization
    above; scales that are already powers of two are expanded as they are.
    """
    _check_gpu_tensor("weight", weight)
    if weight.dtype != torch.float8_e4m3fn:
        raise ValueError(f"weight must be float8_e4m3fn, got {weight.dtype}")
    if m <= 0 or k <= 0 or num_groups <= 0:
        raise ValueError("m, k, and num_groups must be positive")
    _check_mxfp8_k(k)
    if not _scale_is_exact_ue8m0(scale):
        _check_gpu_tensor("scale", scale)
        weight, scale = _requantize_block_fp8_to_ue8m0(weight, scale, m=m, k=k, num_groups=num_groups)
    if num_groups == 1:
        if tuple(weight.shape) != (m, k):
            raise ValueError(f"weight must have shape {(m, k)}, got {tuple(weight.shape)}")
        values = weight.contiguous()
    elif tuple(weight.shape) == (num_groups * m, k):
        values = weight.contiguous().view(num_groups, m, k).permute(1, 2, 0)
    elif tuple(weight.shape) == (m, k, num_groups):
        values = weight
    else:
        raise ValueError(f"weight must have shape {(num_groups * m, k)} or {(m, k, num_groups)}, "
                         f"got {tuple(weight.shape)}")
    scale_rows = _expand_block_scales_to_mxfp8_rows(scale, m=m, k=k, num_groups=num_groups)
    scale_mma = pack_mxfp8_scales_for_dense_gemm(scale_rows, m=m, k=k, num_groups=num_groups)
    return MXFP8Rows(values=values, scale_rows=scale_rows, scale_mma=scale_mma)


def dequantize_mxfp8_rows_torch(values: torch.Tensor, scale_rows: torch.Tensor) -> torch.Tensor:
    """``[M, K]`` E4M3 + ``[1, M, K/32]`` UE8M0 -> FP32 (debug / test helper)."""
    m, k = values.shape[:2]
    if scale_rows.dtype == torch.uint8:
        scale_rows = scale_rows.view(torch.float8_e8m0fnu)
    s = scale_rows.reshape(m, k // 32).to(torch.float32)
    return (values.to(torch.float32).reshape(m, k // 32, 32) * s[..., None]).reshape(m, k)


__all__ = [
    "MXFP8Rows", "MXFP8_SCALE_VEC_SIZE", "MXFP8_SCALE_ROW_TILE", "MXFP8_SCALE_K_TILE",
    "empty_dense_gemm_mnl_view", "empty_mxfp8_rows_bases", "mxfp8_rows_from_bases",
    "empty_mxfp8_rows_for_dense_gemm", "quantize_mxfp8_rows", "pack_mxfp8_scales_for_dense_gemm",
    "pack_fp8_block_scaled_weight_mxfp8", "dequantize_mxfp8_rows_torch",
]
