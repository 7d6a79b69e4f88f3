"""MXFP8 row operands: what they look like in memory, the row quantizer entry point, and the
load-time conversion of checkpoint weights into them.

Interface of b12x/gemm/_shared/wo_mxfp8.py (``MXFP8Rows`` :51-69, storage helpers :717-830,
scale expansion and packing :844-987, block-FP8 weight re-quantization :990-1187) and of
``quantize_mxfp8_rows_cute`` (b12x/_lib/quant/mxfp8_rows.py:398-434). Quantizing activation rows
is a CUDA kernel; weight conversion runs once per checkpoint in torch. Its bytes are pinned
against the reference's own packers by golden files, so the arithmetic here is exact integer
work on the FP32 bit patterns rather than ``log2`` round trips.

Memory picture of one operand ``[M, K]`` (``L`` groups stack along a leading axis):

* ``values``      E4M3 codes, K-major.
* ``scale_rows``  one UE8M0 byte per row and 32 columns, ``[L, M, K / 32]``.
* ``scale_mma``   the same bytes in 512-byte atoms ``[L, ceil(M/128), ceil(K/128), 32, 4, 4]``
  (row ``r`` of a 128-row tile at ``[r % 32, r // 32]``, scale column ``c`` at ``[.., c % 4]`` of
  atom ``c // 4``), handed to the GEMM as the permuted 6-D view ``(32, 4, tiles_m, 4, tiles_k, L)``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import launch
from .launch import cuda_stream_to_int

FP8_E4M3_MAX = 448.0
SCALE_BLOCK = 32           # elements of K that share one UE8M0 scale
ATOM_ROWS = 128            # rows covered by one scale atom
ATOM_COLS = 4              # scale columns covered by one scale atom
UNIT_SCALE = 127           # UE8M0 1.0
# Names the reference exports for the same constants.
MXFP8_SCALE_VEC_SIZE = SCALE_BLOCK
MXFP8_SCALE_ROW_TILE = ATOM_ROWS
MXFP8_SCALE_K_TILE = ATOM_COLS

_ATOM_VIEW = (3, 4, 1, 5, 2, 0)   # physical [L, mt, kt, 32, 4, 4] -> (32, 4, mt, 4, kt, L)


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


def _ceil_div(a: int, b: int) -> int:
    return -(-int(a) // int(b))


def _check_gpu_tensor(name: str, tensor: torch.Tensor) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be on CUDA")


def _check_mxfp8_k(k: int) -> None:
    if k <= 0 or k % 128 != 0:
        raise ValueError(f"MXFP8 dense_gemm K must be a positive multiple of 128, got {k}")


def _atom_grid(m: int, k: int) -> tuple[int, int]:
    return _ceil_div(m, ATOM_ROWS), _ceil_div(k // SCALE_BLOCK, ATOM_COLS)


# ----------------------------------------------------------------------------------------
# Storage
# ----------------------------------------------------------------------------------------
def empty_dense_gemm_mnl_view(m: int, n: int, l: int, *, device, dtype: torch.dtype) -> torch.Tensor:
    """``[M, N, L]`` view backed by physical ``[L, M, N]`` storage."""
    if min(m, n, l) <= 0:
        raise ValueError("m, n, and l must be positive")
    physical = torch.empty((l, m, n), device=device, dtype=dtype)
    return physical.permute(1, 2, 0) if l > 1 else physical.view(m, n, 1)


def empty_mxfp8_rows_bases(m: int, k: int, *, num_groups: int, device,
                           initialize_scales: bool = True):
    """The three contiguous buffers behind an :class:`MXFP8Rows`:
    ``(values [M,K] e4m3, scale_rows [L,M,K/32] u8, scale atoms [L,mt,kt,32,4,4] u8)``.
    Scales start at 127 (UE8M0 1.0) unless ``initialize_scales`` is false."""
    if min(m, k, num_groups) <= 0:
        raise ValueError("m, k, and num_groups must be positive")
    _check_mxfp8_k(k)
    row_tiles, k_tiles = _atom_grid(m, k)

    def scale_bytes(*shape):
        if initialize_scales:
            return torch.full(shape, UNIT_SCALE, dtype=torch.uint8, device=device)
        return torch.empty(shape, dtype=torch.uint8, device=device)

    values = torch.empty((m, k) if num_groups == 1 else (num_groups, m, k), device=device,
                         dtype=torch.float8_e4m3fn)
    return (values, scale_bytes(num_groups, m, k // SCALE_BLOCK),
            scale_bytes(num_groups, row_tiles, k_tiles, 32, 4, 4))


def mxfp8_rows_from_bases(values_base, scale_rows_base, scale_physical_base, m: int, k: int, *,
                          num_groups: int) -> MXFP8Rows:
    """Rebuild the dense-GEMM views over the contiguous bases (views only)."""
    values = values_base if num_groups == 1 else values_base.permute(1, 2, 0)
    return MXFP8Rows(values=values, scale_rows=scale_rows_base.view(torch.float8_e8m0fnu),
                     scale_mma=scale_physical_base.view(torch.float8_e8m0fnu).permute(*_ATOM_VIEW))


def empty_mxfp8_rows_for_dense_gemm(m: int, k: int, *, num_groups: int = 1, device) -> MXFP8Rows:
    bases = empty_mxfp8_rows_bases(m, k, num_groups=num_groups, device=device)
    return mxfp8_rows_from_bases(*bases, m, k, num_groups=num_groups)


def _check_mxfp8_rows_storage(out: MXFP8Rows, *, m: int, k: int, num_groups: int) -> None:
    """Shape, dtype, device and contiguity of caller-provided operand storage."""
    row_tiles, k_tiles = _atom_grid(m, k)
    expected = {
        "values": (torch.float8_e4m3fn, (m, k) if num_groups == 1 else (m, k, num_groups)),
        "scale_rows": (torch.float8_e8m0fnu, (num_groups, m, k // SCALE_BLOCK)),
        "scale_mma": (torch.float8_e8m0fnu, (32, 4, row_tiles, 4, k_tiles, num_groups)),
    }
    for field, (dtype, shape) in expected.items():
        tensor = getattr(out, field)
        _check_gpu_tensor(f"out.{field}", tensor)
        if tensor.dtype != dtype:
            raise ValueError(f"out.{field} must be {str(dtype).split('.')[-1]}, got {tensor.dtype}")
        if tuple(tensor.shape) != shape:
            raise ValueError(f"out.{field} must have shape {shape}, got {tuple(tensor.shape)}")
    if num_groups == 1 and not out.values.is_contiguous():
        raise ValueError("out.values must be contiguous")
    if not out.scale_rows.is_contiguous():
        raise ValueError("out.scale_rows must be contiguous")


# ----------------------------------------------------------------------------------------
# Row quantizer (CUDA)
# ----------------------------------------------------------------------------------------
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
    m, k = (int(v) for v in source.shape)
    if k % SCALE_BLOCK:
        raise ValueError(f"K must be a multiple of {SCALE_BLOCK}, got {k}")
    if values.numel() != m * k or values.element_size() != 1 or not values.is_contiguous():
        raise ValueError(f"values must be a contiguous one-byte tensor of {m * k} elements")
    scale_count = m * (k // SCALE_BLOCK)
    if scale_rows is not None and (scale_rows.numel() != scale_count or not scale_rows.is_contiguous()):
        raise ValueError(f"scale_rows must be contiguous with {scale_count} elements")
    atom_bytes = _ceil_div(m, ATOM_ROWS) * _ceil_div(k, 128) * 512
    if scale_mma is not None and scale_mma.numel() < atom_bytes:
        raise ValueError(f"scale_mma must hold at least {atom_bytes} bytes, got {scale_mma.numel()}")
    if m:
        launch.quantize_mxfp8_rows(source, values, scale_rows, scale_mma,
                                   stream_int=cuda_stream_to_int(stream))


# ----------------------------------------------------------------------------------------
# Load-time weight conversion (torch)
# ----------------------------------------------------------------------------------------
def _ceil_log2_exponent(value: torch.Tensor) -> torch.Tensor:
    """``ceil(log2(v))`` of positive FP32 values, read off the bit pattern: the biased exponent
    minus 127, plus one when any mantissa bit is set (subnormals: everything above 2^-127 is
    -126, the rest -127). Int32."""
    bits = value.to(torch.float32).contiguous().view(torch.int32)
    exponent = (bits >> 23) & 0xFF
    mantissa = bits & 0x7FFFFF
    normal = exponent - 127 + (mantissa != 0).to(torch.int32)
    subnormal = torch.where(mantissa > 0x400000, -126, -127).to(torch.int32)
    return torch.where(exponent == 0, subnormal, normal)


def _scale_u8_from_max_abs(max_abs: torch.Tensor) -> torch.Tensor:
    """UE8M0 byte = 127 + clamp(ceil(log2(amax/448)), -127, 127); 127 for zero blocks."""
    amax = max_abs.to(torch.float32)
    exponent = _ceil_log2_exponent(amax / FP8_E4M3_MAX).clamp(-127, 127)
    return torch.where(amax > 0, exponent + 127, torch.full_like(exponent, UNIT_SCALE)).to(torch.uint8)


def _scale_to_e8m0_u8(scale: torch.Tensor) -> torch.Tensor:
    """Any scale representation -> UE8M0 bytes (float scales are rounded to the nearest power
    of two, non-positive ones count as 1.0)."""
    if scale.dtype == torch.float8_e8m0fnu:
        return scale.view(torch.uint8)
    if scale.dtype == torch.uint8:
        return scale
    if not scale.is_floating_point():
        raise ValueError(f"scale must be e8m0, uint8, or floating-point, got {scale.dtype}")
    positive = torch.where(scale > 0, scale.to(torch.float32), torch.ones((), dtype=torch.float32,
                                                                          device=scale.device))
    return (torch.round(torch.log2(positive)).clamp(-127, 127) + 127).to(torch.uint8)


def _expand_block_scales_to_mxfp8_rows(scale: torch.Tensor, *, m: int, k: int,
                                       num_groups: int) -> torch.Tensor:
    """128x128 block scales -> per-row, per-32-column UE8M0 ``[L, M, K/32]``."""
    _check_mxfp8_k(k)
    row_tiles, k_blocks = _ceil_div(m, 128), k // 128
    if scale.numel() != num_groups * row_tiles * k_blocks:
        raise ValueError(
            f"block scale must have {num_groups * row_tiles * k_blocks} entries "
            f"([{num_groups}*{row_tiles}, {k_blocks}]); got {tuple(scale.shape)}")
    per_block = _scale_to_e8m0_u8(scale).reshape(num_groups, row_tiles, k_blocks)
    per_row = per_block.repeat_interleave(128, dim=1).repeat_interleave(128 // SCALE_BLOCK, dim=2)
    return per_row[:, :m].contiguous().view(torch.float8_e8m0fnu)


def pack_mxfp8_scales_for_dense_gemm(scale_rows: torch.Tensor, *, m: int, k: int,
                                     num_groups: int = 1) -> torch.Tensor:
    """Row-major UE8M0 scales -> 6-D MMA view; padding rows/columns are 127 (UE8M0 1.0)."""
    if scale_rows.dtype not in (torch.uint8, torch.float8_e8m0fnu):
        raise ValueError(f"scale_rows must be uint8/e8m0, got {scale_rows.dtype}")
    _check_mxfp8_k(k)
    cols = k // SCALE_BLOCK
    if scale_rows.numel() != num_groups * m * cols:
        raise ValueError(
            f"scale_rows must have shape {(num_groups, m, cols)}, got {tuple(scale_rows.shape)}")
    row_tiles, k_tiles = _atom_grid(m, k)
    padded = torch.full((num_groups, row_tiles * ATOM_ROWS, k_tiles * ATOM_COLS), UNIT_SCALE,
                        dtype=torch.uint8, device=scale_rows.device)
    padded[:, :m, :cols] = scale_rows.reshape(num_groups, m, cols).view(torch.uint8)
    # [L, mt, (r // 32), (r % 32), kt, (c % 4)] -> atoms [L, mt, kt, r % 32, r // 32, c % 4]
    atoms = padded.view(num_groups, row_tiles, 4, 32, k_tiles, ATOM_COLS).permute(0, 1, 4, 3, 2, 5)
    return atoms.contiguous().view(torch.float8_e8m0fnu).permute(*_ATOM_VIEW)


def _scale_is_exact_ue8m0(scale: torch.Tensor) -> bool:
    """True when the block scales are already powers of two (nothing to re-derive)."""
    if scale.dtype in (torch.uint8, torch.float8_e8m0fnu):
        return True
    if not scale.is_floating_point():
        return False
    as_f32 = scale.detach().to(torch.float32).contiguous()
    return bool(((as_f32 > 0) & ((as_f32.view(torch.int32) & 0x7FFFFF) == 0)).all())


def _groups_first(weight: torch.Tensor, *, m: int, k: int, num_groups: int) -> torch.Tensor:
    """The accepted weight layouts as ``[L, M, K]``."""
    if num_groups == 1 and weight.numel() == m * k:
        return weight.reshape(1, m, k)
    if tuple(weight.shape) == (num_groups * m, k):
        return weight.reshape(num_groups, m, k)
    if tuple(weight.shape) == (m, k, num_groups):
        return weight.permute(2, 0, 1)
    raise ValueError(f"weight must have shape {(num_groups * m, k)} or {(m, k, num_groups)}, "
                     f"got {tuple(weight.shape)}")


def _requantize_block_fp8_to_ue8m0(weight: torch.Tensor, scale: torch.Tensor, *, m: int, k: int,
                                   num_groups: int):
    """Re-derive E4M3 codes on ceil-power-of-two 128x128 block scales: reconstruct ``w * s`` in
    FP32, take each block's amax, ``e = clamp(ceil(log2(amax/448)))`` (0 for an all-zero block),
    cast ``w / 2^e`` back to E4M3. One-time, at weight load
    (b12x/gemm/_shared/wo_mxfp8.py:1010-1095)."""
    row_tiles, k_blocks = _ceil_div(m, 128), k // 128
    if scale.numel() != num_groups * row_tiles * k_blocks:
        raise ValueError(f"block scale must have shape {(num_groups * row_tiles, k_blocks)}; "
                         f"got {tuple(scale.shape)}")
    codes = _groups_first(weight, m=m, k=k, num_groups=num_groups).to(torch.float32)
    block_scale = scale.to(torch.float32).reshape(num_groups, row_tiles, 1, k_blocks, 1)
    padded = codes.new_zeros((num_groups, row_tiles * 128, k))
    padded[:, :m] = codes
    blocks = padded.view(num_groups, row_tiles, 128, k_blocks, 128) * block_scale
    byte = _scale_u8_from_max_abs(blocks.abs().amax(dim=(2, 4)))
    divisor = torch.exp2(byte.to(torch.float32) - 127.0)[:, :, None, :, None]
    recoded = (blocks / divisor).to(torch.float8_e4m3fn).view(num_groups, row_tiles * 128, k)[:, :m]
    recoded = recoded.contiguous()
    return (recoded.view(m, k) if num_groups == 1 else recoded.view(num_groups * m, k)), byte


def pack_fp8_block_scaled_weight_mxfp8(weight: torch.Tensor, scale: torch.Tensor, *, m: int,
                                       k: int, num_groups: int = 1) -> MXFP8Rows:
    """Checkpoint E4M3 weight + 128x128 block scale -> MXFP8 rows for the GEMM.

    Arbitrary FP32 block scales (``weight_scale_inv`` style) trigger the re-quantization
    above; scales that are already powers of two are expanded as they are.
    """
    _check_gpu_tensor("weight", weight)
    if weight.dtype != torch.float8_e4m3fn:
        raise ValueError(f"weight must be float8_e4m3fn, got {weight.dtype}")
    if min(m, k, num_groups) <= 0:
        raise ValueError("m, k, and num_groups must be positive")
    _check_mxfp8_k(k)
    if weight.is_cuda:
        return _pack_block_fp8_weight_on_device(weight, scale, m=m, k=k, num_groups=num_groups)
    # Host tensors (only reachable with the device check lifted, as the CPU tests do): the same
    # arithmetic in torch ops, which is what pins the kernel's bytes.
    if not _scale_is_exact_ue8m0(scale):
        _check_gpu_tensor("scale", scale)
        weight, scale = _requantize_block_fp8_to_ue8m0(weight, scale, m=m, k=k, num_groups=num_groups)
    if num_groups == 1:
        if tuple(weight.shape) != (m, k):
            raise ValueError(f"weight must have shape {(m, k)}, got {tuple(weight.shape)}")
        values = weight.contiguous()
    elif tuple(weight.shape) == (m, k, num_groups):
        values = weight
    else:
        values = _groups_first(weight.contiguous(), m=m, k=k, num_groups=num_groups).permute(1, 2, 0)
    scale_rows = _expand_block_scales_to_mxfp8_rows(scale, m=m, k=k, num_groups=num_groups)
    return MXFP8Rows(values=values, scale_rows=scale_rows,
                     scale_mma=pack_mxfp8_scales_for_dense_gemm(scale_rows, m=m, k=k,
                                                                num_groups=num_groups))


def _pack_block_fp8_weight_on_device(weight: torch.Tensor, scale: torch.Tensor, *, m: int, k: int,
                                     num_groups: int) -> MXFP8Rows:
    """The conversion above as one kernel launch (``b12x_b200_pack_block_fp8_weight_mxfp8``)."""
    from . import launch

    row_tiles, k_blocks = _ceil_div(m, 128), k // 128
    if scale.numel() != num_groups * row_tiles * k_blocks:
        raise ValueError(f"block scale must have shape {(num_groups * row_tiles, k_blocks)}; "
                         f"got {tuple(scale.shape)}")
    requantize = not _scale_is_exact_ue8m0(scale)
    if requantize:
        _check_gpu_tensor("scale", scale)
    if scale.dtype in (torch.uint8, torch.float8_e8m0fnu):
        block_scale = torch.exp2(scale.view(torch.uint8).to(torch.float32) - 127.0)
    elif scale.is_floating_point():
        block_scale = scale.to(torch.float32)
    else:
        raise ValueError(f"scale must be e8m0, uint8, or floating-point, got {scale.dtype}")
    block_scale = block_scale.to(weight.device).reshape(num_groups, row_tiles, k_blocks).contiguous()
    codes = _groups_first(weight, m=m, k=k, num_groups=num_groups).contiguous()
    out = empty_mxfp8_rows_for_dense_gemm(m, k, num_groups=num_groups, device=weight.device)
    # The packed values come back in the layout the torch path produces: [M, K] for one group,
    # the [M, K, L] view over [L, M, K] storage otherwise.
    values_storage = out.values if num_groups == 1 else out.values.permute(2, 0, 1)
    launch.pack_block_fp8_weight_mxfp8(codes.view(torch.uint8), block_scale, values_storage,
                                       out.scale_rows, out.scale_mma, m, k, num_groups, requantize)
    return out


def dequantize_mxfp8_rows_torch(values: torch.Tensor, scale_rows: torch.Tensor) -> torch.Tensor:
    """``[M, K]`` E4M3 + ``[1, M, K/32]`` UE8M0 -> FP32 (debug / test helper)."""
    m, k = values.shape[:2]
    scales = scale_rows.view(torch.float8_e8m0fnu) if scale_rows.dtype == torch.uint8 else scale_rows
    per_block = scales.reshape(m, k // SCALE_BLOCK, 1).to(torch.float32)
    return (values.to(torch.float32).reshape(m, k // SCALE_BLOCK, SCALE_BLOCK) * per_block).reshape(m, k)


__all__ = [
    "MXFP8Rows", "MXFP8_SCALE_VEC_SIZE", "MXFP8_SCALE_ROW_TILE", "MXFP8_SCALE_K_TILE", "SCALE_BLOCK",
    "empty_dense_gemm_mnl_view", "empty_mxfp8_rows_bases", "mxfp8_rows_from_bases",
    "empty_mxfp8_rows_for_dense_gemm", "quantize_mxfp8_rows", "pack_mxfp8_scales_for_dense_gemm",
    "pack_fp8_block_scaled_weight_mxfp8", "dequantize_mxfp8_rows_torch",
]
