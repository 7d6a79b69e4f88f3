"""Host side of the ModelOpt MXFP8 linear (b12x/gemm/mxfp8_linear/_kernel.py:21-266): weight
packing, the ``b12x::mxfp8_linear_fused`` custom op and ``mxfp8_linear``. The forward step
(pad K, quantize rows, GEMM, bias) is the shared core of :mod:`sparkinfer_b200._lib.linear_core`.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..._lib.launch import cuda_stream_to_int
from ..._lib.linear_core import (
    K_STEP,
    SourceRows,
    bias_fuses,
    output_dtype_name,
    pad_columns,
    quantize_then_gemm,
    require_cuda_tensor,
    round_up,
)
from ..._lib.mxfp8_rows import (
    MXFP8Rows,
    SCALE_BLOCK,
    UNIT_SCALE,
    empty_mxfp8_rows_bases,
    mxfp8_rows_from_bases,
    pack_mxfp8_scales_for_dense_gemm,
)

_OWNER = "b12x MXFP8 linear"


@dataclass(frozen=True)
class MXFP8LinearWeight:
    """ModelOpt-style MXFP8 linear weight packed for the dense GEMM."""

    weight: MXFP8Rows
    in_features: int
    padded_in_features: int
    out_features: int


def is_mxfp8_linear_supported() -> tuple[bool, str | None]:
    return True, None


def pack_mxfp8_linear_weight(weight: torch.Tensor, weight_scale: torch.Tensor) -> MXFP8LinearWeight:
    """Pack ModelOpt MXFP8 weights ``[N, K]`` and scales ``[N, K/32]``.

    Checkpoints only guarantee ``K % 32 == 0``; the GEMM consumes K in 128-element steps, so
    K is padded with zero codes and UE8M0 1.0 (byte 127) scales.
    """
    require_cuda_tensor("weight", weight)
    require_cuda_tensor("weight_scale", weight_scale)
    if weight.ndim != 2:
        raise ValueError(f"weight must have shape [N,K], got {tuple(weight.shape)}")
    if weight.dtype != torch.float8_e4m3fn:
        raise ValueError(f"weight must be float8_e4m3fn, got {weight.dtype}")
    if weight_scale.ndim != 2:
        raise ValueError(f"weight_scale must have shape [N,K/32], got {tuple(weight_scale.shape)}")
    if weight_scale.dtype not in (torch.uint8, torch.float8_e8m0fnu):
        raise ValueError(f"weight_scale must be uint8/e8m0, got {weight_scale.dtype}")
    out_features, in_features = (int(v) for v in weight.shape)
    if out_features <= 0:
        raise ValueError("out_features must be positive")
    if in_features <= 0 or in_features % SCALE_BLOCK:
        raise ValueError(
            f"ModelOpt MXFP8 weight K must be a positive multiple of {SCALE_BLOCK}, got {in_features}")
    blocks = in_features // SCALE_BLOCK
    if weight_scale.shape[0] < out_features or weight_scale.shape[1] < blocks:
        raise ValueError(f"weight_scale must have at least shape {(out_features, blocks)}, "
                         f"got {tuple(weight_scale.shape)}")

    padded_in = round_up(in_features, K_STEP)
    codes = pad_columns(weight.view(torch.uint8), padded_in).view(torch.float8_e4m3fn)
    scale_bytes = weight_scale.view(torch.uint8)[:out_features, :blocks]
    scale_rows = torch.nn.functional.pad(scale_bytes, (0, padded_in // SCALE_BLOCK - blocks),
                                         value=UNIT_SCALE).contiguous().view(torch.float8_e8m0fnu)
    return MXFP8LinearWeight(
        weight=MXFP8Rows(values=codes, scale_rows=scale_rows.unsqueeze(0),
                         scale_mma=pack_mxfp8_scales_for_dense_gemm(
                             scale_rows, m=out_features, k=padded_in, num_groups=1)),
        in_features=in_features, padded_in_features=padded_in, out_features=out_features)


def _forward(source_2d: torch.Tensor, weight_values: torch.Tensor, weight_scale_mma: torch.Tensor,
             *, padded_in: int, out_features: int, bias: torch.Tensor | None,
             stream_int: int | None) -> torch.Tensor:
    tokens = int(source_2d.shape[0])
    output_dtype_name(source_2d.dtype, _OWNER)
    x_q = mxfp8_rows_from_bases(
        *empty_mxfp8_rows_bases(tokens, padded_in, num_groups=1, device=source_2d.device),
        tokens, padded_in, num_groups=1)
    out = torch.empty((tokens, out_features, 1), dtype=source_2d.dtype, device=source_2d.device)
    return quantize_then_gemm(pad_columns(source_2d, padded_in), weight_values, weight_scale_mma,
                              padded_k=padded_in, out_features=out_features, x_q=x_q, out=out,
                              bias=bias, stream=stream_int)


@torch.library.custom_op("b12x::mxfp8_linear_fused", mutates_args=())
def _mxfp8_linear_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                           weight_scale_rows: torch.Tensor, weight_scale_mma: torch.Tensor,
                           in_features: int, padded_in_features: int, out_features: int,
                           expected_m: int, stream_int: int | None) -> torch.Tensor:
    del weight_scale_rows, in_features, expected_m
    return _forward(source_2d, weight_values, weight_scale_mma, padded_in=int(padded_in_features),
                    out_features=int(out_features), bias=None, stream_int=stream_int)


@_mxfp8_linear_fused_op.register_fake
def _mxfp8_linear_fused_fake(source_2d, weight_values, weight_scale_rows, weight_scale_mma,
                             in_features, padded_in_features, out_features, expected_m,
                             stream_int) -> torch.Tensor:
    return source_2d.new_empty((source_2d.shape[0], out_features))


@torch.library.custom_op("b12x::mxfp8_linear_bias_fused", mutates_args=())
def _mxfp8_linear_bias_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                                weight_scale_mma: torch.Tensor, bias: torch.Tensor,
                                padded_in_features: int, out_features: int,
                                stream_int: int | None) -> torch.Tensor:
    """The linear with its bias added in the GEMM epilogue (the reference has no such op: its
    bias is a separate add after ``b12x::mxfp8_linear_fused``)."""
    return _forward(source_2d, weight_values, weight_scale_mma, padded_in=int(padded_in_features),
                    out_features=int(out_features), bias=bias, stream_int=stream_int)


@_mxfp8_linear_bias_fused_op.register_fake
def _mxfp8_linear_bias_fused_fake(source_2d, weight_values, weight_scale_mma, bias,
                                  padded_in_features, out_features, stream_int) -> torch.Tensor:
    return source_2d.new_empty((source_2d.shape[0], out_features))


def mxfp8_linear(source: torch.Tensor, packed_weight: MXFP8LinearWeight, *,
                 bias: torch.Tensor | None = None, expected_m: int | None = None,
                 stream: object = None) -> torch.Tensor:
    """``source[..., K] @ W^T (+ bias)`` through the MXFP8 GEMM."""
    require_cuda_tensor("source", source)
    if not isinstance(packed_weight, MXFP8LinearWeight):
        raise TypeError("packed_weight must be an MXFP8LinearWeight")
    rows = SourceRows.of(source, packed_in_features=packed_weight.in_features,
                         dtypes=(torch.bfloat16, torch.float16),
                         dtype_error="source dtype must be bf16/fp16, got {dtype}")
    n = int(packed_weight.out_features)
    weight = packed_weight.weight
    if rows.tokens == 0:
        output = rows.rows.new_empty((0, n))
        return rows.restore(output + bias if bias is not None else output, n)
    if bias_fuses(bias, rows.rows.dtype, n):
        output = torch.ops.b12x.mxfp8_linear_bias_fused(
            rows.rows, weight.values, weight.scale_mma, bias, packed_weight.padded_in_features, n,
            cuda_stream_to_int(stream))
        return rows.restore(output, n)
    output = torch.ops.b12x.mxfp8_linear_fused(
        rows.rows, weight.values, weight.scale_rows, weight.scale_mma, packed_weight.in_features,
        packed_weight.padded_in_features, n,
        int(expected_m) if expected_m is not None else rows.tokens, cuda_stream_to_int(stream))
    if bias is not None:
        output = output + bias
    return rows.restore(output, n)


__all__ = ["MXFP8LinearWeight", "is_mxfp8_linear_supported", "mxfp8_linear",
           "pack_mxfp8_linear_weight"]
