"""Host side of the ModelOpt MXFP8 linear (b12x/gemm/mxfp8_linear/_kernel.py:21-266)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..._lib.dense_gemm import dense_gemm
from ..._lib.launch import cuda_stream_to_int
from ..._lib.mxfp8_rows import (
    MXFP8Rows,
    MXFP8_SCALE_VEC_SIZE,
    _check_gpu_tensor,
    pack_mxfp8_scales_for_dense_gemm,
)
from .._shared.block_fp8 import quantize_block_fp8_linear_input_mxfp8


@dataclass(frozen=True)
class MXFP8LinearWeight:
    """ModelOpt-style MXFP8 linear weight packed for the dense GEMM."""

    weight: MXFP8Rows
    in_features: int
    padded_in_features: int
    out_features: int


def _align_up(value: int, alignment: int) -> int:
    return -(-int(value) // int(alignment)) * int(alignment)


def _c_dtype_name(dtype: torch.dtype) -> str:
    if dtype == torch.bfloat16:
        return "bfloat16"
    if dtype == torch.float16:
        return "float16"
    raise ValueError(f"b12x MXFP8 linear output dtype must be bf16/fp16, got {dtype}")


def _zero_pad_columns(t: torch.Tensor, width: int) -> torch.Tensor:
    rows, cols = map(int, t.shape)
    if cols == width:
        return t.contiguous()
    padded = t.new_zeros((rows, width))
    padded[:, :cols] = t
    return padded


def is_mxfp8_linear_supported() -> tuple[bool, str | None]:
    return True, None


def pack_mxfp8_linear_weight(weight: torch.Tensor, weight_scale: torch.Tensor) -> MXFP8LinearWeight:
    """Pack ModelOpt MXFP8 weights ``[N, K]`` and scales ``[N, K/32]``.

    Checkpoints only guarantee ``K % 32 == 0``; the GEMM consumes K in 128-element steps, so
    K is padded with zero codes and UE8M0 1.0 (byte 127) scales.
    """
    _check_gpu_tensor("weight", weight)
    _check_gpu_tensor("weight_scale", weight_scale)
    if weight.ndim != 2:
        raise ValueError(f"weight must have shape [N,K], got {tuple(weight.shape)}")
    if weight.dtype != torch.float8_e4m3fn:
        raise ValueError(f"weight must be float8_e4m3fn, got {weight.dtype}")
    if weight_scale.ndim != 2:
        raise ValueError(f"weight_scale must have shape [N,K/32], got {tuple(weight_scale.shape)}")
    out_features, in_features = map(int, weight.shape)
    if out_features <= 0:
        raise ValueError("out_features must be positive")
    if in_features <= 0 or in_features % MXFP8_SCALE_VEC_SIZE != 0:
        raise ValueError(
            f"ModelOpt MXFP8 weight K must be a positive multiple of {MXFP8_SCALE_VEC_SIZE}, "
            f"got {in_features}")
    scale_k = in_features // MXFP8_SCALE_VEC_SIZE
    if int(weight_scale.shape[0]) < out_features or int(weight_scale.shape[1]) < scale_k:
        raise ValueError(
            f"weight_scale must have at least shape {(out_features, scale_k)}, "
            f"got {tuple(weight_scale.shape)}")
    if weight_scale.dtype == torch.float8_e8m0fnu:
        scale_u8 = weight_scale.view(torch.uint8)
    elif weight_scale.dtype == torch.uint8:
        scale_u8 = weight_scale
    else:
        raise ValueError(f"weight_scale must be uint8/e8m0, got {weight_scale.dtype}")

    padded_in = _align_up(in_features, 128)
    padded_scale_k = padded_in // MXFP8_SCALE_VEC_SIZE
    values = _zero_pad_columns(weight[:out_features, :in_features].view(torch.uint8), padded_in)
    values = values.view(torch.float8_e4m3fn)
    scale_rows = torch.full((out_features, padded_scale_k), 127, dtype=torch.uint8,
                            device=weight.device)
    scale_rows[:, :scale_k] = scale_u8[:out_features, :scale_k]
    scale_rows = scale_rows.view(torch.float8_e8m0fnu)
    scale_mma = pack_mxfp8_scales_for_dense_gemm(scale_rows, m=out_features, k=padded_in,
                                                 num_groups=1)
    return MXFP8LinearWeight(
        weight=MXFP8Rows(values=values, scale_rows=scale_rows.reshape(1, out_features, padded_scale_k),
                         scale_mma=scale_mma),
        in_features=in_features, padded_in_features=padded_in, out_features=out_features)


@torch.library.custom_op("b12x::mxfp8_linear_fused", mutates_args=())
def _mxfp8_linear_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                           weight_scale_rows: torch.Tensor, weight_scale_mma: torch.Tensor,
                           in_features: int, padded_in_features: int, out_features: int,
                           expected_m: int, stream_int: int | None) -> torch.Tensor:
    del weight_scale_rows
    tokens = int(source_2d.shape[0])
    x_q = quantize_block_fp8_linear_input_mxfp8(_zero_pad_columns(source_2d, int(padded_in_features)))
    return dense_gemm(
        (x_q.values.reshape(tokens, padded_in_features, 1), x_q.scale_mma),
        (weight_values.reshape(out_features, padded_in_features, 1), weight_scale_mma),
        ab_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu",
        c_dtype=_c_dtype_name(source_2d.dtype), sf_vec_size=MXFP8_SCALE_VEC_SIZE,
        expected_m=expected_m, stream=stream_int)[:, :, 0]


@_mxfp8_linear_fused_op.register_fake
def _mxfp8_linear_fused_fake(source_2d, weight_values, weight_scale_rows, weight_scale_mma,
                             in_features, padded_in_features, out_features, expected_m,
                             stream_int) -> torch.Tensor:
    return torch.empty((source_2d.shape[0], out_features), dtype=source_2d.dtype,
                       device=source_2d.device)


def mxfp8_linear(source: torch.Tensor, packed_weight: MXFP8LinearWeight, *,
                 bias: torch.Tensor | None = None, expected_m: int | None = None,
                 stream: object = None) -> torch.Tensor:
    """``source[..., K] @ W^T (+ bias)`` through the MXFP8 GEMM."""
    _check_gpu_tensor("source", source)
    if not isinstance(packed_weight, MXFP8LinearWeight):
        raise TypeError("packed_weight must be an MXFP8LinearWeight")
    if source.ndim < 2:
        raise ValueError(f"source must have at least 2 dims, got {tuple(source.shape)}")
    source_2d = source.reshape(-1, source.shape[-1]).contiguous()
    tokens, in_features = map(int, source_2d.shape)
    if in_features != int(packed_weight.in_features):
        raise ValueError(
            f"input K={in_features} does not match packed weight K={packed_weight.in_features}")
    if source_2d.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"source dtype must be bf16/fp16, got {source_2d.dtype}")
    out_features = int(packed_weight.out_features)
    if tokens == 0:
        output = source_2d.new_empty((0, out_features))
    else:
        output = torch.ops.b12x.mxfp8_linear_fused(
            source_2d, packed_weight.weight.values, packed_weight.weight.scale_rows,
            packed_weight.weight.scale_mma, packed_weight.in_features,
            packed_weight.padded_in_features, packed_weight.out_features,
            int(expected_m) if expected_m is not None else tokens, cuda_stream_to_int(stream))
    if bias is not None:
        output = output + bias
    return output.view(*source.shape[:-1], out_features)


__all__ = ["MXFP8LinearWeight", "is_mxfp8_linear_supported", "mxfp8_linear",
           "pack_mxfp8_linear_weight"]
