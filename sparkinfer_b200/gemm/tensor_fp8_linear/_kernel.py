"""Host side of the per-tensor FP8 linear (b12x/gemm/tensor_fp8_linear/_kernel.py:20-319).

The weight keeps its E4M3 codes (K zero-padded to a multiple of 128), a scale tensor in the
GEMM's atom layout filled with UE8M0 1.0 (byte 127), and the caller's combined FP32 scale. The
activation side uses a cached all-ones scale tensor of the right size per device and shape, so
a call launches exactly one kernel: the MXFP8 GEMM with ``alpha = output_scale``.
"""

from __future__ import annotations

import functools
from collections.abc import Iterable
from dataclasses import dataclass

import torch

from ..._lib.dense_gemm import dense_gemm
from ..._lib.launch import cuda_stream_to_int
from ..._lib.mxfp8_rows import (
    MXFP8_SCALE_VEC_SIZE,
    _check_gpu_tensor,
    pack_mxfp8_scales_for_dense_gemm,
)

_OUT_DTYPE_NAMES = {torch.bfloat16: "bfloat16", torch.float16: "float16"}


@dataclass(frozen=True)
class TensorFP8LinearWeight:
    """E4M3 weight ``[N, K_padded]``, unit block scales in MMA layout, one FP32 output scale."""

    values: torch.Tensor
    scale_mma: torch.Tensor
    output_scale: torch.Tensor
    in_features: int
    padded_in_features: int
    out_features: int


def _out_dtype_name(dtype: torch.dtype) -> str:
    try:
        return _OUT_DTYPE_NAMES[dtype]
    except KeyError:
        raise ValueError(f"tensor FP8 linear output must be bf16/fp16, got {dtype}") from None


def _zero_pad_columns(t: torch.Tensor, width: int) -> torch.Tensor:
    rows, cols = map(int, t.shape)
    if cols == width:
        return t.contiguous()
    padded = t.new_zeros((rows, width))
    padded[:, :cols] = t
    return padded


def _unit_scales(rows: int, width: int, device: torch.device) -> torch.Tensor:
    ones = torch.full((rows, width // MXFP8_SCALE_VEC_SIZE), 127, dtype=torch.uint8, device=device)
    return pack_mxfp8_scales_for_dense_gemm(ones, m=rows, k=width, num_groups=1)


@functools.cache
def _unit_scales_cached(device_type: str, device_index: int, rows: int,
                        width: int) -> torch.Tensor:
    return _unit_scales(rows, width, torch.device(device_type, device_index))


def _activation_unit_scales(source: torch.Tensor, rows: int, width: int) -> torch.Tensor:
    index = source.device.index
    if index is None:
        index = torch.cuda.current_device()
    return _unit_scales_cached(source.device.type, int(index), int(rows), int(width))


def is_tensor_fp8_linear_supported() -> tuple[bool, str | None]:
    return True, None


def pack_tensor_fp8_linear_weight(weight: torch.Tensor,
                                  output_scale: torch.Tensor) -> TensorFP8LinearWeight:
    """Pack an E4M3 ``[N, K]`` weight with the one scale that dequantizes the product."""
    _check_gpu_tensor("weight", weight)
    _check_gpu_tensor("output_scale", output_scale)
    if weight.ndim != 2:
        raise ValueError(f"weight must have shape [N,K], got {tuple(weight.shape)}")
    if weight.dtype != torch.float8_e4m3fn:
        raise ValueError(f"weight must be float8_e4m3fn, got {weight.dtype}")
    if output_scale.dtype != torch.float32 or output_scale.numel() != 1:
        raise ValueError(
            "output_scale must be one float32 value, got "
            f"dtype={output_scale.dtype}, shape={tuple(output_scale.shape)}")
    if output_scale.device != weight.device:
        raise ValueError("weight and output_scale must be on the same device")
    if not bool(torch.isfinite(output_scale).all()) or bool((output_scale < 0).any()):
        raise ValueError("output_scale must be finite and non-negative")
    out_features, in_features = map(int, weight.shape)
    if out_features <= 0:
        raise ValueError("out_features must be positive")
    if in_features <= 0 or in_features % MXFP8_SCALE_VEC_SIZE != 0:
        raise ValueError(
            f"tensor FP8 weight K must be a positive multiple of {MXFP8_SCALE_VEC_SIZE}, "
            f"got {in_features}")
    padded_in = -(-in_features // 128) * 128
    values = _zero_pad_columns(weight.view(torch.uint8), padded_in).view(torch.float8_e4m3fn)
    return TensorFP8LinearWeight(
        values=values, scale_mma=_unit_scales(out_features, padded_in, weight.device),
        output_scale=output_scale.reshape(1).contiguous(), in_features=in_features,
        padded_in_features=padded_in, out_features=out_features)


@torch.library.custom_op("b12x::tensor_fp8_linear_fused", mutates_args=())
def _tensor_fp8_linear_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                                weight_scale_mma: torch.Tensor, output_scale: torch.Tensor,
                                padded_in_features: int, out_features: int, expected_m: int,
                                out_dtype: torch.dtype, stream_int: int | None) -> torch.Tensor:
    tokens = int(source_2d.shape[0])
    padded_in = int(padded_in_features)
    x = _zero_pad_columns(source_2d.view(torch.uint8), padded_in).view(torch.float8_e4m3fn)
    return dense_gemm(
        (x.reshape(tokens, padded_in, 1), _activation_unit_scales(x, tokens, padded_in)),
        (weight_values.reshape(out_features, padded_in, 1), weight_scale_mma),
        alpha=output_scale, ab_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu",
        c_dtype=_out_dtype_name(out_dtype), sf_vec_size=MXFP8_SCALE_VEC_SIZE,
        expected_m=expected_m, stream=stream_int, plain_fp8=True)[:, :, 0]


@_tensor_fp8_linear_fused_op.register_fake
def _tensor_fp8_linear_fused_fake(source_2d, weight_values, weight_scale_mma, output_scale,
                                  padded_in_features, out_features, expected_m, out_dtype,
                                  stream_int) -> torch.Tensor:
    return torch.empty((source_2d.shape[0], out_features), dtype=out_dtype,
                       device=source_2d.device)


def tensor_fp8_linear(source: torch.Tensor, packed_weight: TensorFP8LinearWeight, *,
                      bias: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
                      expected_m: int | None = None, stream: object = None) -> torch.Tensor:
    """``output_scale * (source[..., K] @ W^T) (+ bias)`` for E4M3 ``source``."""
    _check_gpu_tensor("source", source)
    if not isinstance(packed_weight, TensorFP8LinearWeight):
        raise TypeError("packed_weight must be a TensorFP8LinearWeight")
    if source.ndim < 2:
        raise ValueError(f"source must have at least 2 dims, got {tuple(source.shape)}")
    source_2d = source.reshape(-1, source.shape[-1]).contiguous()
    tokens, in_features = map(int, source_2d.shape)
    if source_2d.dtype != torch.float8_e4m3fn:
        raise ValueError(f"source must be float8_e4m3fn, got {source_2d.dtype}")
    if in_features != int(packed_weight.in_features):
        raise ValueError(
            f"input K={in_features} does not match packed weight K={packed_weight.in_features}")
    if packed_weight.values.device != source_2d.device:
        raise ValueError("source and packed weight must be on the same device")
    if expected_m is not None and int(expected_m) <= 0:
        raise ValueError("expected_m must be positive when provided")
    _out_dtype_name(out_dtype)
    out_features = int(packed_weight.out_features)
    if bias is not None:
        _check_gpu_tensor("bias", bias)
        if bias.device != source_2d.device:
            raise ValueError("bias must be on the same device as source")
        if bias.dtype != out_dtype or bias.shape != (out_features,):
            raise ValueError(
                f"bias must have shape {(out_features,)} and dtype {out_dtype}, "
                f"got shape={tuple(bias.shape)}, dtype={bias.dtype}")
    if tokens == 0:
        output = torch.empty((0, out_features), dtype=out_dtype, device=source_2d.device)
    else:
        output = torch.ops.b12x.tensor_fp8_linear_fused(
            source_2d, packed_weight.values, packed_weight.scale_mma,
            packed_weight.output_scale, packed_weight.padded_in_features,
            packed_weight.out_features, int(expected_m) if expected_m is not None else tokens,
            out_dtype, cuda_stream_to_int(stream))
    if bias is not None:
        output = output + bias
    return output.view(*source.shape[:-1], out_features)


def prewarm_tensor_fp8_linear(packed_weight: TensorFP8LinearWeight, token_counts: Iterable[int],
                              *, out_dtype: torch.dtype = torch.bfloat16,
                              stream: object = None) -> int:
    """Run each token count once (library load, kernel attributes, the cached unit-scale
    tensors and decode scratch) so that a later CUDA-graph capture allocates nothing."""
    warmed = 0
    with torch.inference_mode():
        for tokens in sorted({int(t) for t in token_counts if int(t) > 0}):
            source = torch.zeros((tokens, packed_weight.in_features), dtype=torch.float8_e4m3fn,
                                 device=packed_weight.values.device)
            tensor_fp8_linear(source, packed_weight, out_dtype=out_dtype, expected_m=tokens,
                              stream=stream)
            warmed += 1
    return warmed


__all__ = ["TensorFP8LinearWeight", "is_tensor_fp8_linear_supported",
           "pack_tensor_fp8_linear_weight", "prewarm_tensor_fp8_linear", "tensor_fp8_linear"]
