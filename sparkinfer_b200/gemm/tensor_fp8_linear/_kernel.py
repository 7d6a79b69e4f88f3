"""Host side of the per-tensor FP8 linear (b12x/gemm/tensor_fp8_linear/_kernel.py:20-319):
``output_scale * (x_e4m3 @ W_e4m3^T) (+ bias)``.

Both operands arrive already in E4M3, so there is nothing to quantize: a call is one GEMM with
``alpha = output_scale``. Shapes of the tiled kernels run the unscaled E4M3 MMA (no scale bytes
move); decode shapes run the weight-streaming MXFP8 kernel fed with block scales of exactly 1.0
(UE8M0 byte 127) on both sides, taken from a per-device, per-shape cache. As in the reference
(``plain_fp8``), the scale storage a packed weight carries is never read.
"""

from __future__ import annotations

from collections.abc import Iterable
from dataclasses import dataclass

import torch

from ..._lib import launch
from ..._lib.launch import cuda_stream_to_int
from ..._lib.linear_core import (
    K_STEP,
    LINEAR_DTYPES,
    SourceRows,
    bias_fuses,
    pad_columns,
    require_cuda_tensor,
    round_up,
)
from ..._lib.mxfp8_rows import SCALE_BLOCK, UNIT_SCALE
from ... import _native

_UNIT_ATOMS: dict[tuple[int, int, int], torch.Tensor] = {}


@dataclass(frozen=True)
class TensorFP8LinearWeight:
    """E4M3 weight ``[N, K_padded]``, unit block scales in MMA layout, one FP32 output scale."""

    values: torch.Tensor
    scale_mma: torch.Tensor
    output_scale: torch.Tensor
    in_features: int
    padded_in_features: int
    out_features: int


def _unit_scale_atoms(rows: int, width: int, device: torch.device) -> torch.Tensor:
    """Scale atoms for ``[rows, width]`` with every byte 127, as the 6-D view the GEMM takes
    (a constant fill: the atom layout does not matter when all bytes are equal)."""
    row_tiles, k_tiles = -(-rows // 128), -(-(width // SCALE_BLOCK) // 4)
    atoms = torch.full((1, row_tiles, k_tiles, 32, 4, 4), UNIT_SCALE, dtype=torch.uint8, device=device)
    return atoms.view(torch.float8_e8m0fnu).permute(3, 4, 1, 5, 2, 0)


def _cached_unit_atoms(rows: int, width: int, device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (int(index), -(-rows // 128), width)
    atoms = _UNIT_ATOMS.get(key)
    if atoms is None:
        atoms = _UNIT_ATOMS[key] = _unit_scale_atoms(rows, width, torch.device("cuda", index))
    return atoms


def is_tensor_fp8_linear_supported() -> tuple[bool, str | None]:
    return True, None


def is_supported(device=None) -> bool:
    """The op's capability probe: the device / library check every op makes, and the kernel's
    own verdict (always yes here: the kernels are compiled ahead of time)."""
    from ..._lib.gating import default_is_supported

    return default_is_supported(device) and is_tensor_fp8_linear_supported()[0]


def _check_out_dtype(dtype: torch.dtype) -> None:
    if dtype not in LINEAR_DTYPES:
        raise ValueError(f"tensor FP8 linear output must be bf16/fp16, got {dtype}")


def pack_tensor_fp8_linear_weight(weight: torch.Tensor,
                                  output_scale: torch.Tensor) -> TensorFP8LinearWeight:
    """Pack an E4M3 ``[N, K]`` weight with the one scale that dequantizes the product."""
    require_cuda_tensor("weight", weight)
    require_cuda_tensor("output_scale", output_scale)
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
    scale_value = float(output_scale)
    if not (scale_value >= 0.0 and scale_value != float("inf")):
        raise ValueError("output_scale must be finite and non-negative")
    out_features, in_features = (int(v) for v in weight.shape)
    if out_features <= 0:
        raise ValueError("out_features must be positive")
    if in_features <= 0 or in_features % SCALE_BLOCK:
        raise ValueError(
            f"tensor FP8 weight K must be a positive multiple of {SCALE_BLOCK}, got {in_features}")
    padded_in = round_up(in_features, K_STEP)
    return TensorFP8LinearWeight(
        values=pad_columns(weight.view(torch.uint8), padded_in).view(torch.float8_e4m3fn),
        scale_mma=_unit_scale_atoms(out_features, padded_in, weight.device),
        output_scale=output_scale.reshape(1).contiguous(), in_features=in_features,
        padded_in_features=padded_in, out_features=out_features)


def _forward(source_2d: torch.Tensor, weight_values: torch.Tensor, weight_scale_mma: torch.Tensor,
             output_scale: torch.Tensor, *, padded_in: int, out_features: int,
             out_dtype: torch.dtype, bias: torch.Tensor | None, stream_int: int | None) -> torch.Tensor:
    tokens = int(source_2d.shape[0])
    codes = pad_columns(source_2d.view(torch.uint8), padded_in)
    out = torch.empty((tokens, out_features), dtype=out_dtype, device=source_2d.device)
    del weight_scale_mma  # plain FP8: every block scale is 1.0 whatever the weight carries
    device = source_2d.device
    if launch.route_to_decode_kernel(tokens, out_features, device, 0):
        # Decode shapes: the weight-streaming kernel, which is written for block scales, fed
        # with cached scales of exactly 1.0 on both sides.
        launch.gemm_blockscaled(
            _native.KIND_MXFP8, codes, _cached_unit_atoms(tokens, padded_in, device).view(torch.uint8),
            weight_values, _cached_unit_atoms(out_features, padded_in, device).view(torch.uint8), out,
            output_scale, tokens, out_features, padded_in, stream_int=stream_int, bias=bias)
    else:
        # Everything else: the unscaled E4M3 MMA, no scale bytes at all.
        launch.gemm_blockscaled(_native.KIND_FP8, codes, None, weight_values, None, out,
                                output_scale, tokens, out_features, padded_in,
                                stream_int=stream_int, bias=bias)
    return out


@torch.library.custom_op("b12x::tensor_fp8_linear_fused", mutates_args=())
def _tensor_fp8_linear_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                                weight_scale_mma: torch.Tensor, output_scale: torch.Tensor,
                                padded_in_features: int, out_features: int, expected_m: int,
                                out_dtype: torch.dtype, stream_int: int | None) -> torch.Tensor:
    del expected_m
    return _forward(source_2d, weight_values, weight_scale_mma, output_scale,
                    padded_in=int(padded_in_features), out_features=int(out_features),
                    out_dtype=out_dtype, bias=None, stream_int=stream_int)


@_tensor_fp8_linear_fused_op.register_fake
def _tensor_fp8_linear_fused_fake(source_2d, weight_values, weight_scale_mma, output_scale,
                                  padded_in_features, out_features, expected_m, out_dtype,
                                  stream_int) -> torch.Tensor:
    return torch.empty((source_2d.shape[0], out_features), dtype=out_dtype,
                       device=source_2d.device)


@torch.library.custom_op("b12x::tensor_fp8_linear_bias_fused", mutates_args=())
def _tensor_fp8_linear_bias_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                                     weight_scale_mma: torch.Tensor, output_scale: torch.Tensor,
                                     bias: torch.Tensor, padded_in_features: int,
                                     out_features: int, stream_int: int | None) -> torch.Tensor:
    """The linear with its bias added in the GEMM epilogue (no counterpart op in the reference,
    which adds the bias after ``b12x::tensor_fp8_linear_fused``)."""
    return _forward(source_2d, weight_values, weight_scale_mma, output_scale,
                    padded_in=int(padded_in_features), out_features=int(out_features),
                    out_dtype=bias.dtype, bias=bias, stream_int=stream_int)


@_tensor_fp8_linear_bias_fused_op.register_fake
def _tensor_fp8_linear_bias_fused_fake(source_2d, weight_values, weight_scale_mma, output_scale,
                                       bias, padded_in_features, out_features,
                                       stream_int) -> torch.Tensor:
    return torch.empty((source_2d.shape[0], out_features), dtype=bias.dtype,
                       device=source_2d.device)


def tensor_fp8_linear(source: torch.Tensor, packed_weight: TensorFP8LinearWeight, *,
                      bias: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
                      expected_m: int | None = None, stream: object = None) -> torch.Tensor:
    """``output_scale * (source[..., K] @ W^T) (+ bias)`` for E4M3 ``source``."""
    require_cuda_tensor("source", source)
    if not isinstance(packed_weight, TensorFP8LinearWeight):
        raise TypeError("packed_weight must be a TensorFP8LinearWeight")
    if source.ndim < 2:
        raise ValueError(f"source must have at least 2 dims, got {tuple(source.shape)}")
    if source.dtype != torch.float8_e4m3fn:
        raise ValueError(f"source must be float8_e4m3fn, got {source.dtype}")
    rows = SourceRows.of(source, packed_in_features=packed_weight.in_features,
                         dtypes=(torch.float8_e4m3fn,),
                         dtype_error="source must be float8_e4m3fn, got {dtype}")
    if packed_weight.values.device != rows.rows.device:
        raise ValueError("source and packed weight must be on the same device")
    if expected_m is not None and int(expected_m) <= 0:
        raise ValueError("expected_m must be positive when provided")
    _check_out_dtype(out_dtype)
    n = int(packed_weight.out_features)
    if bias is not None:
        require_cuda_tensor("bias", bias)
        if bias.device != rows.rows.device:
            raise ValueError("bias must be on the same device as source")
        if bias.dtype != out_dtype or tuple(bias.shape) != (n,):
            raise ValueError(f"bias must have shape {(n,)} and dtype {out_dtype}, "
                             f"got shape={tuple(bias.shape)}, dtype={bias.dtype}")
    if rows.tokens == 0:
        return rows.restore(torch.empty((0, n), dtype=out_dtype, device=rows.rows.device), n)
    if bias_fuses(bias, out_dtype, n):
        output = torch.ops.b12x.tensor_fp8_linear_bias_fused(
            rows.rows, packed_weight.values, packed_weight.scale_mma, packed_weight.output_scale,
            bias, packed_weight.padded_in_features, n, cuda_stream_to_int(stream))
        return rows.restore(output, n)
    output = torch.ops.b12x.tensor_fp8_linear_fused(
        rows.rows, packed_weight.values, packed_weight.scale_mma, packed_weight.output_scale,
        packed_weight.padded_in_features, n,
        int(expected_m) if expected_m is not None else rows.tokens, out_dtype,
        cuda_stream_to_int(stream))
    if bias is not None:
        output = output + bias
    return rows.restore(output, n)


def prewarm_tensor_fp8_linear(packed_weight: TensorFP8LinearWeight, token_counts: Iterable[int],
                              *, out_dtype: torch.dtype = torch.bfloat16,
                              stream: object = None) -> int:
    """Run each token count once (library load, kernel attributes, the cached unit-scale atoms
    and workspaces) so that a later CUDA-graph capture allocates nothing but its output."""
    counts = sorted({int(t) for t in token_counts if int(t) > 0})
    with torch.inference_mode():
        for tokens in counts:
            probe = torch.zeros((tokens, packed_weight.in_features), dtype=torch.float8_e4m3fn,
                                device=packed_weight.values.device)
            tensor_fp8_linear(probe, packed_weight, out_dtype=out_dtype, expected_m=tokens,
                              stream=stream)
    return len(counts)


__all__ = ["TensorFP8LinearWeight", "is_tensor_fp8_linear_supported",
           "pack_tensor_fp8_linear_weight", "prewarm_tensor_fp8_linear", "tensor_fp8_linear"]
