"""What the three FP8 linears share: source-row handling, the byte plan of a quantized
activation, and the forward step ``quantize rows -> block-scaled GEMM (+ bias)``.

The linears of the reference (b12x/gemm/mxfp8_linear/_kernel.py, b12x/gemm/_shared/block_fp8.py,
b12x/gemm/tensor_fp8_linear/_kernel.py) each carry their own copy of this logic; here they are
thin front ends over one core, and the bias add rides in the GEMM epilogue whenever the bias
has the output's dtype (otherwise it is added afterwards, with torch's type promotion, exactly
as ``output + bias`` would).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import _native
from . import launch
from .launch import cuda_stream_to_int
from .mxfp8_rows import MXFP8Rows, SCALE_BLOCK, quantize_mxfp8_rows

K_STEP = 128            # the GEMM consumes K in 128-element steps
REGION_ALIGN = 1024     # byte alignment of the regions inside an activation scratch
LINEAR_DTYPES = {torch.bfloat16: "bfloat16", torch.float16: "float16"}


def round_up(value: int, multiple: int) -> int:
    return -(-int(value) // int(multiple)) * int(multiple)


def output_dtype_name(dtype: torch.dtype, owner: str) -> str:
    """dtype string of a linear's output; the linears produce BF16 or FP16 only."""
    name = LINEAR_DTYPES.get(dtype)
    if name is None:
        raise ValueError(f"{owner} output dtype must be bf16/fp16, got {dtype}")
    return name


def require_cuda_tensor(name: str, tensor) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not tensor.is_cuda:
        raise ValueError(f"{name} must be on CUDA")


def pad_columns(rows: torch.Tensor, width: int) -> torch.Tensor:
    """``rows [T, K]`` with K brought up to ``width`` by zero columns (a copy only if needed)."""
    have = int(rows.shape[1])
    if have == width:
        return rows.contiguous()
    return torch.nn.functional.pad(rows, (0, width - have))


@dataclass(frozen=True)
class SourceRows:
    """A linear's input seen as ``[tokens, K]`` rows."""

    rows: torch.Tensor
    tokens: int
    in_features: int
    leading_shape: tuple[int, ...]

    @classmethod
    def of(cls, source: torch.Tensor, *, packed_in_features: int, dtypes: tuple[torch.dtype, ...],
           dtype_error: str, copy: bool = True) -> "SourceRows":
        if source.ndim == 0:
            raise ValueError("source must have at least one dimension")
        k = int(source.shape[-1])
        rows = source.reshape(-1, k)
        if copy:
            rows = rows.contiguous()
        if k != int(packed_in_features):
            raise ValueError(f"input K={k} does not match packed weight K={packed_in_features}")
        if rows.dtype not in dtypes:
            raise ValueError(dtype_error.format(dtype=rows.dtype))
        return cls(rows=rows, tokens=int(rows.shape[0]), in_features=k,
                   leading_shape=tuple(source.shape[:-1]))

    def restore(self, output_2d: torch.Tensor, out_features: int) -> torch.Tensor:
        return output_2d.view(*self.leading_shape, out_features)


@dataclass(frozen=True)
class ActivationPlan:
    """Byte plan of one MXFP8-quantized activation ``[tokens, K]`` inside a flat ``uint8``
    buffer: E4M3 codes, then the row-major UE8M0 bytes, then the scale atoms, each region
    starting on a 1 KiB boundary."""

    tokens: int
    in_features: int

    @property
    def scale_cols(self) -> int:
        return self.in_features // SCALE_BLOCK

    @property
    def atom_grid(self) -> tuple[int, int]:
        return math.ceil(self.tokens / 128), math.ceil(self.scale_cols / 4)

    @property
    def offsets(self) -> tuple[int, int, int]:
        rows_at = round_up(self.tokens * self.in_features, REGION_ALIGN)
        atoms_at = round_up(rows_at + self.tokens * self.scale_cols, REGION_ALIGN)
        return 0, rows_at, atoms_at

    @property
    def nbytes(self) -> int:
        row_tiles, k_tiles = self.atom_grid
        return max(self.offsets[2] + row_tiles * k_tiles * 512, 1)

    def carve(self, scratch: torch.Tensor) -> MXFP8Rows:
        """Views of ``scratch`` (no allocation). Scale bytes start as UE8M0 1.0 so that lanes the
        quantizer never writes (rows beyond ``tokens`` inside the last atom row) are neutral."""
        if scratch.dtype != torch.uint8:
            raise TypeError(f"block FP8 linear scratch must have dtype torch.uint8, got {scratch.dtype}")
        if not scratch.is_contiguous():
            raise ValueError("block FP8 linear scratch must be contiguous")
        if int(scratch.numel()) < self.nbytes:
            raise ValueError(
                f"block FP8 linear scratch has {int(scratch.numel())} bytes, requires {self.nbytes}")
        values_at, rows_at, atoms_at = self.offsets
        row_tiles, k_tiles = self.atom_grid
        values = scratch.narrow(0, values_at, self.tokens * self.in_features)
        scale_rows = scratch.narrow(0, rows_at, self.tokens * self.scale_cols)
        atoms = scratch.narrow(0, atoms_at, row_tiles * k_tiles * 512)
        scale_rows.fill_(127)
        atoms.fill_(127)
        return MXFP8Rows(
            values=values.view(torch.float8_e4m3fn).view(self.tokens, self.in_features),
            scale_rows=scale_rows.view(torch.float8_e8m0fnu).view(1, self.tokens, self.scale_cols),
            scale_mma=atoms.view(torch.float8_e8m0fnu).view(1, row_tiles, k_tiles, 32, 4, 4)
            .permute(3, 4, 1, 5, 2, 0))


def bias_fuses(bias: torch.Tensor | None, out_dtype: torch.dtype, out_features: int) -> bool:
    """Whether the GEMM epilogue can take the bias: a contiguous CUDA ``[N]`` vector of the output
    dtype. Anything else (FP32 bias on a BF16 linear, broadcast shapes) goes through torch."""
    return (bias is not None and bias.is_cuda and bias.dtype == out_dtype and bias.ndim == 1
            and int(bias.shape[0]) == out_features and bias.stride(0) == 1)


def mxfp8_gemm(x_q: MXFP8Rows, weight_values: torch.Tensor, weight_scale_mma: torch.Tensor, *,
               tokens: int, k: int, out_features: int, out: torch.Tensor,
               bias: torch.Tensor | None, stream: object) -> None:
    """``out [T, N, 1] = x_q @ W^T (+ bias)`` on MXFP8 rows, straight through the launcher."""
    atoms = x_q.scale_mma
    launch.gemm_blockscaled(
        _native.KIND_MXFP8, x_q.values, atoms.view(torch.uint8) if atoms.dtype != torch.uint8 else atoms,
        weight_values, weight_scale_mma.view(torch.uint8) if weight_scale_mma.dtype != torch.uint8
        else weight_scale_mma, out.select(2, 0), None, tokens, out_features, k,
        ldc=out.stride(0) if tokens > 1 else out_features, stream_int=cuda_stream_to_int(stream),
        bias=bias)


def quantize_then_gemm(rows: torch.Tensor, weight_values: torch.Tensor,
                       weight_scale_mma: torch.Tensor, *, padded_k: int, out_features: int,
                       x_q: MXFP8Rows, out: torch.Tensor, bias: torch.Tensor | None,
                       stream: object, bias_in_place: bool = False) -> torch.Tensor:
    """The forward step of the MXFP8-based linears on caller-provided buffers: row-quantize
    ``rows [T, padded_k]`` into ``x_q``, multiply into ``out [T, N, 1]``. Returns ``out[:, :, 0]``
    with the bias applied: in the GEMM epilogue when :func:`bias_fuses`, else by torch (into
    ``out`` itself with ``bias_in_place``, as a bound call must, or as a new tensor)."""
    tokens = int(rows.shape[0])
    quantize_mxfp8_rows(rows, x_q.values, x_q.scale_rows, x_q.scale_mma, stream=stream)
    fused = bias_fuses(bias, out.dtype, out_features)
    mxfp8_gemm(x_q, weight_values, weight_scale_mma, tokens=tokens, k=padded_k,
               out_features=out_features, out=out, bias=bias if fused else None, stream=stream)
    result = out[:, :, 0]
    if bias is not None and not fused:
        result = result.add_(bias) if bias_in_place else result + bias
    return result


__all__ = ["ActivationPlan", "K_STEP", "LINEAR_DTYPES", "SourceRows", "bias_fuses", "mxfp8_gemm",
           "output_dtype_name", "pad_columns", "quantize_then_gemm", "require_cuda_tensor",
           "round_up"]
