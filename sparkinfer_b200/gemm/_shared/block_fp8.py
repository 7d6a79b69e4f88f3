"""Block-FP8 linear (DeepSeek-style 128x128 weight scales) on the MXFP8 GEMM.

Planned lifecycle ``Caps -> plan -> bind -> run`` plus the one-shot form and the two torch
custom ops, standing in for b12x/gemm/_shared/block_fp8.py:53-818. ``plan`` and ``bind`` are
host code over views of one caller-owned ``uint8`` scratch (they work on CPU tensors);
``run`` enqueues the row quantizer and the block-scaled GEMM and allocates nothing when a
binding is given.

Scratch layout (bytes, each region 1024-aligned): E4M3 activations ``[T, K]`` | UE8M0
row scales ``[1, T, K/32]`` | MMA-layout scale atoms ``ceil(T/128) * (K/128) * 512``.
"""

from __future__ import annotations

import logging
import math
import os
import time
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Iterable, Sequence

import torch

from ..._lib.dense_gemm import dense_gemm
from ..._lib.launch import cuda_stream_to_int
from ..._lib.mxfp8_rows import (
    MXFP8Rows,
    MXFP8_SCALE_K_TILE,
    MXFP8_SCALE_ROW_TILE,
    MXFP8_SCALE_VEC_SIZE,
    _check_gpu_tensor,
    _check_mxfp8_k,
    _check_mxfp8_rows_storage,
    empty_dense_gemm_mnl_view,
    empty_mxfp8_rows_bases,
    mxfp8_rows_from_bases,
    pack_fp8_block_scaled_weight_mxfp8,
    quantize_mxfp8_rows,
)
from ..._lib.scratch import ScratchBufferSpec, scratch_buffer_spec, scratch_tensor

logger = logging.getLogger(__name__)
_B12X_TIMING = os.getenv("B12X_TIMING", "0") == "1"
_B12X_TIMING_THRESHOLD_MS = float(os.getenv("B12X_TIMING_THRESHOLD_MS", "0"))
_SCRATCH_ALIGN_BYTES = 1024


@dataclass(frozen=True)
class BlockFP8LinearWeight:
    weight: MXFP8Rows
    in_features: int
    out_features: int
    block_size: tuple[int, int]


@dataclass(frozen=True, kw_only=True)
class BlockFP8LinearBinding:
    """Runtime tensors of one bound call; the scratch views live in ``x_q``."""

    source: torch.Tensor
    packed_weight: BlockFP8LinearWeight
    x_q: MXFP8Rows
    output: torch.Tensor
    bias: torch.Tensor | None = None
    expected_m: int | None = None

    def run(self, *, stream: object = None) -> torch.Tensor:
        return block_fp8_linear_mxfp8(binding=self, stream=stream)


@dataclass(frozen=True, kw_only=True)
class BlockFP8LinearScratchCaps:
    device: torch.device | str
    max_tokens: int
    in_features: int
    out_features: int
    output_dtype: torch.dtype = torch.bfloat16

    def __post_init__(self) -> None:
        device = torch.device(self.device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        object.__setattr__(self, "device", device)
        for name in ("max_tokens", "in_features", "out_features"):
            object.__setattr__(self, name, max(int(getattr(self, name)), 1))
        _check_mxfp8_k(self.in_features)
        if self.output_dtype not in (torch.bfloat16, torch.float16):
            raise ValueError(f"output_dtype must be bf16/fp16, got {self.output_dtype}")


@dataclass(frozen=True, kw_only=True)
class _ScratchLayout:
    nbytes: int
    values_offset: int
    scale_rows_offset: int
    scale_mma_offset: int
    scale_mma_shape: tuple[int, int, int, int, int, int]


def _align_up(value: int, alignment: int) -> int:
    return -(-int(value) // int(alignment)) * int(alignment)


def _c_dtype_name(dtype: torch.dtype) -> str:
    if dtype == torch.bfloat16:
        return "bfloat16"
    if dtype == torch.float16:
        return "float16"
    raise ValueError(f"b12x block FP8 linear output dtype must be bf16/fp16, got {dtype}")


def _scratch_layout(*, tokens: int, in_features: int, output_dtype: torch.dtype) -> _ScratchLayout:
    tokens = max(int(tokens), 1)
    in_features = max(int(in_features), 1)
    _check_mxfp8_k(in_features)
    _c_dtype_name(output_dtype)
    sf_k = in_features // MXFP8_SCALE_VEC_SIZE
    values_offset = 0
    scale_rows_offset = _align_up(values_offset + tokens * in_features, _SCRATCH_ALIGN_BYTES)
    scale_mma_offset = _align_up(scale_rows_offset + tokens * sf_k, _SCRATCH_ALIGN_BYTES)
    shape = (1, math.ceil(tokens / MXFP8_SCALE_ROW_TILE), math.ceil(sf_k / MXFP8_SCALE_K_TILE),
             32, 4, 4)
    return _ScratchLayout(
        nbytes=max(scale_mma_offset + math.prod(shape), 1), values_offset=values_offset,
        scale_rows_offset=scale_rows_offset, scale_mma_offset=scale_mma_offset,
        scale_mma_shape=shape)


def _scratch_view(scratch: torch.Tensor, *, offset: int, shape: tuple[int, ...],
                  dtype: torch.dtype) -> torch.Tensor:
    return scratch.narrow(0, offset, math.prod(shape)).view(dtype).view(shape)


def _x_q_from_scratch(scratch: torch.Tensor, *, tokens: int, in_features: int,
                      output_dtype: torch.dtype) -> MXFP8Rows:
    layout = _scratch_layout(tokens=tokens, in_features=in_features, output_dtype=output_dtype)
    if scratch.dtype != torch.uint8:
        raise TypeError(f"block FP8 linear scratch must have dtype torch.uint8, got {scratch.dtype}")
    if not scratch.is_contiguous():
        raise ValueError("block FP8 linear scratch must be contiguous")
    if int(scratch.numel()) < layout.nbytes:
        raise ValueError(
            f"block FP8 linear scratch has {int(scratch.numel())} bytes, requires {layout.nbytes}")
    values = _scratch_view(scratch, offset=layout.values_offset, shape=(tokens, in_features),
                           dtype=torch.float8_e4m3fn)
    scale_rows = _scratch_view(scratch, offset=layout.scale_rows_offset,
                               shape=(1, tokens, in_features // MXFP8_SCALE_VEC_SIZE),
                               dtype=torch.uint8)
    scale_mma = _scratch_view(scratch, offset=layout.scale_mma_offset,
                              shape=layout.scale_mma_shape, dtype=torch.uint8)
    # Neutral UE8M0 (1.0) in every lane the quantizer may not touch.
    scale_rows.fill_(127)
    scale_mma.fill_(127)
    return MXFP8Rows(
        values=values,
        scale_rows=scale_rows.view(torch.float8_e8m0fnu),
        scale_mma=scale_mma.view(torch.float8_e8m0fnu).permute(3, 4, 1, 5, 2, 0),
    )


def _source_2d(source: torch.Tensor) -> torch.Tensor:
    if source.ndim == 0:
        raise ValueError("source must have at least one dimension")
    return source.view(-1, source.shape[-1])


def _check_block_fp8_linear_tensors(x_q: MXFP8Rows, output: torch.Tensor, *, tokens: int,
                                    packed_weight: BlockFP8LinearWeight,
                                    output_dtype: torch.dtype) -> None:
    _check_mxfp8_rows_storage(x_q, m=tokens, k=packed_weight.in_features, num_groups=1)
    want = (tokens, packed_weight.out_features, 1)
    if tuple(output.shape) != want:
        raise ValueError(f"output must have shape {want}, got {tuple(output.shape)}")
    if output.dtype != output_dtype:
        raise ValueError(f"output dtype {output.dtype} does not match input {output_dtype}")


def build_block_fp8_linear_binding(*, source: torch.Tensor, packed_weight: BlockFP8LinearWeight,
                                   x_q: MXFP8Rows, output: torch.Tensor,
                                   bias: torch.Tensor | None = None,
                                   expected_m: int | None = None) -> BlockFP8LinearBinding:
    if not isinstance(packed_weight, BlockFP8LinearWeight):
        raise TypeError("packed_weight must be a BlockFP8LinearWeight")
    source_2d = _source_2d(source)
    tokens, in_features = map(int, source_2d.shape)
    if in_features != packed_weight.in_features:
        raise ValueError(
            f"input K={in_features} does not match packed weight K={packed_weight.in_features}")
    if source_2d.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"source dtype must be bf16/fp16, got {source_2d.dtype}")
    _check_block_fp8_linear_tensors(x_q, output, tokens=tokens, packed_weight=packed_weight,
                                    output_dtype=source_2d.dtype)
    return BlockFP8LinearBinding(source=source, packed_weight=packed_weight, x_q=x_q,
                                 output=output, bias=bias, expected_m=expected_m)


@dataclass(frozen=True)
class BlockFP8LinearScratchPlan:
    caps: BlockFP8LinearScratchCaps
    _scratch_specs: tuple[ScratchBufferSpec, ...]

    def scratch_specs(self) -> tuple[ScratchBufferSpec, ...]:
        return self._scratch_specs

    def shapes_and_dtypes(self) -> tuple[tuple[tuple[int, ...], torch.dtype], ...]:
        return tuple((spec.shape, spec.dtype) for spec in self._scratch_specs)

    def bind(self, *, scratch: torch.Tensor | Mapping[str, torch.Tensor] | Sequence[torch.Tensor],
             source: torch.Tensor, packed_weight: BlockFP8LinearWeight, output: torch.Tensor,
             bias: torch.Tensor | None = None,
             expected_m: int | None = None) -> BlockFP8LinearBinding:
        source_2d = _source_2d(source)
        tokens, in_features = map(int, source_2d.shape)
        if tokens > int(self.caps.max_tokens):
            raise ValueError(
                f"source tokens {tokens} exceed block-FP8 scratch capacity {self.caps.max_tokens}")
        if in_features != int(self.caps.in_features):
            raise ValueError(
                f"source K={in_features} does not match scratch in_features={self.caps.in_features}")
        if int(packed_weight.out_features) != int(self.caps.out_features):
            raise ValueError(
                f"packed weight out_features {packed_weight.out_features} does not match "
                f"scratch out_features={self.caps.out_features}")
        if source_2d.dtype != self.caps.output_dtype:
            raise ValueError(
                f"source dtype {source_2d.dtype} does not match scratch "
                f"output_dtype={self.caps.output_dtype}")
        flat = scratch_tensor(scratch, self._scratch_specs, owner="block FP8 linear")
        x_q = _x_q_from_scratch(flat, tokens=tokens, in_features=self.caps.in_features,
                                output_dtype=self.caps.output_dtype)
        return build_block_fp8_linear_binding(source=source, packed_weight=packed_weight, x_q=x_q,
                                              output=output, bias=bias, expected_m=expected_m)


def plan_block_fp8_linear_scratch(caps: BlockFP8LinearScratchCaps) -> BlockFP8LinearScratchPlan:
    layout = _scratch_layout(tokens=caps.max_tokens, in_features=caps.in_features,
                             output_dtype=caps.output_dtype)
    spec = scratch_buffer_spec("block_fp8_linear.scratch", nbytes=layout.nbytes, device=caps.device)
    return BlockFP8LinearScratchPlan(caps=caps, _scratch_specs=(spec,))


def pack_block_fp8_linear_weight_mxfp8(weight: torch.Tensor, weight_scale: torch.Tensor, *,
                                       block_size: Sequence[int] = (128, 128)) -> BlockFP8LinearWeight:
    """E4M3 checkpoint weight ``[N, K]`` + 128x128 block scales -> GEMM-ready MXFP8 rows
    (codes re-derived on power-of-two scales when the checkpoint scales are not)."""
    _check_gpu_tensor("weight", weight)
    _check_gpu_tensor("weight_scale", weight_scale)
    if len(block_size) != 2 or (int(block_size[0]), int(block_size[1])) != (128, 128):
        raise ValueError(
            f"b12x block FP8 linear currently supports 128x128 weight blocks, got {block_size}")
    if weight.ndim != 2:
        raise ValueError(f"weight must have shape [N,K], got {tuple(weight.shape)}")
    out_features, in_features = map(int, weight.shape)
    _check_mxfp8_k(in_features)
    if out_features <= 0:
        raise ValueError("out_features must be positive")
    packed = pack_fp8_block_scaled_weight_mxfp8(weight.detach(), weight_scale.detach(),
                                                m=out_features, k=in_features, num_groups=1)
    return BlockFP8LinearWeight(weight=packed, in_features=in_features, out_features=out_features,
                                block_size=(128, 128))


@torch.library.custom_op("b12x::quantize_block_fp8_linear_input_mxfp8_alloc", mutates_args=())
def _quantize_input_alloc_op(source_tk: torch.Tensor, tokens: int,
                             in_features: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    bases = empty_mxfp8_rows_bases(tokens, in_features, num_groups=1, device=source_tk.device)
    out = mxfp8_rows_from_bases(*bases, tokens, in_features, num_groups=1)
    quantize_mxfp8_rows(source_tk, out.values, out.scale_rows, out.scale_mma)
    return bases


@_quantize_input_alloc_op.register_fake
def _quantize_input_alloc_fake(source_tk: torch.Tensor, tokens: int, in_features: int):
    return empty_mxfp8_rows_bases(tokens, in_features, num_groups=1, device=source_tk.device)


def quantize_block_fp8_linear_input_mxfp8(source_tk: torch.Tensor, *,
                                          out: MXFP8Rows | None = None) -> MXFP8Rows:
    """Quantize dense BF16/FP16 rows ``[tokens, K]`` to MXFP8 rows."""
    _check_gpu_tensor("source_tk", source_tk)
    if source_tk.ndim != 2:
        raise ValueError(f"source_tk must have shape [tokens,K], got {tuple(source_tk.shape)}")
    tokens, in_features = map(int, source_tk.shape)
    if tokens <= 0:
        raise ValueError("tokens must be positive")
    _check_mxfp8_k(in_features)
    if out is None:
        bases = torch.ops.b12x.quantize_block_fp8_linear_input_mxfp8_alloc(
            source_tk, tokens, in_features)
        return mxfp8_rows_from_bases(*bases, tokens, in_features, num_groups=1)
    _check_mxfp8_rows_storage(out, m=tokens, k=in_features, num_groups=1)
    quantize_mxfp8_rows(source_tk, out.values, out.scale_rows, out.scale_mma)
    return out


def _gemm_on_quantized(x_q: MXFP8Rows, weight: MXFP8Rows, *, tokens: int, in_features: int,
                       out_features: int, c_dtype: str, out: torch.Tensor | None,
                       expected_m: int | None, stream: object) -> torch.Tensor:
    return dense_gemm(
        (x_q.values.reshape(tokens, in_features, 1), x_q.scale_mma),
        (weight.values.reshape(out_features, in_features, 1), weight.scale_mma),
        ab_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu", c_dtype=c_dtype,
        sf_vec_size=MXFP8_SCALE_VEC_SIZE, out=out, expected_m=expected_m,
        sfb_k_replicated=True, stream=stream)


@torch.library.custom_op("b12x::block_fp8_linear_mxfp8_fused", mutates_args=())
def _block_fp8_linear_mxfp8_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                                     weight_scale_rows: torch.Tensor,
                                     weight_scale_mma: torch.Tensor, in_features: int,
                                     out_features: int, expected_m: int,
                                     stream_int: int | None) -> torch.Tensor:
    tokens = int(source_2d.shape[0])
    x_q = quantize_block_fp8_linear_input_mxfp8(source_2d)
    weight = MXFP8Rows(values=weight_values, scale_rows=weight_scale_rows,
                       scale_mma=weight_scale_mma)
    return _gemm_on_quantized(
        x_q, weight, tokens=tokens, in_features=in_features, out_features=out_features,
        c_dtype=_c_dtype_name(source_2d.dtype), out=None,
        expected_m=None if expected_m == 0 else expected_m, stream=stream_int)[:, :, 0]


@_block_fp8_linear_mxfp8_fused_op.register_fake
def _block_fp8_linear_mxfp8_fused_fake(source_2d, weight_values, weight_scale_rows,
                                       weight_scale_mma, in_features, out_features, expected_m,
                                       stream_int) -> torch.Tensor:
    return torch.empty((source_2d.shape[0], out_features), dtype=source_2d.dtype,
                       device=source_2d.device)


def block_fp8_linear_mxfp8(source: torch.Tensor | None = None,
                           packed_weight: BlockFP8LinearWeight | None = None, *,
                           bias: torch.Tensor | None = None,
                           binding: BlockFP8LinearBinding | None = None,
                           expected_m: int | None = None, stream: object = None) -> torch.Tensor:
    """Run a block-FP8 linear: quantize activation rows to MXFP8, then the MXFP8 GEMM.

    With ``binding=`` every tensor (scratch views, output) is caller-owned and nothing is
    allocated; the one-shot form dispatches through ``b12x::block_fp8_linear_mxfp8_fused``.
    """
    if binding is not None:
        extras = [name for name, value in (("source", source), ("packed_weight", packed_weight),
                                           ("bias", bias)) if value is not None]
        if extras:
            raise ValueError(
                "block FP8 linear binding owns source, packed weight, scratch tensors, and bias; "
                f"do not also pass {', '.join(extras)}")
        source, packed_weight = binding.source, binding.packed_weight
        bias, expected_m = binding.bias, binding.expected_m
    if source is None or packed_weight is None:
        raise TypeError("block_fp8_linear_mxfp8 requires source and packed_weight or binding")
    _check_gpu_tensor("source", source)
    if not isinstance(packed_weight, BlockFP8LinearWeight):
        raise TypeError("packed_weight must be a BlockFP8LinearWeight")
    source_2d = _source_2d(source)
    tokens, in_features = map(int, source_2d.shape)
    if in_features != packed_weight.in_features:
        raise ValueError(
            f"input K={in_features} does not match packed weight K={packed_weight.in_features}")
    if source_2d.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"source dtype must be bf16/fp16, got {source_2d.dtype}")

    if binding is None:
        output = torch.ops.b12x.block_fp8_linear_mxfp8_fused(
            source_2d, packed_weight.weight.values, packed_weight.weight.scale_rows,
            packed_weight.weight.scale_mma, packed_weight.in_features,
            packed_weight.out_features, int(expected_m) if expected_m is not None else 0,
            cuda_stream_to_int(stream))
        if bias is not None:
            output = output + bias
        return output.view(*source.shape[:-1], packed_weight.out_features)

    _check_block_fp8_linear_tensors(binding.x_q, binding.output, tokens=tokens,
                                    packed_weight=packed_weight, output_dtype=source_2d.dtype)
    t0 = time.perf_counter() if _B12X_TIMING else 0.0
    quantize_mxfp8_rows(source_2d, binding.x_q.values, binding.x_q.scale_rows,
                        binding.x_q.scale_mma, stream=stream)
    t_quant = time.perf_counter() if _B12X_TIMING else 0.0
    output = _gemm_on_quantized(
        binding.x_q, packed_weight.weight, tokens=tokens, in_features=in_features,
        out_features=packed_weight.out_features, c_dtype=_c_dtype_name(source_2d.dtype),
        out=binding.output, expected_m=expected_m, stream=stream)[:, :, 0]
    if bias is not None:
        output += bias
    if _B12X_TIMING:
        t_done = time.perf_counter()
        total_ms = (t_done - t0) * 1000.0
        if total_ms >= _B12X_TIMING_THRESHOLD_MS:
            logger.warning(
                "b12x_block_fp8_linear timing tokens=%d in=%d out=%d quant_enqueue=%.3fms "
                "dense_gemm=%.3fms total=%.3fms", tokens, in_features,
                packed_weight.out_features, (t_quant - t0) * 1000.0,
                (t_done - t_quant) * 1000.0, total_ms)
    return output.view(*source.shape[:-1], packed_weight.out_features)


def prewarm_block_fp8_linear_mxfp8(packed_weight: BlockFP8LinearWeight,
                                   token_counts: Iterable[int], *,
                                   output_dtype: torch.dtype = torch.bfloat16,
                                   expected_m: int | None = None, stream: object = None) -> None:
    """Run the bound path once per planned token count (loads the library, sets kernel
    attributes, creates the per-device status buffer) so later calls are capture safe."""
    if not isinstance(packed_weight, BlockFP8LinearWeight):
        raise TypeError("packed_weight must be a BlockFP8LinearWeight")
    if output_dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"output_dtype must be bf16/fp16, got {output_dtype}")
    device = packed_weight.weight.values.device
    counts = sorted({int(t) for t in token_counts if int(t) > 0})
    with torch.inference_mode():
        for tokens in counts:
            plan = plan_block_fp8_linear_scratch(BlockFP8LinearScratchCaps(
                device=device, max_tokens=tokens, in_features=packed_weight.in_features,
                out_features=packed_weight.out_features, output_dtype=output_dtype))
            spec = plan.scratch_specs()[0]
            binding = plan.bind(
                scratch=torch.empty(spec.shape, dtype=spec.dtype, device=spec.device),
                source=torch.zeros((tokens, packed_weight.in_features), dtype=output_dtype,
                                   device=device),
                packed_weight=packed_weight,
                output=empty_dense_gemm_mnl_view(tokens, packed_weight.out_features, 1,
                                                 device=device, dtype=output_dtype),
                expected_m=expected_m)
            block_fp8_linear_mxfp8(binding=binding, stream=stream)
        if counts:
            torch.cuda.synchronize(device)


__all__ = [
    "BlockFP8LinearBinding", "BlockFP8LinearScratchCaps", "BlockFP8LinearScratchPlan",
    "BlockFP8LinearWeight", "build_block_fp8_linear_binding", "block_fp8_linear_mxfp8",
    "pack_block_fp8_linear_weight_mxfp8", "plan_block_fp8_linear_scratch",
    "prewarm_block_fp8_linear_mxfp8", "quantize_block_fp8_linear_input_mxfp8",
]
