"""Block-FP8 linear (DeepSeek-style 128x128 weight scales) on the MXFP8 GEMM.

Lifecycle ``Caps -> plan -> bind -> run`` plus the one-shot form and the two torch custom ops
of b12x/gemm/_shared/block_fp8.py:53-818 (same names, fields, op schemas and errors).
``plan`` sizes one opaque ``uint8`` scratch; ``bind`` carves the quantized-activation views out
of the caller's scratch (host code, works on CPU tensors, allocates nothing); ``run`` enqueues
the row quantizer and the GEMM, with the bias folded into the GEMM epilogue when it has the
output's dtype. The scratch bytes are described by :class:`ActivationPlan`:
E4M3 activations ``[T, K]`` | UE8M0 row scales ``[1, T, K/32]`` | scale atoms, each region
1 KiB aligned.
"""

from __future__ import annotations

import logging
import os
import time
from collections.abc import Mapping
from dataclasses import dataclass, field
from typing import Iterable, Sequence

import torch

from ..._lib.linear_core import (
    ActivationPlan,
    SourceRows,
    mxfp8_gemm,
    output_dtype_name,
    quantize_then_gemm,
)
from ..._lib.launch import cuda_stream_to_int
from ..._lib.mxfp8_rows import (
    MXFP8Rows,
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
_LOG_TIMING = os.getenv("B12X_TIMING", "0") == "1"
_LOG_TIMING_FROM_MS = float(os.getenv("B12X_TIMING_THRESHOLD_MS", "0"))
_OWNER = "b12x block FP8 linear"
_SOURCE_DTYPES = (torch.bfloat16, torch.float16)
_SOURCE_DTYPE_ERROR = "source dtype must be bf16/fp16, got {dtype}"


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
    # Set by build_block_fp8_linear_binding, which has validated every tensor against the
    # packed weight: a bound run then goes straight to the two launches. A binding made by
    # hand (this constructor) is validated on every run.
    prechecked_rows: SourceRows | None = field(default=None, repr=False, compare=False)

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
        for field in ("max_tokens", "in_features", "out_features"):
            object.__setattr__(self, field, max(int(getattr(self, field)), 1))
        _check_mxfp8_k(self.in_features)
        if self.output_dtype not in _SOURCE_DTYPES:
            raise ValueError(f"output_dtype must be bf16/fp16, got {self.output_dtype}")


def _source_rows(source: torch.Tensor, packed_weight: BlockFP8LinearWeight) -> SourceRows:
    return SourceRows.of(source, packed_in_features=packed_weight.in_features,
                         dtypes=_SOURCE_DTYPES, dtype_error=_SOURCE_DTYPE_ERROR, copy=False)


def _check_bound_tensors(x_q: MXFP8Rows, output: torch.Tensor, rows: SourceRows,
                         packed_weight: BlockFP8LinearWeight) -> None:
    _check_mxfp8_rows_storage(x_q, m=rows.tokens, k=packed_weight.in_features, num_groups=1)
    want = (rows.tokens, packed_weight.out_features, 1)
    if tuple(output.shape) != want:
        raise ValueError(f"output must have shape {want}, got {tuple(output.shape)}")
    if output.dtype != rows.rows.dtype:
        raise ValueError(f"output dtype {output.dtype} does not match input {rows.rows.dtype}")


def build_block_fp8_linear_binding(*, source: torch.Tensor, packed_weight: BlockFP8LinearWeight,
                                   x_q: MXFP8Rows, output: torch.Tensor,
                                   bias: torch.Tensor | None = None,
                                   expected_m: int | None = None) -> BlockFP8LinearBinding:
    if not isinstance(packed_weight, BlockFP8LinearWeight):
        raise TypeError("packed_weight must be a BlockFP8LinearWeight")
    rows = _source_rows(source, packed_weight)
    _check_bound_tensors(x_q, output, rows, packed_weight)
    on_gpu = isinstance(source, torch.Tensor) and source.is_cuda
    return BlockFP8LinearBinding(source=source, packed_weight=packed_weight, x_q=x_q,
                                 output=output, bias=bias, expected_m=expected_m,
                                 prechecked_rows=rows if on_gpu else None)


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
        caps = self.caps
        tokens = source.numel() // max(int(source.shape[-1]), 1) if source.ndim else 0
        k = int(source.shape[-1]) if source.ndim else 0
        if tokens > caps.max_tokens:
            raise ValueError(
                f"source tokens {tokens} exceed block-FP8 scratch capacity {caps.max_tokens}")
        if k != caps.in_features:
            raise ValueError(
                f"source K={k} does not match scratch in_features={caps.in_features}")
        if int(packed_weight.out_features) != caps.out_features:
            raise ValueError(
                f"packed weight out_features {packed_weight.out_features} does not match "
                f"scratch out_features={caps.out_features}")
        if source.dtype != caps.output_dtype:
            raise ValueError(
                f"source dtype {source.dtype} does not match scratch "
                f"output_dtype={caps.output_dtype}")
        flat = scratch_tensor(scratch, self._scratch_specs, owner="block FP8 linear")
        x_q = ActivationPlan(tokens=tokens, in_features=caps.in_features).carve(flat)
        return build_block_fp8_linear_binding(source=source, packed_weight=packed_weight, x_q=x_q,
                                              output=output, bias=bias, expected_m=expected_m)


def plan_block_fp8_linear_scratch(caps: BlockFP8LinearScratchCaps) -> BlockFP8LinearScratchPlan:
    output_dtype_name(caps.output_dtype, _OWNER)
    nbytes = ActivationPlan(tokens=caps.max_tokens, in_features=caps.in_features).nbytes
    spec = scratch_buffer_spec("block_fp8_linear.scratch", nbytes=nbytes, device=caps.device)
    return BlockFP8LinearScratchPlan(caps=caps, _scratch_specs=(spec,))


def pack_block_fp8_linear_weight_mxfp8(weight: torch.Tensor, weight_scale: torch.Tensor, *,
                                       block_size: Sequence[int] = (128, 128)) -> BlockFP8LinearWeight:
    """E4M3 checkpoint weight ``[N, K]`` + 128x128 block scales -> GEMM-ready MXFP8 rows
    (codes re-derived on power-of-two scales when the checkpoint scales are not)."""
    _check_gpu_tensor("weight", weight)
    _check_gpu_tensor("weight_scale", weight_scale)
    if tuple(int(b) for b in block_size) != (128, 128):
        raise ValueError(
            f"b12x block FP8 linear currently supports 128x128 weight blocks, got {block_size}")
    if weight.ndim != 2:
        raise ValueError(f"weight must have shape [N,K], got {tuple(weight.shape)}")
    out_features, in_features = (int(v) for v in weight.shape)
    _check_mxfp8_k(in_features)
    if out_features <= 0:
        raise ValueError("out_features must be positive")
    rows = pack_fp8_block_scaled_weight_mxfp8(weight.detach(), weight_scale.detach(),
                                              m=out_features, k=in_features, num_groups=1)
    return BlockFP8LinearWeight(weight=rows, in_features=in_features, out_features=out_features,
                                block_size=(128, 128))


# ----------------------------------------------------------------------------------------
# torch custom ops (names and schemas are the reference's)
# ----------------------------------------------------------------------------------------
@torch.library.custom_op("b12x::quantize_block_fp8_linear_input_mxfp8_alloc", mutates_args=())
def _quantize_input_alloc_op(source_tk: torch.Tensor, tokens: int,
                             in_features: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Fresh contiguous bases (codes, row scales, atoms) holding the quantized rows."""
    bases = empty_mxfp8_rows_bases(tokens, in_features, num_groups=1, device=source_tk.device)
    views = mxfp8_rows_from_bases(*bases, tokens, in_features, num_groups=1)
    quantize_mxfp8_rows(source_tk, views.values, views.scale_rows, views.scale_mma)
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
    tokens, in_features = (int(v) for v in source_tk.shape)
    if tokens <= 0:
        raise ValueError("tokens must be positive")
    _check_mxfp8_k(in_features)
    if out is not None:
        _check_mxfp8_rows_storage(out, m=tokens, k=in_features, num_groups=1)
        quantize_mxfp8_rows(source_tk, out.values, out.scale_rows, out.scale_mma)
        return out
    bases = torch.ops.b12x.quantize_block_fp8_linear_input_mxfp8_alloc(source_tk, tokens, in_features)
    return mxfp8_rows_from_bases(*bases, tokens, in_features, num_groups=1)


@torch.library.custom_op("b12x::block_fp8_linear_mxfp8_fused", mutates_args=())
def _block_fp8_linear_mxfp8_fused_op(source_2d: torch.Tensor, weight_values: torch.Tensor,
                                     weight_scale_rows: torch.Tensor,
                                     weight_scale_mma: torch.Tensor, in_features: int,
                                     out_features: int, expected_m: int,
                                     stream_int: int | None) -> torch.Tensor:
    del weight_scale_rows, expected_m  # the kernels pick their tile from the live shape
    tokens = int(source_2d.shape[0])
    x_q = mxfp8_rows_from_bases(
        *empty_mxfp8_rows_bases(tokens, in_features, num_groups=1, device=source_2d.device),
        tokens, in_features, num_groups=1)
    out = torch.empty((tokens, out_features, 1), dtype=source_2d.dtype, device=source_2d.device)
    return quantize_then_gemm(source_2d.contiguous(), weight_values, weight_scale_mma,
                              padded_k=in_features, out_features=out_features, x_q=x_q, out=out,
                              bias=None, stream=stream_int)


@_block_fp8_linear_mxfp8_fused_op.register_fake
def _block_fp8_linear_mxfp8_fused_fake(source_2d, weight_values, weight_scale_rows,
                                       weight_scale_mma, in_features, out_features, expected_m,
                                       stream_int) -> torch.Tensor:
    return source_2d.new_empty((source_2d.shape[0], out_features))


# ----------------------------------------------------------------------------------------
# run
# ----------------------------------------------------------------------------------------
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
        clashing = [name for name, value in (("source", source), ("packed_weight", packed_weight),
                                             ("bias", bias)) if value is not None]
        if clashing:
            raise ValueError(
                "block FP8 linear binding owns source, packed weight, scratch tensors, and bias; "
                f"do not also pass {', '.join(clashing)}")
        source, packed_weight, bias = binding.source, binding.packed_weight, binding.bias
        expected_m = binding.expected_m
        rows = binding.prechecked_rows
        if rows is not None and rows.rows.data_ptr() == source.data_ptr():
            # Validated when it was built and frozen since: quantize, multiply, done.
            output = quantize_then_gemm(rows.rows, packed_weight.weight.values,
                                        packed_weight.weight.scale_mma,
                                        padded_k=packed_weight.in_features,
                                        out_features=packed_weight.out_features, x_q=binding.x_q,
                                        out=binding.output, bias=bias, stream=stream,
                                        bias_in_place=True)
            return rows.restore(output, packed_weight.out_features)
    if source is None or packed_weight is None:
        raise TypeError("block_fp8_linear_mxfp8 requires source and packed_weight or binding")
    _check_gpu_tensor("source", source)
    if not isinstance(packed_weight, BlockFP8LinearWeight):
        raise TypeError("packed_weight must be a BlockFP8LinearWeight")
    rows = _source_rows(source, packed_weight)
    weight = packed_weight.weight

    if binding is None:
        output = torch.ops.b12x.block_fp8_linear_mxfp8_fused(
            rows.rows, weight.values, weight.scale_rows, weight.scale_mma,
            packed_weight.in_features, packed_weight.out_features,
            int(expected_m) if expected_m is not None else 0, cuda_stream_to_int(stream))
        if bias is not None:
            output = output + bias
        return rows.restore(output, packed_weight.out_features)

    _check_bound_tensors(binding.x_q, binding.output, rows, packed_weight)
    started = time.perf_counter() if _LOG_TIMING else 0.0
    output = quantize_then_gemm(rows.rows, weight.values, weight.scale_mma,
                                padded_k=packed_weight.in_features,
                                out_features=packed_weight.out_features, x_q=binding.x_q,
                                out=binding.output, bias=bias, stream=stream, bias_in_place=True)
    if _LOG_TIMING:
        elapsed_ms = (time.perf_counter() - started) * 1000.0
        if elapsed_ms >= _LOG_TIMING_FROM_MS:
            logger.warning("b12x_block_fp8_linear timing tokens=%d in=%d out=%d enqueue=%.3fms",
                           rows.tokens, rows.in_features, packed_weight.out_features, elapsed_ms)
    return rows.restore(output, packed_weight.out_features)


def prewarm_block_fp8_linear_mxfp8(packed_weight: BlockFP8LinearWeight,
                                   token_counts: Iterable[int], *,
                                   output_dtype: torch.dtype = torch.bfloat16,
                                   expected_m: int | None = None, stream: object = None) -> None:
    """Run the bound path once per planned token count (loads the library, sets kernel
    attributes, creates the per-device status word and workspaces) so later calls are capture
    safe."""
    if not isinstance(packed_weight, BlockFP8LinearWeight):
        raise TypeError("packed_weight must be a BlockFP8LinearWeight")
    if output_dtype not in _SOURCE_DTYPES:
        raise ValueError(f"output_dtype must be bf16/fp16, got {output_dtype}")
    device = packed_weight.weight.values.device
    ran = False
    with torch.inference_mode():
        for tokens in sorted({int(t) for t in token_counts if int(t) > 0}):
            plan = plan_block_fp8_linear_scratch(BlockFP8LinearScratchCaps(
                device=device, max_tokens=tokens, in_features=packed_weight.in_features,
                out_features=packed_weight.out_features, output_dtype=output_dtype))
            (spec,) = plan.scratch_specs()
            plan.bind(
                scratch=torch.empty(spec.shape, dtype=spec.dtype, device=spec.device),
                source=torch.zeros((tokens, packed_weight.in_features), dtype=output_dtype,
                                   device=device),
                packed_weight=packed_weight,
                output=empty_dense_gemm_mnl_view(tokens, packed_weight.out_features, 1,
                                                 device=device, dtype=output_dtype),
                expected_m=expected_m).run(stream=stream)
            ran = True
    if ran:
        torch.cuda.synchronize(device)


def bind_block_fp8_linear_scratch(plan: BlockFP8LinearScratchPlan, **kwargs) -> BlockFP8LinearBinding:
    """``block_fp8_linear.bind``: attach the run-time tensors and the caller's scratch to a plan.
    Only views are made (b12x/gemm/block_fp8_linear/api.py:40-44)."""
    return plan.bind(**kwargs)


__all__ = [
    "BlockFP8LinearBinding", "BlockFP8LinearScratchCaps", "BlockFP8LinearScratchPlan",
    "BlockFP8LinearWeight", "bind_block_fp8_linear_scratch", "build_block_fp8_linear_binding",
    "block_fp8_linear_mxfp8",
    "pack_block_fp8_linear_weight_mxfp8", "plan_block_fp8_linear_scratch",
    "prewarm_block_fp8_linear_mxfp8", "quantize_block_fp8_linear_input_mxfp8",
]
