"""Host side of the NVFP4 row quantizer: shape plans, output storage, launch validation.

Counterpart of b12x/quantization/nvfp4/_impl.py:32-224. The reference compiles one kernel
per (M, K) and requires both to be multiples of 128; the ahead-of-time kernel here takes
any M >= 1 (it covers the padded scale rows itself) and K % 64 == 0.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from ..._lib import launch as _launch
from ..._lib.layout import align_up, convert_sf_to_mma_layout

_SF_VEC_SIZE = 16
_K_ALIGN = 64


def _validate_shape(m: int, k: int) -> None:
    if m <= 0 or k <= 0:
        raise ValueError(f"M and K must be positive, got M={m}, K={k}")
    if k % _K_ALIGN != 0:
        raise ValueError(f"K must be a multiple of {_K_ALIGN}, got K={k}")


def _validate_launch_tensor(tensor: torch.Tensor, *, name: str, dtype: torch.dtype,
                            shape: tuple[int, ...], device: torch.device) -> None:
    if tensor.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {tensor.dtype}")
    if tuple(tensor.shape) != shape:
        raise ValueError(f"{name} must have shape {shape}, got {tuple(tensor.shape)}")
    if tensor.device != device or tensor.device.type != "cuda":
        raise ValueError(f"{name} must be on {device}, got {tensor.device}")
    if not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _byte_interval(tensor: torch.Tensor) -> tuple[int, int]:
    begin = tensor.untyped_storage().data_ptr() + tensor.storage_offset() * tensor.element_size()
    return begin, begin + tensor.numel() * tensor.element_size()


def _overlaps(lhs: torch.Tensor, rhs: torch.Tensor) -> bool:
    a0, a1 = _byte_interval(lhs)
    b0, b1 = _byte_interval(rhs)
    return a0 < b1 and b0 < a1


def scale_storage_numel(m: int, k: int) -> int:
    return align_up(m, 128) * align_up(k // _SF_VEC_SIZE, 4)


@dataclass
class BF16ToFP4TMAOutputs:
    """Packed codes ``(1, M, K/2)`` u8 and flat MMA-layout scale bytes."""

    packed_a_storage: torch.Tensor
    scale_storage: torch.Tensor

    @property
    def packed_a_flat(self) -> torch.Tensor:
        return self.packed_a_storage.view(-1)

    @property
    def scale_flat(self) -> torch.Tensor:
        return self.scale_storage.view(-1)

    @property
    def packed_a_view(self) -> torch.Tensor:
        """``[M, K/2, 1]`` view, the ``A`` operand ``gemm.blockscaled.mm`` expects."""
        return self.packed_a_storage.permute(1, 2, 0)

    def scale_mma_view(self, m: int, k: int) -> torch.Tensor:
        """6-D ``(32, 4, m_tiles, 4, k_tiles, 1)`` view of the scale bytes."""
        return convert_sf_to_mma_layout(self.scale_storage, m, k, 1, _SF_VEC_SIZE)


def allocate_bf16_to_fp4_tma_outputs(m: int, k: int, *,
                                     device: torch.device = torch.device("cuda")) -> BF16ToFP4TMAOutputs:
    _validate_shape(m, k)
    return BF16ToFP4TMAOutputs(
        packed_a_storage=torch.zeros(1, m, k // 2, dtype=torch.uint8, device=device),
        scale_storage=torch.zeros(scale_storage_numel(m, k), dtype=torch.uint8, device=device),
    )


def compile_bf16_to_fp4_tma(m: int, k: int) -> Callable[..., None]:
    """Return ``launch(bf16_input, global_scale, packed_a_flat, scale_flat)`` for (m, k).

    Nothing is compiled at run time; the callable validates its arguments like the
    reference's launcher (dtype, shape, device, contiguity, no overlap) and enqueues the
    kernel on torch's current stream.
    """
    _validate_shape(m, k)
    scale_numel = scale_storage_numel(m, k)

    def launch(bf16_input, global_scale, packed_a_flat, scale_flat):
        device = bf16_input.device
        _validate_launch_tensor(bf16_input, name="bf16_input", dtype=torch.bfloat16,
                                shape=(m, k), device=device)
        _validate_launch_tensor(global_scale, name="global_scale", dtype=torch.float32,
                                shape=(1,), device=device)
        _validate_launch_tensor(packed_a_flat, name="packed_a_flat", dtype=torch.uint8,
                                shape=(m * k // 2,), device=device)
        _validate_launch_tensor(scale_flat, name="scale_flat", dtype=torch.uint8,
                                shape=(scale_numel,), device=device)
        if _overlaps(packed_a_flat, scale_flat):
            raise ValueError("packed_a_flat and scale_flat must not overlap")
        if _overlaps(bf16_input, packed_a_flat) or _overlaps(bf16_input, scale_flat):
            raise ValueError("bf16_input must not overlap either output")
        if _overlaps(global_scale, packed_a_flat) or _overlaps(global_scale, scale_flat):
            raise ValueError("global_scale must not overlap either output")
        _launch.quantize_nvfp4_rows(bf16_input, global_scale, packed_a_flat, scale_flat)

    return launch


__all__ = ["BF16ToFP4TMAOutputs", "allocate_bf16_to_fp4_tma_outputs", "compile_bf16_to_fp4_tma",
           "scale_storage_numel"]
