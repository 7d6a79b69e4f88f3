"""Public surface of quantization.nvfp4."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from ..._lib.gating import default_is_supported
from ._impl import BF16ToFP4TMAOutputs as Outputs
from ._impl import allocate_bf16_to_fp4_tma_outputs as _allocate
from ._impl import compile_bf16_to_fp4_tma as _compile
from . import META


@dataclass(frozen=True)
class Plan:
    """An (m, k) shape bound to its launcher; produced by :func:`plan`."""

    m: int
    k: int
    launch: Callable[..., None]


def plan(m: int, k: int) -> Plan:
    """Validate (m, k) and build its launcher; host-side only."""
    return Plan(m=int(m), k=int(k), launch=_compile(int(m), int(k)))


def allocate_outputs(plan: Plan, *, device: torch.device | str = "cuda") -> Outputs:
    """Allocate the packed-FP4 + MMA-layout-scale output pair for a plan."""
    return _allocate(plan.m, plan.k, device=torch.device(device))


def run(*, plan: Plan, x: torch.Tensor, global_scale: torch.Tensor, outputs: Outputs) -> None:
    """Quantize ``x`` into ``outputs`` (allocation-free, CUDA-graph-capture safe)."""
    plan.launch(x, global_scale, outputs.packed_a_flat, outputs.scale_flat)


def is_supported(device=None) -> bool:
    return default_is_supported(device, requires=META.requires)


__all__ = ["Outputs", "Plan", "plan", "allocate_outputs", "run", "is_supported"]
