"""plan / allocate_outputs / run of ``quantization.nvfp4`` (the reference's
b12x/quantization/nvfp4/api.py:22-58): a plan is a validated ``(m, k)`` with its launcher."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from . import _impl


@dataclass(frozen=True)
class Plan:
    """Rows, columns and the launcher :func:`plan` built for them."""

    m: int
    k: int
    launch: Callable[..., None]


def plan(m: int, k: int) -> Plan:
    """Host-side only: checks the shape and binds the kernel launcher to it."""
    rows, cols = int(m), int(k)
    return Plan(m=rows, k=cols, launch=_impl.compile_bf16_to_fp4_tma(rows, cols))


def allocate_outputs(plan: Plan, *, device: torch.device | str = "cuda") -> _impl.BF16ToFP4TMAOutputs:
    """Packed FP4 codes and MMA-layout scale bytes sized for ``plan``."""
    return _impl.allocate_bf16_to_fp4_tma_outputs(plan.m, plan.k, device=torch.device(device))


def run(*, plan: Plan, x: torch.Tensor, global_scale: torch.Tensor,
        outputs: _impl.BF16ToFP4TMAOutputs) -> None:
    """One kernel launch on the current stream; allocates nothing, so it can be captured."""
    plan.launch(x, global_scale, outputs.packed_a_flat, outputs.scale_flat)
