"""Scratch memory the caller owns. A planned op states what it needs as
:class:`ScratchBufferSpec` records (today always one flat ``uint8`` buffer); the caller
allocates, and at bind time hands the memory back as the tensor itself, as ``{name: tensor}``
or as a one-element list. The contract, the names and the error texts are those of
b12x/_lib/scratch.py:11-78."""

from __future__ import annotations

import math
from collections.abc import Mapping, Sequence
from dataclasses import dataclass

import torch


@dataclass(frozen=True, kw_only=True)
class ScratchBufferSpec:
    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype
    device: torch.device

    @property
    def nbytes(self) -> int:
        return math.prod(int(extent) for extent in self.shape) * self.dtype.itemsize


def scratch_buffer_spec(name: str, *, nbytes: int, device: torch.device) -> ScratchBufferSpec:
    """A flat byte buffer of at least one byte."""
    return ScratchBufferSpec(name=name, dtype=torch.uint8, device=device, shape=(max(1, int(nbytes)),))


def _unwrap(container, wanted: str) -> torch.Tensor:
    """The tensor inside whatever the caller passed as scratch."""
    if isinstance(container, torch.Tensor):
        return container
    if isinstance(container, Mapping):
        try:
            return container[wanted]
        except KeyError:
            raise KeyError(f"scratch mapping is missing {wanted!r}") from None
    if isinstance(container, Sequence):
        if len(container) == 1:
            return container[0]
        raise ValueError(f"scratch sequence must contain exactly one tensor, got {len(container)}")
    raise TypeError(f"unsupported scratch container {type(container).__name__}")


def scratch_tensor(scratch, specs: tuple[ScratchBufferSpec, ...], *, owner: str) -> torch.Tensor:
    """The caller's scratch as a flat tensor, after checking it against the plan's one spec."""
    if len(specs) != 1:
        raise RuntimeError(f"{owner} scratch plans currently expect exactly one scratch buffer")
    (spec,) = specs
    buffer = _unwrap(scratch, spec.name)
    need, have = int(spec.shape[0]), int(buffer.numel())
    problems = (
        (buffer.dtype != spec.dtype, TypeError,
         f"{spec.name} scratch must have dtype {spec.dtype}, got {buffer.dtype}"),
        (buffer.device != spec.device, ValueError,
         f"{spec.name} scratch device {buffer.device} does not match {spec.device}"),
        (have < need, ValueError, f"{spec.name} scratch has {have} bytes, requires {need}"),
        (not buffer.is_contiguous(), ValueError, f"{spec.name} scratch must be contiguous"),
    )
    for failed, error, text in problems:
        if failed:
            raise error(text)
    return buffer.reshape(-1)


__all__ = ["ScratchBufferSpec", "scratch_buffer_spec", "scratch_tensor"]
