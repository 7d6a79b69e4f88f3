"""Capability gating, the sm_100 counterpart of b12x/_lib/gating.py:28-95.

The reference gates every op on compute capability 12.x plus its JIT toolchain. These ops
need a compute-capability 10.x device (B200) and the in-tree CUDA library, nothing else.
"""

from __future__ import annotations


def get_compute_capability(device=None) -> tuple[int, int] | None:
    import torch

    if not torch.cuda.is_available():
        return None
    dev = torch.device(device) if device is not None else torch.device("cuda")
    if dev.type != "cuda":
        return None
    return torch.cuda.get_device_capability(dev)


def is_b200(device=None) -> bool:
    """True when the device is datacenter Blackwell (compute capability 10.x)."""
    cap = get_compute_capability(device)
    return cap is not None and cap[0] == 10


def has_native_library() -> bool:
    from .. import _native

    return _native.library_path().exists()


def _requirement_met(requirement: str) -> bool:
    if requirement == "multi_gpu":
        import torch

        return torch.cuda.is_available() and torch.cuda.device_count() >= 2
    raise ValueError(f"unknown op requirement {requirement!r}")


def default_is_supported(device=None, *, requires: tuple[str, ...] = ()) -> bool:
    """The ``is_supported`` of every op without extra constraints."""
    if not is_b200(device) or not has_native_library():
        return False
    return all(_requirement_met(req) for req in requires)


__all__ = ["get_compute_capability", "is_b200", "has_native_library", "default_is_supported"]
