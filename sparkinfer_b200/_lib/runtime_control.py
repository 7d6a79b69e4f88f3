"""Kernel-resolution freeze controls, mirroring b12x/_lib/runtime_control.py:9-65.

The reference JIT-compiles kernels and lets a serving stack forbid new compilations after
warm-up. Here every kernel is compiled ahead of time, so nothing is ever resolved at run
time; the switches are kept so callers written against the reference keep working, and
:func:`raise_if_kernel_resolution_frozen` still fails closed for code that asks.
"""

from __future__ import annotations

from threading import Lock


class KernelResolutionFrozenError(RuntimeError):
    """Raised when a new kernel would have to be resolved after the freeze."""


_LOCK = Lock()
_frozen = False
_reason: str | None = None


def freeze_kernel_resolution(reason: str | None = None) -> None:
    global _frozen, _reason
    with _LOCK:
        _frozen = True
        _reason = reason


def unfreeze_kernel_resolution() -> None:
    global _frozen, _reason
    with _LOCK:
        _frozen = False
        _reason = None


def kernel_resolution_frozen() -> bool:
    with _LOCK:
        return _frozen


freeze_compilation = freeze_kernel_resolution
unfreeze_compilation = unfreeze_kernel_resolution
compilation_frozen = kernel_resolution_frozen


def raise_if_kernel_resolution_frozen(kind: str, *, target: object | None = None,
                                      cache_key: object | None = None) -> None:
    with _LOCK:
        frozen, reason = _frozen, _reason
    if not frozen:
        return
    parts = [f"b12x kernel resolution is frozen; refusing {kind}"]
    if target is not None:
        parts.append(f"target={getattr(target, '__qualname__', type(target).__qualname__)}")
    if cache_key is not None:
        parts.append(f"key={cache_key!r:.120}")
    if reason is not None:
        parts.append(f"reason={reason}")
    raise KernelResolutionFrozenError("; ".join(parts))


__all__ = [
    "KernelResolutionFrozenError", "freeze_kernel_resolution", "unfreeze_kernel_resolution",
    "kernel_resolution_frozen", "freeze_compilation", "unfreeze_compilation",
    "compilation_frozen", "raise_if_kernel_resolution_frozen",
]
