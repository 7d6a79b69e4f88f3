"""B200-native implementation of the b12x block-scaled GEMM hot path.

Ops live at ``sparkinfer_b200.<group>.<op>`` with the reference's grammar
(b12x/__init__.py:7-11, 41-62): planned ops ``Caps -> plan() -> bind() -> run()``, one-shot
ops as plain functions. Importing this package (or an op package) imports neither torch nor
the CUDA library; entry points resolve lazily on first attribute access.

    from sparkinfer_b200.gemm import blockscaled, mxfp8_linear, block_fp8_linear
    from sparkinfer_b200.quantization import nvfp4, mxfp8

:func:`install_as_b12x` additionally exposes the package under the name ``b12x`` so code
written against the reference's import paths for these ops runs unchanged.
"""

from __future__ import annotations

import importlib
import sys
from typing import Any

from ._lib import registry as _registry
from ._lib.registry import OpMeta, Provenance
from ._lib.runtime_control import (
    KernelResolutionFrozenError,
    compilation_frozen,
    freeze_compilation,
    freeze_kernel_resolution,
    kernel_resolution_frozen,
    unfreeze_compilation,
    unfreeze_kernel_resolution,
)

__version__ = "0.1.0"

# group -> op names, read off the op table; one directory per op, checked by
# tests/test_registry.py.
_OPS: dict[str, tuple[str, ...]] = {}
for _qualname in _registry.OPS:
    _group, _, _name = _qualname.partition(".")
    _OPS[_group] = (*_OPS.get(_group, ()), _name)
del _qualname, _group, _name

# A group-level function cannot share its name with a child module: ``gemm.bmm`` is a function,
# its metadata and implementation live in a private package (b12x/__init__.py:64-72).
_OP_MODULE_OVERRIDES: dict[str, str] = {"gemm.bmm": "gemm._bmm"}


def _op_module(group: str, name: str):
    path = _OP_MODULE_OVERRIDES.get(f"{group}.{name}", f"{group}.{name}")
    return importlib.import_module(f"{__name__}.{path}")


def list_ops() -> list[OpMeta]:
    """META of every op, in registry order."""
    return [_op_module(group, name).META for group, names in _OPS.items() for name in names]


def find_op(qualname: str) -> OpMeta:
    """META of ``"group.name"``; ``KeyError`` when unknown."""
    group, _, name = qualname.partition(".")
    if name not in _OPS.get(group, ()):
        raise KeyError(f"unknown op {qualname!r}")
    return _op_module(group, name).META


def clear_all_caches() -> None:
    """Drop host-side caches (alpha scalars, unit-scale tensors). Kernels are compiled ahead of
    time, so there is no compile cache to clear. The per-device status words and the decode
    workspaces are deliberately kept: a captured CUDA graph may hold their addresses."""
    dense = sys.modules.get(f"{__name__}._lib.dense_gemm")
    if dense is not None:
        dense._ALPHA_ONE_CACHE.clear()
        dense._UNIT_SCALE_CACHE.clear()


def install_as_b12x() -> None:
    """Alias this package (and its sub-packages as they load) to the name ``b12x``."""
    import importlib.abc
    import importlib.util

    if isinstance(sys.modules.get("b12x"), type(sys)) and sys.modules["b12x"] is not sys.modules[__name__]:
        raise RuntimeError("a different 'b12x' package is already imported")
    sys.modules["b12x"] = sys.modules[__name__]

    class _Alias(importlib.abc.MetaPathFinder, importlib.abc.Loader):
        def find_spec(self, fullname, path=None, target=None):
            if fullname == "b12x" or fullname.startswith("b12x."):
                real = __name__ + fullname[len("b12x"):]
                try:
                    module = importlib.import_module(real)
                except ImportError:
                    return None
                sys.modules[fullname] = module
                return importlib.util.spec_from_loader(fullname, self, origin=real)
            return None

        def create_module(self, spec):
            return sys.modules[spec.name]

        def exec_module(self, module):
            return None

    if not any(type(f).__name__ == "_Alias" for f in sys.meta_path):
        sys.meta_path.insert(0, _Alias())


__all__ = [
    "OpMeta", "Provenance", "list_ops", "find_op", "clear_all_caches", "install_as_b12x",
    "KernelResolutionFrozenError", "freeze_kernel_resolution", "unfreeze_kernel_resolution",
    "kernel_resolution_frozen", "freeze_compilation", "unfreeze_compilation",
    "compilation_frozen", "ScratchBufferSpec",
]


def __getattr__(name: str) -> Any:
    if name == "ScratchBufferSpec":  # needs torch; resolved lazily
        from ._lib.scratch import ScratchBufferSpec

        return ScratchBufferSpec
    if name in _OPS:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
