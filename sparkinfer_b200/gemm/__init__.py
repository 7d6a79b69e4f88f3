"""The ``gemm`` group.

Op packages: ``blockscaled``, ``block_fp8_linear``, ``mxfp8_linear``, ``tensor_fp8_linear``.
Plain functions of the group: ``mm`` (what ``blockscaled.mm`` is), ``bmm`` and its helpers
``prewarm_bmm`` / ``can_implement_bmm`` / ``is_bmm_supported`` (a batched BF16 x MXFP8 product;
implementation under the private package ``_bmm`` because a function and a child package
cannot share one name). The group's layout follows b12x/gemm/__init__.py:18-50. Nothing is
imported until a name is first used, so ``import sparkinfer_b200.gemm`` pulls in neither torch
nor the CUDA library.
"""

from __future__ import annotations

from importlib import import_module

_PACKAGES = frozenset({"blockscaled", "block_fp8_linear", "mxfp8_linear", "tensor_fp8_linear"})

# public name -> "module:attribute" (module relative to this package)
_ALIASES = {
    "mm": ".._lib.dense_gemm:dense_gemm",
    **{name: f"._bmm.api:{name}"
       for name in ("bmm", "prewarm_bmm", "can_implement_bmm", "is_bmm_supported")},
}

__all__ = sorted(_PACKAGES | set(_ALIASES))


def __getattr__(name: str):
    if name in _PACKAGES:
        found = import_module(f"{__name__}.{name}")
    elif name in _ALIASES:
        module, _, attribute = _ALIASES[name].partition(":")
        found = getattr(import_module(module, __name__), attribute)
    else:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    globals()[name] = found   # next access skips this hook
    return found


def __dir__():
    return list(__all__)
