"""Op metadata contract, mirroring b12x/_lib/meta.py:28-88.

Each op package's ``__init__`` holds a docstring, an :class:`OpMeta` named ``META`` and one
call to :func:`install_lazy_api`; its entry points resolve from the sibling ``api`` module
on first attribute access, so importing the package does not import torch, load the CUDA
library or register torch custom ops. This module is stdlib-only for the same reason.
"""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any, Literal


@dataclass(frozen=True, kw_only=True)
class Provenance:
    """Which reference sources an op stands in for."""

    repo: str
    commit: str
    paths: tuple[str, ...]


@dataclass(frozen=True, kw_only=True)
class OpMeta:
    """Machine-readable description of one op.

    ``api_style``: ``planned`` = ``Caps -> plan() -> bind() -> run()`` (plan may allocate,
    bind only creates views, run is CUDA-graph-capture safe); ``oneshot`` = plain functions;
    ``stateful`` = long-lived instances.
    """

    name: str
    group: str
    api_style: Literal["planned", "oneshot", "stateful"]
    entry_points: tuple[str, ...]
    archs: tuple[str, ...] = ("sm100a",)
    dtypes: tuple[str, ...] = ()
    recipes: tuple[str, ...] = ()
    requires: tuple[str, ...] = ()
    status: Literal["experimental"] = "experimental"
    provenance: Provenance = field(
        default_factory=lambda: Provenance(repo="", commit="", paths=())
    )
    test_path: str = ""
    since: str = ""
    notes: str = ""

    @property
    def qualname(self) -> str:
        return f"{self.group}.{self.name}"


def install_lazy_api(module_globals: dict[str, Any], meta: OpMeta) -> None:
    """Give an op module a PEP 562 ``__getattr__`` that pulls entry points from ``.api``."""
    module_name = module_globals["__name__"]

    def __getattr__(name: str) -> Any:
        if name in meta.entry_points:
            value = getattr(importlib.import_module(".api", module_name), name)
            module_globals[name] = value
            return value
        raise AttributeError(f"module {module_name!r} has no attribute {name!r}")

    def __dir__() -> list[str]:
        return sorted([*meta.entry_points, "META"])

    module_globals["__getattr__"] = __getattr__
    module_globals["__dir__"] = __dir__
    module_globals["__all__"] = [*meta.entry_points, "META"]


__all__ = ["OpMeta", "Provenance", "install_lazy_api"]
