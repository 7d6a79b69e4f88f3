"""The names the reference keeps in ``b12x/_lib/meta.py`` (:28-88), re-exported from the
package's op table (``registry``), where the dataclasses and the lazy resolution live."""

from __future__ import annotations

from .registry import OpMeta, Provenance, install


def install_lazy_api(module_globals: dict, meta: OpMeta) -> None:
    """Reference-style spelling of ``registry.install`` for an op that is in the table."""
    install(module_globals, meta.qualname)


__all__ = ["OpMeta", "Provenance", "install_lazy_api"]
