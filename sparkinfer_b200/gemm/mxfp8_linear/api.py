"""Public surface of gemm.mxfp8_linear."""

from __future__ import annotations

from ..._lib.gating import default_is_supported
from ._kernel import MXFP8LinearWeight as Weight
from ._kernel import mxfp8_linear as mm
from ._kernel import pack_mxfp8_linear_weight as pack_weight
from . import META


def is_supported(device=None) -> bool:
    return default_is_supported(device, requires=META.requires)


__all__ = ["Weight", "mm", "pack_weight", "is_supported"]
