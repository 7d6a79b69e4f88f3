"""Public surface of quantization.mxfp8."""

from __future__ import annotations

from ..._lib.gating import default_is_supported
from ..._lib.mxfp8_rows import quantize_mxfp8_rows as quantize_rows
from . import META


def is_supported(device=None) -> bool:
    return default_is_supported(device, requires=META.requires)


__all__ = ["quantize_rows", "is_supported"]
