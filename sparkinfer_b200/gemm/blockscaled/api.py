"""Public surface of gemm.blockscaled (documentation lives in the op ``__init__``)."""

from __future__ import annotations

from ..._lib.dense_gemm import dense_gemm as mm
from ..._lib.dense_gemm import dense_gemm_fused_quant_a as mm_fused_quant_a
from ..._lib.dense_gemm import dense_gemm_fused_quant_a_grouped as mm_fused_quant_a_grouped
from ..._lib.dense_gemm import dense_gemm_fused_quant_a_nvfp4 as mm_fused_quant_a_nvfp4
from ..._lib.gating import default_is_supported
from . import META


def is_supported(device=None) -> bool:
    """True on a compute-capability 10.x device with the CUDA library built."""
    return default_is_supported(device, requires=META.requires)


__all__ = ["mm", "mm_fused_quant_a", "mm_fused_quant_a_grouped", "mm_fused_quant_a_nvfp4",
           "is_supported"]
