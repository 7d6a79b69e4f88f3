"""MXFP8 row quantizer: BF16/FP16 rows -> E4M3 values + UE8M0 scales per 32 elements.

``quantize_rows(x, values, scale_rows, scale_mma)`` writes caller-owned tensors (row-major
scales and the MMA-layout scales the block-scaled GEMM consumes). Stands in for
``b12x.quantization.mxfp8`` (b12x/quantization/mxfp8/api.py).
"""

from ..._lib.registry import install

install(globals(), "quantization.mxfp8")
