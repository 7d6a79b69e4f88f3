"""MXFP8 row quantizer: BF16/FP16 rows -> E4M3 values + UE8M0 scales per 32 elements.

``quantize_rows(x, values, scale_rows, scale_mma)`` writes caller-owned tensors (row-major
scales and the MMA-layout scales the block-scaled GEMM consumes). Stands in for
``b12x.quantization.mxfp8`` (b12x/quantization/mxfp8/api.py).
"""

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="mxfp8",
    group="quantization",
    api_style="oneshot",
    entry_points=("quantize_rows", "is_supported"),
    dtypes=("bf16", "fp16", "fp8_e4m3"),
    recipes=("mxfp8",),
    provenance=Provenance(
        repo="local-inference-lab/sparkinfer",
        commit="b12x-1.1.0",
        paths=("b12x/quantization/mxfp8/api.py", "b12x/_lib/quant/mxfp8_rows.py"),
    ),
    test_path="tests/test_quantizers_gpu.py",
    since="0.1.0",
)

if TYPE_CHECKING:
    from .api import is_supported, quantize_rows  # noqa: F401

install_lazy_api(globals(), META)
