"""Dense block-scaled GEMM for B200: ``C = (A.SFA) @ (B.SFB)^T``.

One-shot functional op over the sm_100a tcgen05 engine (TMEM accumulators, block-scaled
MMA). Recipes: NVFP4 (E2M1 values, E4M3 scales per 16) and MXFP8 (E4M3 values, E8M0 scales
per 32); with ``block_fp8=True`` E4M3 values with compact FP32 scales (1x128 / 128x128).
Stands in for ``b12x.gemm.blockscaled`` (b12x/gemm/blockscaled/__init__.py).

Example:
    from sparkinfer_b200.gemm import blockscaled

    out = blockscaled.mm(
        (a_fp4, a_sf), (b_fp4, b_sf),
        ab_dtype="float4_e2m1fn", sf_dtype="float8_e4m3fn", sf_vec_size=16,
        c_dtype="bfloat16", alpha=alpha, expected_m=m,
    )
"""

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="blockscaled",
    group="gemm",
    api_style="oneshot",
    entry_points=("mm", "mm_fused_quant_a", "mm_fused_quant_a_grouped", "mm_fused_quant_a_nvfp4",
                  "is_supported"),
    dtypes=("bf16", "fp16", "fp32", "fp8_e4m3", "fp4_e2m1"),
    recipes=("nvfp4", "mxfp8", "block_fp8"),
    provenance=Provenance(
        repo="local-inference-lab/sparkinfer",
        commit="b12x-1.1.0",
        paths=("b12x/gemm/blockscaled/api.py", "b12x/_lib/dense_gemm.py"),
    ),
    test_path="tests/test_gemm_blockscaled_gpu.py",
    since="0.1.0",
)

if TYPE_CHECKING:  # static analysis only; runtime resolution is lazy
    from .api import (is_supported, mm, mm_fused_quant_a, mm_fused_quant_a_grouped,  # noqa: F401
                      mm_fused_quant_a_nvfp4)

install_lazy_api(globals(), META)
