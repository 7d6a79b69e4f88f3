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

from ..._lib.registry import install

install(globals(), "gemm.blockscaled")
