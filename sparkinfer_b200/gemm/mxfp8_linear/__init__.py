"""ModelOpt MXFP8 linear for B200 (one-shot).

``pack_weight`` converts a ModelOpt MXFP8 checkpoint weight (``[N, K]`` E4M3 + ``[N, K/32]``
UE8M0) into the GEMM layout once, padding K to a multiple of 128; ``mm`` quantizes the
BF16/FP16 input rows and runs the MXFP8 GEMM through an opaque torch custom op. Stands in
for ``b12x.gemm.mxfp8_linear`` (b12x/gemm/mxfp8_linear/api.py).

Example:
    from sparkinfer_b200.gemm import mxfp8_linear

    weight = mxfp8_linear.pack_weight(w_mxfp8, w_scale)   # one-time
    out = mxfp8_linear.mm(x, weight, expected_m=x.shape[0])
"""

from ..._lib.registry import install

install(globals(), "gemm.mxfp8_linear")
