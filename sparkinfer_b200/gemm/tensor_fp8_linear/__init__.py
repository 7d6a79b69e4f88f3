"""Static per-tensor FP8 linear for B200 (one-shot).

Both operands are E4M3 with one FP32 dequantization scale for the whole product
(``output_scale = activation_scale * weight_scale``). The MXFP8 GEMM computes it with every
block scale at 2^0 and ``alpha = output_scale``. Stands in for ``b12x.gemm.tensor_fp8_linear``
(b12x/gemm/tensor_fp8_linear/api.py).

Example:
    from sparkinfer_b200.gemm import tensor_fp8_linear

    weight = tensor_fp8_linear.pack_weight(w_e4m3, output_scale)   # one-time
    out = tensor_fp8_linear.mm(x_e4m3, weight, out_dtype=torch.bfloat16)
"""

from ..._lib.registry import install

install(globals(), "gemm.tensor_fp8_linear")
