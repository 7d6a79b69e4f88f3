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

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="tensor_fp8_linear",
    group="gemm",
    api_style="oneshot",
    entry_points=("Weight", "mm", "pack_weight", "prewarm", "is_supported"),
    dtypes=("bf16", "fp16"),
    recipes=("fp8",),
    provenance=Provenance(
        repo="local-inference-lab/sparkinfer",
        commit="b12x-1.1.0",
        paths=("b12x/gemm/tensor_fp8_linear/api.py", "b12x/gemm/tensor_fp8_linear/_kernel.py"),
    ),
    test_path="tests/test_linears_gpu.py",
    since="0.1.0",
)

if TYPE_CHECKING:
    from .api import Weight, is_supported, mm, pack_weight, prewarm  # noqa: F401

install_lazy_api(globals(), META)
