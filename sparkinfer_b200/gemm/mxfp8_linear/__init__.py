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

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="mxfp8_linear",
    group="gemm",
    api_style="oneshot",
    entry_points=("Weight", "mm", "pack_weight", "is_supported"),
    dtypes=("bf16", "fp16"),
    recipes=("mxfp8",),
    provenance=Provenance(
        repo="local-inference-lab/sparkinfer",
        commit="b12x-1.1.0",
        paths=("b12x/gemm/mxfp8_linear/api.py", "b12x/gemm/mxfp8_linear/_kernel.py"),
    ),
    test_path="tests/test_linears_gpu.py",
    since="0.1.0",
)

if TYPE_CHECKING:
    from .api import Weight, is_supported, mm, pack_weight  # noqa: F401

install_lazy_api(globals(), META)
