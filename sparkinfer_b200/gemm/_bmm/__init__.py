"""Private implementation package of :func:`sparkinfer_b200.gemm.bmm`.

``bmm`` dispatches from dtype and layout metadata; the one specialization multiplies BF16
activations ``[B, M, K]`` (``M <= 32``) by a rowwise-MXFP8 right-hand side and writes BF16
``[B, M, N]`` into a caller-owned tensor. The right-hand side is a ``(values, scales)`` pair of
zero-copy views, K-major (``[B, N, K]`` / ``[B, N, K/32]``) or N-major (``[B, K, N]`` /
``[B, K, N/32]``). Stands in for ``b12x.gemm.bmm`` (b12x/gemm/_bmm/api.py,
b12x/gemm/_shared/mxfp8_bmm.py).

The launch takes no workspace and allocates nothing. The kernels are compiled ahead of time,
so ``prewarm_bmm`` only validates the operands and launches each declared ``M`` once; there is
no compile miss under CUDA-graph capture.

Example::

    from sparkinfer_b200 import gemm

    spec = dict(a_dtype="bfloat16", b_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu",
                c_dtype="bfloat16", sf_vec_size=32, b_major="k", sf_axis="k")
    gemm.prewarm_bmm((b_values, b_scales), (1, 4, 8), **spec)
    gemm.bmm(lhs, (b_values, b_scales), out, **spec)
"""

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="bmm",
    group="gemm",
    api_style="oneshot",
    entry_points=("bmm", "prewarm_bmm", "can_implement_bmm", "is_bmm_supported"),
    dtypes=("bf16", "fp8_e4m3"),
    recipes=("mxfp8",),
    provenance=Provenance(
        repo="local-inference-lab/sparkinfer",
        commit="b12x-1.1.0",
        paths=("b12x/gemm/_bmm/api.py", "b12x/gemm/_shared/mxfp8_bmm.py"),
    ),
    test_path="tests/test_bmm_gpu.py",
    since="0.2.0",
    notes="Generic BMM API with a BF16 x rowwise-MXFP8 backend.",
)

if TYPE_CHECKING:
    from .api import bmm, can_implement_bmm, is_bmm_supported, prewarm_bmm  # noqa: F401

install_lazy_api(globals(), META)
