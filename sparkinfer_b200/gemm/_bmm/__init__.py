"""Home of the group-level function ``sparkinfer_b200.gemm.bmm`` (metadata here, code in
``api``), the stand-in for ``b12x.gemm.bmm`` (b12x/gemm/_bmm/api.py,
b12x/gemm/_shared/mxfp8_bmm.py).

What it computes: for every head ``h``, ``out[h] = lhs[h] @ W[h]`` with BF16 ``lhs [H, M, K]``
(at most 32 rows), BF16 ``out [H, M, N]`` owned by the caller, and ``W`` held as rowwise MXFP8:
E4M3 codes plus one E8M0 byte per 32 codes along the storage's inner axis. ``W`` may be stored
``[H, N, K]`` (``b_major="k"``) or ``[H, K, N]`` (``b_major="n"``); both are typically slices of
one larger allocation and are read in place through their strides.

One kernel launch, no scratch memory, nothing allocated. Because the kernels are built ahead
of time, ``prewarm_bmm`` has nothing to compile: it checks the weight views and runs each
requested row count once, and a row count that was never warmed can still be captured in a
CUDA graph.

    from sparkinfer_b200 import gemm

    kind = dict(a_dtype="bfloat16", b_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu",
                c_dtype="bfloat16", sf_vec_size=32, b_major="n", sf_axis="n")
    if gemm.can_implement_bmm(batch=16, max_m=8, n=512, k=192, **kind):
        gemm.bmm(q_nope, (w_codes, w_scales), absorbed, **kind)
"""

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

_REFERENCE = Provenance(
    repo="local-inference-lab/sparkinfer",
    commit="b12x-1.1.0",
    paths=("b12x/gemm/_bmm/api.py", "b12x/gemm/_shared/mxfp8_bmm.py"),
)

META = OpMeta(
    group="gemm",
    name="bmm",
    entry_points=("bmm", "prewarm_bmm", "can_implement_bmm", "is_bmm_supported"),
    api_style="oneshot",
    recipes=("mxfp8",),
    dtypes=("bf16", "fp8_e4m3"),
    provenance=_REFERENCE,
    since="0.2.0",
    test_path="tests/test_bmm_gpu.py",
    notes="dtype-dispatched batched product; one backend: BF16 activations x rowwise MXFP8",
)

install_lazy_api(globals(), META)

if TYPE_CHECKING:
    from .api import bmm, can_implement_bmm, is_bmm_supported, prewarm_bmm  # noqa: F401
