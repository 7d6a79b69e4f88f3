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

from ..._lib.registry import install

install(globals(), "gemm.bmm")
