"""Block-FP8 linear (128x128 FP32 weight block scales) for B200, planned lifecycle.

``pack_weight`` turns a DeepSeek-style checkpoint weight into MXFP8 rows once;
``plan(Caps)`` sizes one caller-owned scratch buffer; ``bind`` carves views out of it;
``run(binding=...)`` quantizes the activations and runs the MXFP8 GEMM without allocating.
Stands in for ``b12x.gemm.block_fp8_linear`` (b12x/gemm/block_fp8_linear/api.py).

Example:
    from sparkinfer_b200.gemm import block_fp8_linear as bfl

    weight = bfl.pack_weight(w_fp8, w_scale_inv)                       # one-time
    plan = bfl.plan(bfl.Caps(device="cuda", max_tokens=T, in_features=K, out_features=N))
    spec = plan.scratch_specs()[0]
    scratch = torch.empty(spec.shape, dtype=spec.dtype, device=spec.device)
    binding = bfl.bind(plan, scratch=scratch, source=x, packed_weight=weight, output=out)
    y = bfl.run(binding=binding)
"""

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="block_fp8_linear",
    group="gemm",
    api_style="planned",
    entry_points=("Caps", "Plan", "Binding", "Weight", "plan", "bind", "run", "pack_weight",
                  "quantize_input", "prewarm", "is_supported"),
    dtypes=("bf16", "fp16", "fp8_e4m3"),
    recipes=("block_fp8", "mxfp8"),
    provenance=Provenance(
        repo="local-inference-lab/sparkinfer",
        commit="b12x-1.1.0",
        paths=("b12x/gemm/block_fp8_linear/api.py", "b12x/gemm/_shared/block_fp8.py"),
    ),
    test_path="tests/test_linears_gpu.py",
    since="0.1.0",
)

if TYPE_CHECKING:
    from .api import (  # noqa: F401
        Binding, Caps, Plan, Weight, bind, is_supported, pack_weight, plan, prewarm,
        quantize_input, run,
    )

install_lazy_api(globals(), META)
