"""NVFP4 row quantizer: BF16 rows -> packed E2M1 values + E4M3 scales per 16 elements.

Planned lifecycle, as in ``b12x.quantization.nvfp4`` (b12x/quantization/nvfp4/api.py):

    p = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(p, device="cuda")
    nvfp4.run(plan=p, x=x, global_scale=gs, outputs=outs)   # allocation-free, capture safe

``global_scale`` is the caller's FP32 device scalar ``448 * 6 / amax``. Unlike the
reference kernel M may be any positive number of rows (decode shapes); K must be a
multiple of 64.
"""

from __future__ import annotations

from typing import TYPE_CHECKING

from ..._lib.meta import OpMeta, Provenance, install_lazy_api

META = OpMeta(
    name="nvfp4",
    group="quantization",
    api_style="planned",
    entry_points=("Outputs", "Plan", "plan", "allocate_outputs", "run", "is_supported"),
    dtypes=("bf16", "fp4_e2m1"),
    recipes=("nvfp4",),
    provenance=Provenance(
        repo="local-inference-lab/sparkinfer",
        commit="b12x-1.1.0",
        paths=("b12x/quantization/nvfp4/api.py", "b12x/quantization/nvfp4/_impl.py",
               "b12x/quantization/nvfp4/_kernel.py"),
    ),
    test_path="tests/test_quantizers_gpu.py",
    since="0.1.0",
)

if TYPE_CHECKING:
    from .api import Outputs, Plan, allocate_outputs, is_supported, plan, run  # noqa: F401

install_lazy_api(globals(), META)
