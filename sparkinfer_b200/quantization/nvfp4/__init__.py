"""NVFP4 row quantizer: BF16 rows -> packed E2M1 values + E4M3 scales per 16 elements.

Planned lifecycle, as in ``b12x.quantization.nvfp4`` (b12x/quantization/nvfp4/api.py):

    p = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(p, device="cuda")
    nvfp4.run(plan=p, x=x, global_scale=gs, outputs=outs)   # allocation-free, capture safe

``global_scale`` is the caller's FP32 device scalar ``448 * 6 / amax``. Unlike the
reference kernel M may be any positive number of rows (decode shapes); K must be a
multiple of 64.
"""

from ..._lib.registry import install

install(globals(), "quantization.nvfp4")
