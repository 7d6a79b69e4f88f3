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

from ..._lib.registry import install

install(globals(), "gemm.block_fp8_linear")
