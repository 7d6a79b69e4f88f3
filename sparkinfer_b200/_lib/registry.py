"""One table for every op of the package: its metadata and where each public name lives.

An op package (``sparkinfer_b200.<group>.<op>``) is a docstring plus one call,
``install(globals(), "<group>.<op>")``. That call gives the package its ``META`` and a PEP 562
``__getattr__`` which resolves a public name from this table the first time it is used, so
importing an op package imports neither torch nor the CUDA library and registers no torch
custom op. The metadata fields are the reference's (b12x/_lib/meta.py:28-88) so that tooling
written against ``b12x.list_ops()`` reads the same attributes; this module is stdlib-only.

A target is ``"relative.module:attribute"`` (relative to the op package) or ``SUPPORTED``, the
default capability probe (compute capability 10.x and the in-tree library present).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from importlib import import_module
from typing import Any, Literal

SUPPORTED = "@supported"


@dataclass(frozen=True, kw_only=True)
class Provenance:
    """Which reference sources an op stands in for."""

    repo: str
    commit: str
    paths: tuple[str, ...]


@dataclass(frozen=True, kw_only=True)
class OpMeta:
    """Machine-readable description of one op. ``api_style``: ``planned`` means
    ``Caps -> plan() -> bind() -> run()`` (plan may allocate, bind only makes views, run can be
    captured in a CUDA graph); ``oneshot`` means plain functions; ``stateful`` long-lived objects."""

    name: str
    group: str
    api_style: Literal["planned", "oneshot", "stateful"]
    entry_points: tuple[str, ...]
    archs: tuple[str, ...] = ("sm100a",)
    dtypes: tuple[str, ...] = ()
    recipes: tuple[str, ...] = ()
    requires: tuple[str, ...] = ()
    status: Literal["experimental"] = "experimental"
    provenance: Provenance = field(default_factory=lambda: Provenance(repo="", commit="", paths=()))
    test_path: str = ""
    since: str = ""
    notes: str = ""

    @property
    def qualname(self) -> str:
        return f"{self.group}.{self.name}"


def _op(qualname: str, style: str, exports: dict[str, str], *, dtypes, recipes, stands_in_for,
        tested_by: str, since: str = "0.1.0", notes: str = "") -> tuple[OpMeta, dict[str, str]]:
    group, _, name = qualname.partition(".")
    meta = OpMeta(
        name=name, group=group, api_style=style, entry_points=tuple(exports), dtypes=tuple(dtypes),
        recipes=tuple(recipes), test_path=tested_by, since=since, notes=notes,
        provenance=Provenance(repo="local-inference-lab/sparkinfer", commit="b12x-1.1.0",
                              paths=tuple(stands_in_for)))
    return meta, exports


_DENSE = "..._lib.dense_gemm"
_BLOCK = ".._shared.block_fp8"

OPS: dict[str, tuple[OpMeta, dict[str, str]]] = dict((
    ("gemm.blockscaled", _op(
        "gemm.blockscaled", "oneshot",
        {"mm": f"{_DENSE}:dense_gemm",
         "mm_fused_quant_a": f"{_DENSE}:dense_gemm_fused_quant_a",
         "mm_fused_quant_a_grouped": f"{_DENSE}:dense_gemm_fused_quant_a_grouped",
         "mm_fused_quant_a_nvfp4": f"{_DENSE}:dense_gemm_fused_quant_a_nvfp4",
         "is_supported": SUPPORTED},
        dtypes=("bf16", "fp16", "fp32", "fp8_e4m3", "fp4_e2m1"),
        recipes=("nvfp4", "mxfp4", "mxfp8", "block_fp8"),
        stands_in_for=("b12x/gemm/blockscaled/api.py", "b12x/_lib/dense_gemm.py"),
        tested_by="tests/test_gemm_blockscaled_gpu.py")),
    ("gemm.mxfp8_linear", _op(
        "gemm.mxfp8_linear", "oneshot",
        {"Weight": "._kernel:MXFP8LinearWeight", "mm": "._kernel:mxfp8_linear",
         "pack_weight": "._kernel:pack_mxfp8_linear_weight", "is_supported": SUPPORTED},
        dtypes=("bf16", "fp16"), recipes=("mxfp8",),
        stands_in_for=("b12x/gemm/mxfp8_linear/api.py", "b12x/gemm/mxfp8_linear/_kernel.py"),
        tested_by="tests/test_linears_gpu.py")),
    ("gemm.block_fp8_linear", _op(
        "gemm.block_fp8_linear", "planned",
        {"Caps": f"{_BLOCK}:BlockFP8LinearScratchCaps",
         "Plan": f"{_BLOCK}:BlockFP8LinearScratchPlan",
         "Binding": f"{_BLOCK}:BlockFP8LinearBinding",
         "Weight": f"{_BLOCK}:BlockFP8LinearWeight",
         "plan": f"{_BLOCK}:plan_block_fp8_linear_scratch",
         "bind": f"{_BLOCK}:bind_block_fp8_linear_scratch",
         "run": f"{_BLOCK}:block_fp8_linear_mxfp8",
         "pack_weight": f"{_BLOCK}:pack_block_fp8_linear_weight_mxfp8",
         "quantize_input": f"{_BLOCK}:quantize_block_fp8_linear_input_mxfp8",
         "prewarm": f"{_BLOCK}:prewarm_block_fp8_linear_mxfp8",
         "is_supported": SUPPORTED},
        dtypes=("bf16", "fp16", "fp8_e4m3"), recipes=("block_fp8", "mxfp8"),
        stands_in_for=("b12x/gemm/block_fp8_linear/api.py", "b12x/gemm/_shared/block_fp8.py"),
        tested_by="tests/test_linears_gpu.py")),
    ("gemm.tensor_fp8_linear", _op(
        "gemm.tensor_fp8_linear", "oneshot",
        {"Weight": "._kernel:TensorFP8LinearWeight", "mm": "._kernel:tensor_fp8_linear",
         "pack_weight": "._kernel:pack_tensor_fp8_linear_weight",
         "prewarm": "._kernel:prewarm_tensor_fp8_linear",
         "is_supported": "._kernel:is_supported"},
        dtypes=("bf16", "fp16"), recipes=("fp8",),
        stands_in_for=("b12x/gemm/tensor_fp8_linear/api.py",
                       "b12x/gemm/tensor_fp8_linear/_kernel.py"),
        tested_by="tests/test_linears_gpu.py")),
    ("gemm.bmm", _op(
        "gemm.bmm", "oneshot",
        {"bmm": ".api:bmm", "prewarm_bmm": ".api:prewarm_bmm",
         "can_implement_bmm": ".api:can_implement_bmm", "is_bmm_supported": ".api:is_bmm_supported"},
        dtypes=("bf16", "fp8_e4m3"), recipes=("mxfp8",),
        stands_in_for=("b12x/gemm/_bmm/api.py", "b12x/gemm/_shared/mxfp8_bmm.py"),
        tested_by="tests/test_bmm_gpu.py", since="0.2.0",
        notes="dtype-dispatched batched product; one backend: BF16 activations x rowwise MXFP8")),
    ("quantization.nvfp4", _op(
        "quantization.nvfp4", "planned",
        {"Outputs": "._impl:BF16ToFP4TMAOutputs", "Plan": "._plan:Plan", "plan": "._plan:plan",
         "allocate_outputs": "._plan:allocate_outputs", "run": "._plan:run",
         "is_supported": SUPPORTED},
        dtypes=("bf16", "fp4_e2m1"), recipes=("nvfp4",),
        stands_in_for=("b12x/quantization/nvfp4/api.py", "b12x/quantization/nvfp4/_impl.py",
                       "b12x/quantization/nvfp4/_kernel.py"),
        tested_by="tests/test_quantizers_gpu.py")),
    ("quantization.mxfp8", _op(
        "quantization.mxfp8", "oneshot",
        {"quantize_rows": "..._lib.mxfp8_rows:quantize_mxfp8_rows", "is_supported": SUPPORTED},
        dtypes=("bf16", "fp16", "fp8_e4m3"), recipes=("mxfp8",),
        stands_in_for=("b12x/quantization/mxfp8/api.py", "b12x/_lib/quant/mxfp8_rows.py"),
        tested_by="tests/test_quantizers_gpu.py")),
))


def _capability_probe(meta: OpMeta):
    def is_supported(device=None) -> bool:
        """True on a compute-capability 10.x device with the in-tree CUDA library built."""
        from .gating import default_is_supported

        return default_is_supported(device, requires=meta.requires)

    return is_supported


def install(namespace: dict[str, Any], qualname: str) -> OpMeta:
    """Turn the module whose globals are ``namespace`` into the op package ``qualname``."""
    meta, exports = OPS[qualname]
    package = namespace["__name__"]
    public = [*exports, "META"]

    def __getattr__(name: str) -> Any:
        target = exports.get(name)
        if target is None:
            raise AttributeError(f"module {package!r} has no attribute {name!r}")
        if target == SUPPORTED:
            found = _capability_probe(meta)
        else:
            module, _, attribute = target.partition(":")
            found = getattr(import_module(module, package), attribute)
        namespace[name] = found
        return found

    namespace.update(META=meta, __getattr__=__getattr__, __dir__=lambda: sorted(public),
                     __all__=public)
    return meta


__all__ = ["OPS", "OpMeta", "Provenance", "SUPPORTED", "install"]
