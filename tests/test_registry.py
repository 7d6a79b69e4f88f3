"""Registry and packaging contract (modelled on the reference's tests/test_registry.py:33-94
and its arch lint): op table <-> directories, META shape, lazy resolution, sm_100a only."""

from __future__ import annotations

import importlib
import subprocess
import sys

import pytest

import sparkinfer_b200 as pkg
from conftest import ROOT


def test_ops_table_matches_directories():
    for group, names in pkg._OPS.items():
        group_dir = ROOT / "sparkinfer_b200" / group
        on_disk = {p.name for p in group_dir.iterdir()
                   if p.is_dir() and not p.name.startswith("_")}
        private = {q.split(".")[1] for q in pkg._OP_MODULE_OVERRIDES if q.startswith(group + ".")}
        assert on_disk == set(names) - private, (group, on_disk, names)
        for qualname, path in pkg._OP_MODULE_OVERRIDES.items():
            assert (ROOT / "sparkinfer_b200" / path.replace(".", "/")).is_dir(), qualname


@pytest.mark.parametrize("meta", pkg.list_ops(), ids=lambda m: m.qualname)
def test_meta_shape_and_entry_points(meta):
    assert meta.archs == ("sm100a",)
    assert meta.api_style in ("planned", "oneshot")
    assert meta.entry_points and any(e in meta.entry_points
                                     for e in ("is_supported", f"is_{meta.name}_supported"))
    module = pkg._op_module(meta.group, meta.name)
    for name in meta.entry_points:
        assert getattr(module, name) is not None
    assert sorted(dir(module)) == sorted([*meta.entry_points, "META"])
    with pytest.raises(AttributeError):
        getattr(module, "no_such_entry_point")
    assert pkg.find_op(meta.qualname) is meta


def test_find_op_rejects_unknown():
    with pytest.raises(KeyError):
        pkg.find_op("gemm.nope")


def test_importing_op_packages_is_side_effect_free():
    code = (
        "import sys; import sparkinfer_b200; "
        "from sparkinfer_b200.gemm import blockscaled, mxfp8_linear, block_fp8_linear; "
        "from sparkinfer_b200.quantization import nvfp4, mxfp8; "
        "assert 'torch' not in sys.modules and 'ctypes' not in sys.modules, sorted(sys.modules)"
    )
    subprocess.run([sys.executable, "-c", code], check=True, cwd=ROOT)


def test_install_as_b12x_aliases_import_paths():
    code = (
        "import sparkinfer_b200 as s; s.install_as_b12x(); import b12x; "
        "from b12x.gemm import blockscaled; from b12x.quantization import nvfp4; "
        "from b12x.gemm.block_fp8_linear import Caps; "
        "import sparkinfer_b200.gemm.blockscaled as real; assert blockscaled is real; "
        "assert b12x.find_op('gemm.blockscaled').name == 'blockscaled'"
    )
    subprocess.run([sys.executable, "-c", code], check=True, cwd=ROOT)


def test_freeze_controls_are_present_and_fail_closed():
    from sparkinfer_b200._lib import runtime_control as rc

    assert not pkg.kernel_resolution_frozen()
    pkg.freeze_kernel_resolution("serving")
    try:
        assert pkg.kernel_resolution_frozen() and pkg.compilation_frozen()
        with pytest.raises(pkg.KernelResolutionFrozenError, match="serving"):
            rc.raise_if_kernel_resolution_frozen("cute.compile", cache_key=(1, 2))
    finally:
        pkg.unfreeze_kernel_resolution()
    rc.raise_if_kernel_resolution_frozen("cute.compile")


def test_cuda_sources_target_sm100a_only_and_never_multicast():
    csrc = ROOT / "sparkinfer_b200" / "csrc"
    text = "".join(p.read_text() for p in csrc.iterdir())
    forbidden = "multi" + "cast" + "::cluster"  # spelled in pieces so this file does not name it
    assert forbidden not in text
    build_py = (ROOT / "sparkinfer_b200" / "build.py").read_text()
    assert "compute_100a" in build_py and "sm_100a" in build_py
    for other in ("sm_90", "sm_120", "compute_120"):
        assert other not in build_py


def test_graft_entry_build_runs_without_a_gpu():
    """``build()`` is the does-it-build check that runs on a CPU-only machine: it compiles the
    library (a no-op when it is current), loads it and imports the package."""
    import __graft_entry__ as entry

    entry.build()


def test_gemm_group_exposes_flat_functions():
    """``gemm.mm`` is ``blockscaled.mm``; ``gemm.bmm`` is a function, not an op package
    (the reference's tests/gemm/test_bmm.py:116-140)."""
    from sparkinfer_b200 import gemm

    pkg.list_ops()
    flat = gemm.bmm
    assert callable(flat) and not hasattr(flat, "mm")
    pkg.list_ops()
    assert gemm.bmm is flat
    assert gemm.mm is gemm.blockscaled.mm
    meta = pkg.find_op("gemm.bmm")
    assert meta.qualname == "gemm.bmm"
    assert set(meta.entry_points) == {"bmm", "prewarm_bmm", "can_implement_bmm", "is_bmm_supported"}
    assert not hasattr(gemm, "Weight")
    with pytest.raises(AttributeError):
        gemm.no_such_function


def test_bmm_host_checks_need_no_gpu():
    import torch

    from sparkinfer_b200 import gemm

    spec = dict(a_dtype="bfloat16", b_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu",
                c_dtype="bfloat16", sf_vec_size=32)
    lhs = torch.zeros(16, 1, 192, dtype=torch.bfloat16)
    values = torch.zeros(16, 192, 512, dtype=torch.float8_e4m3fn)
    scales = torch.zeros(16, 192, 16, dtype=torch.uint8)
    out = torch.empty(16, 1, 512, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError, match="supports only"):
        gemm.bmm(lhs, (values, scales), out, **{**spec, "b_dtype": "bfloat16"},
                 b_major="n", sf_axis="n")
    with pytest.raises(NotImplementedError, match="sf_axis to match b_major"):
        gemm.bmm(lhs, (values, scales), out, **spec, b_major="n", sf_axis="k")
    with pytest.raises(TypeError, match="tensor tuple"):
        gemm.bmm(lhs, [values, scales], out, **spec, b_major="n", sf_axis="n")
    with pytest.raises(ValueError, match="rhs scales must have shape"):
        gemm.bmm(lhs, (values, scales[:, :, :8]), out, **spec, b_major="n", sf_axis="n")
    with pytest.raises(ValueError, match="rhs values must be float8_e4m3fn"):
        gemm.bmm(lhs, (values.to(torch.bfloat16), scales), out, **spec, b_major="n", sf_axis="n")
    overlapped = torch.as_strided(torch.empty(1024, dtype=torch.bfloat16), (16, 2, 512), (2, 2, 1))
    with pytest.raises(ValueError, match="internal storage overlap"):
        gemm.bmm(torch.zeros(16, 2, 192, dtype=torch.bfloat16), (values, scales), overlapped,
                 **spec, b_major="n", sf_axis="n")
    with pytest.raises(ValueError, match="CUDA"):
        gemm.bmm(lhs, (values, scales), out, **spec, b_major="n", sf_axis="n")
    kwargs = dict(batch=16, max_m=32, n=512, k=192, **spec, b_major="n", sf_axis="n")
    assert not gemm.can_implement_bmm(**kwargs)            # no sm_100 device here
    assert not gemm.can_implement_bmm(**{**kwargs, "b_dtype": "bfloat16"})
