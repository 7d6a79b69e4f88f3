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
        assert on_disk == set(names), (group, on_disk, names)


@pytest.mark.parametrize("meta", pkg.list_ops(), ids=lambda m: m.qualname)
def test_meta_shape_and_entry_points(meta):
    assert meta.archs == ("sm100a",)
    assert meta.api_style in ("planned", "oneshot")
    assert meta.entry_points and "is_supported" in meta.entry_points
    module = importlib.import_module(f"sparkinfer_b200.{meta.group}.{meta.name}")
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
