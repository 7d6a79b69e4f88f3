"""The C-ABI library loads without a GPU and exports every function include/*.h declares."""

from __future__ import annotations

import ctypes
import re

from conftest import ROOT
from sparkinfer_b200 import _native


def _declared_functions() -> set[str]:
    names: set[str] = set()
    for header in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(b12x_b200_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    declared = _declared_functions()
    assert {"b12x_b200_gemm_blockscaled", "b12x_b200_quantize_mxfp8_rows",
            "b12x_b200_quantize_nvfp4_rows", "b12x_b200_version"} <= declared
    lib = ctypes.CDLL(str(_native.library_path()))
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_python_binding_covers_every_declared_symbol():
    assert set(_native.SIGNATURES) == _declared_functions()


def test_version_string():
    assert _native.version().startswith("b12x_b200 ") and "sm_100a" in _native.version()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("B12X_B200_LIBRARY", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_native, "_LIB", None)
    try:
        _native.load()
    except _native.NativeLibraryError as exc:
        assert "no CPU or PyTorch fallback" in str(exc)
    else:  # pragma: no cover
        raise AssertionError("loading a missing library must raise")
