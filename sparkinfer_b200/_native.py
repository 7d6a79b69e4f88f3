"""ctypes binding of the C-ABI library ``_b12x_b200.so`` (declared in include/b12x_b200.h).

The library is built in-tree by :mod:`sparkinfer_b200.build`. There is no fallback: if the
shared object is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path
from threading import Lock

_LIB_NAME = "_b12x_b200.so"
_LOCK = Lock()
_LIB: ctypes.CDLL | None = None

KIND_MXFP8 = 0
KIND_NVFP4 = 1
KIND_FP8 = 2      # E4M3 without block scales (tiled and CTA-pair kernels only)
KIND_MXFP4 = 3    # E2M1 codes with UE8M0 scales per 32 elements (no fused activation quantizer)
DT_BF16 = 0
DT_FP16 = 1
DT_FP32 = 2
BLOCK_N_PAIR = -256  # B12X_B200_BLOCK_N_PAIR: force the CTA-pair kernel

_c_void_p = ctypes.c_void_p
_c_int = ctypes.c_int
_c_i64 = ctypes.c_int64


class Epilogue(ctypes.Structure):
    """``b12x_b200_epilogue_t``: optional bias and MXFP8 re-quantization of the output."""

    _fields_ = [("bias", _c_void_p), ("quant_values", _c_void_p), ("quant_scale_rows", _c_void_p),
                ("quant_scale_mma", _c_void_p), ("quant_ld", _c_i64), ("quant_col0", _c_i64),
                ("quant_cols", _c_i64)]


_c_epilogue_p = ctypes.POINTER(Epilogue)

# name -> (restype, argtypes); one entry per function declared in include/b12x_b200.h.
SIGNATURES = {
    "b12x_b200_version": (ctypes.c_char_p, []),
    "b12x_b200_last_error": (ctypes.c_char_p, []),
    "b12x_b200_gemm_blockscaled": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_blockscaled_workspace_bytes": (
        _c_i64, [_c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int]),
    "b12x_b200_gemm_blockscaled_ex": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_void_p, _c_i64, _c_epilogue_p,
         _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_grouped_workspace_bytes": (
        _c_i64, [_c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_int]),
    "b12x_b200_gemm_blockscaled_grouped": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_void_p, _c_i64, _c_epilogue_p,
         _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_blockscaled_smallm_grouped": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_void_p, _c_i64, _c_epilogue_p, _c_int,
         _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_blockscaled_smallm_ex": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_void_p, _c_i64, _c_epilogue_p, _c_int, _c_void_p,
         _c_void_p],
    ),
    "b12x_b200_gemm_block_fp8_ex": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_epilogue_p, _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_smallm_workspace_bytes": (_c_i64, [_c_int, _c_i64, _c_i64, _c_i64, _c_int]),
    "b12x_b200_gemm_blockscaled_smallm": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_void_p, _c_i64, _c_int, _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_smallm_fused_quant": (
        _c_int,
        [_c_int, _c_void_p, _c_i64, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_void_p, _c_i64, _c_epilogue_p, _c_int, _c_void_p,
         _c_void_p],
    ),
    "b12x_b200_gemm_smallm_fused_quant_grouped": (
        _c_int,
        [_c_int, _c_void_p, _c_i64, _c_i64, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
         _c_void_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_void_p, _c_i64, _c_epilogue_p,
         _c_int, _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_smallm_fused_quant_grouped_inv_rope": (
        _c_int,
        [_c_void_p, _c_i64, _c_i64, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int,
         _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_i64, _c_i64, _c_i64, _c_i64,
         _c_i64, _c_void_p, _c_i64, _c_int, _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_smallm_timeline": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_void_p, _c_i64, _c_int, _c_void_p, _c_i64,
         _c_void_p, _c_void_p],
    ),
    "b12x_b200_selftest_wait_timeout": (_c_int, [_c_void_p, _c_int, _c_void_p]),
    "b12x_b200_pack_block_fp8_weight_mxfp8": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_i64, _c_i64, _c_i64, _c_int,
         _c_void_p],
    ),
    "b12x_b200_bmm_mxfp8": (
        _c_int,
        [_c_void_p, _c_i64, _c_i64, _c_void_p, _c_i64, _c_i64, _c_void_p, _c_i64, _c_i64,
         _c_void_p, _c_i64, _c_i64, _c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_void_p],
    ),
    "b12x_b200_allreduce_peer_signal_bytes": (_c_i64, []),
    "b12x_b200_gemm_blockscaled_scatter": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int,
         _c_void_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_void_p, _c_i64, _c_void_p,
         _c_void_p],
    ),
    "b12x_b200_allreduce_peer_scattered": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_int,
         _c_i64, _c_void_p, _c_void_p],
    ),
    "b12x_b200_allreduce_peer": (
        _c_int,
        [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_i64,
         _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_smallm_noalloc_capacity_bytes": (_c_i64, []),
    "b12x_b200_gemm_blockscaled_smallm_noalloc": (
        _c_int,
        [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_void_p, _c_void_p],
    ),
    "b12x_b200_gemm_block_fp8": (
        _c_int,
        [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
         _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_void_p, _c_void_p],
    ),
    "b12x_b200_quantize_mxfp8_rows": (
        _c_int,
        [_c_void_p, _c_int, _c_i64, _c_void_p, _c_void_p, _c_void_p, _c_i64, _c_i64, _c_void_p],
    ),
    "b12x_b200_quantize_nvfp4_rows": (
        _c_int,
        [_c_void_p, _c_int, _c_i64, _c_void_p, _c_void_p, _c_void_p, _c_i64, _c_i64, _c_void_p],
    ),
}


class NativeLibraryError(RuntimeError):
    """The CUDA extension is missing, failed to load, or a call returned an error."""


def library_path() -> Path:
    override = os.environ.get("B12X_B200_LIBRARY")
    return Path(override) if override else Path(__file__).resolve().parent / _LIB_NAME


def load() -> ctypes.CDLL:
    """Load the shared object once and declare every prototype."""
    global _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not path.exists():
            raise NativeLibraryError(
                f"{path} not found: build it with `python -m sparkinfer_b200.build` "
                "(there is no CPU or PyTorch fallback for these ops)"
            )
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise NativeLibraryError(f"cannot load {path}: {exc}") from exc
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = lib
        return lib


def last_error() -> str:
    return load().b12x_b200_last_error().decode("utf-8", "replace")


def check(code: int, what: str) -> None:
    if code != 0:
        raise NativeLibraryError(f"{what} failed with code {code}: {last_error()}")


def version() -> str:
    return load().b12x_b200_version().decode()
