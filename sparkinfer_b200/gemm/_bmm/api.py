"""Dtype dispatch, validation and launch of :func:`sparkinfer_b200.gemm.bmm`.

Argument meaning and error behaviour follow b12x/gemm/_bmm/api.py:41-159 and the validation
of its MXFP8 backend (b12x/gemm/_shared/mxfp8_bmm.py:1561-1769): the same qualified envelope
(``B`` in {8, 16}; ``[B, K, N] = [B, 192, 512]`` N-major or ``[B, N, K] = [B, 256, 512]``
K-major; ``1 <= M <= 32``), the same stride and alignment rules, the same overlap checks.
"""

from __future__ import annotations

from collections.abc import Iterable
from typing import Literal, Optional

import torch

from ..._lib import launch
from ..._lib.gating import default_is_supported
from . import META

_SPECIALIZATION = ("bfloat16", "float8_e4m3fn", "float8_e8m0fnu", "bfloat16", 32)
_MAX_M = 32
_QUALIFIED_BATCHES = frozenset((8, 16))
_QUALIFIED_K_N = {"n": (192, 512), "k": (512, 256)}


def _require_specialization(a_dtype, b_dtype, sf_dtype, c_dtype, sf_vec_size) -> None:
    requested = (a_dtype, b_dtype, sf_dtype, c_dtype, sf_vec_size)
    if requested != _SPECIALIZATION:
        raise NotImplementedError(
            "gemm.bmm supports only a_dtype='bfloat16', b_dtype='float8_e4m3fn', "
            "sf_dtype='float8_e8m0fnu', c_dtype='bfloat16', sf_vec_size=32; "
            f"got {requested!r}")


def _major(b_major) -> str:
    name = b_major.lower() if isinstance(b_major, str) else None
    if name not in ("k", "n"):
        raise ValueError(f"b_major must be 'k' or 'n', got {b_major!r}")
    return name


def _rhs_pair(rhs) -> tuple[torch.Tensor, torch.Tensor]:
    if (not isinstance(rhs, tuple) or len(rhs) != 2
            or not all(isinstance(t, torch.Tensor) for t in rhs)):
        raise TypeError("rhs must be a (values, scales) tensor tuple")
    return rhs


def _rhs_geometry(values: torch.Tensor, scales: torch.Tensor, b_major, sf_axis):
    major = _major(b_major)
    if not isinstance(sf_axis, str) or sf_axis.lower() != major:
        raise NotImplementedError(
            "the BMM MXFP8 specialization requires sf_axis to match b_major, "
            f"got b_major={major!r}, sf_axis={sf_axis!r}")
    if values.ndim != 3:
        raise ValueError(f"rhs values must be 3-D, got shape {tuple(values.shape)}")
    if major == "n":
        groups, k, n = (int(s) for s in values.shape)
        scale_shape = (groups, k, n // 32)
    else:
        groups, n, k = (int(s) for s in values.shape)
        scale_shape = (groups, n, k // 32)
    if n <= 0 or k <= 0:
        raise ValueError(f"rhs dimensions must be positive, got N={n}, K={k}")
    if int(values.shape[-1]) % 32:
        raise ValueError("rhs physical inner dimension must be divisible by sf_vec_size=32, "
                         f"got {values.shape[-1]}")
    if tuple(scales.shape) != scale_shape:
        raise ValueError(f"rhs scales must have shape {scale_shape} for b_major={major!r}, "
                         f"sf_axis={sf_axis!r}; got {tuple(scales.shape)}")
    return major, groups, n, k


def _qualified(major: str, groups: int, m: int, n: int, k: int) -> bool:
    return (1 <= int(m) <= _MAX_M and int(groups) in _QUALIFIED_BATCHES
            and (int(k), int(n)) == _QUALIFIED_K_N[major])


def _check_strided(name: str, t: torch.Tensor, *, stride_mod: int, ptr_align: int) -> None:
    if t.stride(2) != 1:
        raise ValueError(f"{name} physical inner dimension must be contiguous")
    if t.stride(0) <= 0 or t.stride(1) <= 0:
        raise ValueError(f"{name} outer strides must be positive, got {t.stride()}")
    if t.stride(0) % stride_mod or t.stride(1) % stride_mod:
        raise ValueError(f"{name} outer strides {t.stride(0)}/{t.stride(1)} must be multiples "
                         f"of {stride_mod} elements")
    if t.data_ptr() % ptr_align:
        raise ValueError(f"{name} base pointer must be {ptr_align}-byte aligned")


def _check_operand(name: str, t: torch.Tensor, shape, *, stride_mod: int, ptr_align: int) -> None:
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    _check_strided(name, t, stride_mod=stride_mod, ptr_align=ptr_align)


def _validate_rhs_storage(values: torch.Tensor, scales: torch.Tensor) -> None:
    if values.dtype != torch.float8_e4m3fn:
        raise ValueError(f"rhs values must be float8_e4m3fn, got {values.dtype}")
    if scales.dtype not in (torch.uint8, torch.float8_e8m0fnu):
        raise ValueError(f"rhs scales must be uint8/e8m0, got {scales.dtype}")
    if not values.is_cuda or not scales.is_cuda:
        raise ValueError("BMM RHS tensors must be CUDA tensors")
    if values.device != scales.device:
        raise ValueError("BMM RHS tensors must be on the same CUDA device")
    for name, t, align in (("rhs values", values, 16), ("rhs scales", scales, 4)):
        if t.ndim != 3:
            raise ValueError(f"{name} must be 3-D, got shape {tuple(t.shape)}")
        _check_strided(name, t, stride_mod=align, ptr_align=align)


def _interval(t: torch.Tensor) -> tuple[int, int]:
    extent = 1 + sum((int(size) - 1) * int(stride)
                     for size, stride in zip(t.shape, t.stride()) if int(size) > 0)
    start = int(t.data_ptr())
    return start, start + extent * t.element_size()


def _overlaps(x: torch.Tensor, y: torch.Tensor) -> bool:
    if x.device != y.device:
        return False
    (x0, x1), (y0, y1) = _interval(x), _interval(y)
    return max(x0, y0) < min(x1, y1)


def _has_internal_overlap(t: torch.Tensor) -> bool:
    """True when two index tuples can reach one element (sizes sorted by stride must nest)."""
    dims = sorted(((int(st), int(sz)) for sz, st in zip(t.shape, t.stride()) if int(sz) > 1))
    reach = 1
    for stride, size in dims:
        if stride < reach:
            return True
        reach = stride * (size - 1) + reach
    return False


def _validate_launch(a, values, scales, out, b_major, sf_axis):
    major, b_groups, n, b_k = _rhs_geometry(values, scales, b_major, sf_axis)
    if a.ndim != 3:
        raise ValueError(f"lhs must have shape [B,M,K], got {tuple(a.shape)}")
    groups, m, k = (int(s) for s in a.shape)
    if groups != b_groups or k != b_k:
        raise ValueError("lhs and rhs batch/K dimensions must match: "
                         f"lhs is [B,M,K]=[{groups},{m},{k}], rhs implies B={b_groups}, K={b_k}")
    _check_operand("lhs", a, (groups, m, k), stride_mod=8, ptr_align=16)
    _check_operand("out", out, (groups, m, n), stride_mod=2, ptr_align=4)
    if _has_internal_overlap(out):
        raise ValueError("out must not have internal storage overlap")
    _validate_rhs_storage(values, scales)
    tensors = (a, values, scales, out)
    if not all(t.is_cuda for t in tensors):
        raise ValueError("BMM operands must be CUDA tensors")
    if any(t.device != a.device for t in tensors[1:]):
        raise ValueError("BMM operands must be on the same CUDA device")
    if not _qualified(major, groups, m, n, k):
        raise NotImplementedError(
            "the BMM MXFP8 specialization is qualified for b_major='n' [B,K,N]=[16,192,512] or "
            "b_major='k' [B,N,K]=[16,256,512], with 1<=M<=32; "
            f"got b_major={major!r}, B={groups}, M={m}, N={n}, K={k}")
    for name, source in (("lhs", a), ("rhs values", values), ("rhs scales", scales)):
        if _overlaps(out, source):
            raise ValueError(f"out must not overlap {name}")
    return major, groups, m, n, k


@torch.library.custom_op("b12x::bmm_mxfp8_launch", mutates_args=("out",))
def _bmm_launch_op(a: torch.Tensor, values: torch.Tensor, scales: torch.Tensor,
                   out: torch.Tensor, n_major: bool, stream_int: Optional[int]) -> None:
    groups, m, k = (int(s) for s in a.shape)
    launch.bmm_mxfp8(a, values, scales, out, n_major=n_major, batch=groups, m=m,
                     n=int(out.shape[2]), k=k, stream_int=stream_int)


@_bmm_launch_op.register_fake
def _bmm_launch_fake(a, values, scales, out, n_major, stream_int) -> None:
    return None


def _run(a, values, scales, out, *, b_major, sf_axis, stream) -> None:
    if torch.compiler.is_compiling() or type(a) is not torch.Tensor:
        # Tracing: shapes are checked by the eager call that follows the trace.
        major = _major(b_major)
        _bmm_launch_op(a, values, scales, out, major == "n", launch.cuda_stream_to_int(stream))
        return
    major, groups, m, n, k = _validate_launch(a, values, scales, out, b_major, sf_axis)
    stream_int = launch.cuda_stream_to_int(stream)
    if stream is not None:
        owner = (torch.cuda.default_stream(a.device) if stream_int == 0
                 else torch.cuda.ExternalStream(stream_int, device=a.device))
        for t in (a, values, scales, out):
            t.record_stream(owner)
    launch.bmm_mxfp8(a, values, scales, out, n_major=major == "n", batch=groups, m=m, n=n, k=k,
                     stream_int=stream_int)


def bmm(lhs: torch.Tensor, rhs: tuple[torch.Tensor, torch.Tensor], out: torch.Tensor, *,
        a_dtype: str, b_dtype: str, sf_dtype: str, c_dtype: str, sf_vec_size: int,
        b_major: Literal["k", "n"] = "k", sf_axis: Literal["k", "n"] = "k",
        stream: Optional[object] = None) -> torch.Tensor:
    """Compute a batch of ``C = A @ B`` into caller-owned ``out`` and return it.

    ``lhs`` and ``out`` have logical shapes ``[B, M, K]`` and ``[B, M, N]``. ``rhs`` is
    ``(values, scales)``: ``torch.float8_e4m3fn`` values and E8M0 scale bytes (``torch.uint8``
    or ``torch.float8_e8m0fnu``). ``b_major='k'`` stores them as ``[B, N, K]`` and
    ``[B, N, K/32]``; ``b_major='n'`` as ``[B, K, N]`` and ``[B, K, N/32]``. ``sf_axis`` must
    equal ``b_major``."""
    _require_specialization(a_dtype, b_dtype, sf_dtype, c_dtype, sf_vec_size)
    values, scales = _rhs_pair(rhs)
    _run(lhs, values, scales, out, b_major=b_major, sf_axis=sf_axis, stream=stream)
    return out


def prewarm_bmm(rhs: tuple[torch.Tensor, torch.Tensor], m_values: Iterable[int], *,
                a_dtype: str, b_dtype: str, sf_dtype: str, c_dtype: str, sf_vec_size: int,
                b_major: Literal["k", "n"] = "k", sf_axis: Literal["k", "n"] = "k",
                stream: Optional[object] = None, synchronize: bool = True) -> int:
    """First-launch every caller-declared ``M`` on zero activations; returns how many distinct
    ``M`` were launched. Nothing is compiled: the kernels ship in the library."""
    _require_specialization(a_dtype, b_dtype, sf_dtype, c_dtype, sf_vec_size)
    values, scales = _rhs_pair(rhs)
    major, groups, n, k = _rhs_geometry(values, scales, b_major, sf_axis)
    _validate_rhs_storage(values, scales)
    wanted = sorted({int(m) for m in m_values})
    for m in wanted:
        if not _qualified(major, groups, m, n, k):
            raise NotImplementedError(
                f"M={m} is outside the qualified envelope for b_major={major!r}, B={groups}, "
                f"N={n}, K={k}")
    stream_int = launch.cuda_stream_to_int(stream)
    ctx = (torch.cuda.stream(torch.cuda.ExternalStream(stream_int, device=values.device))
           if stream_int else torch.cuda.device(values.device))
    with ctx:
        for m in wanted:
            lhs = torch.zeros((groups, m, k), dtype=torch.bfloat16, device=values.device)
            out = torch.empty((groups, m, n), dtype=torch.bfloat16, device=values.device)
            launch.bmm_mxfp8(lhs, values, scales, out, n_major=major == "n", batch=groups, m=m,
                             n=n, k=k, stream_int=stream_int)
    if synchronize:
        torch.cuda.synchronize(values.device)
    return len(wanted)


def can_implement_bmm(*, batch: int, max_m: int, n: int, k: int, a_dtype: str, b_dtype: str,
                      sf_dtype: str, c_dtype: str, sf_vec_size: int,
                      b_major: Literal["k", "n"] = "k", sf_axis: Literal["k", "n"] = "k",
                      device=None) -> bool:
    """Whether the qualified specialization covers a plan (never raises)."""
    if (a_dtype, b_dtype, sf_dtype, c_dtype, sf_vec_size) != _SPECIALIZATION:
        return False
    if not isinstance(b_major, str) or b_major.lower() not in ("k", "n"):
        return False
    if not isinstance(sf_axis, str) or sf_axis.lower() != b_major.lower():
        return False
    return is_bmm_supported(device) and _qualified(b_major.lower(), batch, max_m, n, k) \
        and int(max_m) >= 1


def is_bmm_supported(device=None) -> bool:
    """True on a compute-capability 10.x device with the in-tree CUDA library built."""
    return default_is_supported(device, requires=META.requires)


def clear_bmm_caches() -> None:
    """Nothing is cached: the kernels are compiled ahead of time."""


__all__ = ["bmm", "can_implement_bmm", "is_bmm_supported", "prewarm_bmm"]
