"""torch tensors -> C-ABI calls. Every public op funnels through these few functions.

They validate what the C ABI cannot (device, dtype, contiguity), pick the stream, and pass
raw pointers. Nothing here computes on tensors: if the CUDA library is missing the import
of :mod:`sparkinfer_b200._native` raises.
"""

from __future__ import annotations

import ctypes
from threading import Lock

import torch

from .. import _native

_STATUS_LOCK = Lock()
_STATUS: dict[int, torch.Tensor] = {}
_WORKSPACE: dict[int, torch.Tensor] = {}
SMALL_M_MAX = 128        # largest M the decode kernel accepts
SMALL_M_AUTO = 64        # largest M routed to it automatically

_DTYPE_CODE = {torch.bfloat16: _native.DT_BF16, torch.float16: _native.DT_FP16,
               torch.float32: _native.DT_FP32}

import os as _os

_SMALL_M_DISABLED = _os.getenv("B12X_B200_DISABLE_SMALL_M", "0") == "1"

KERNEL_STATUS_TEXT = {
    1: "TMA producer timed out waiting for a free pipeline stage",
    2: "MMA issuer timed out waiting for operands or a free accumulator",
    3: "epilogue timed out waiting for a finished accumulator",
    4: "split-K reduction timed out waiting for its peers",
    5: "tensor memory was not allocated from column 0",
}


def cuda_stream_to_int(stream: object | None) -> int | None:
    """Raw CUDA stream handle of ``stream`` (object with ``.cuda_stream`` or int); ``None``
    stays ``None`` and means torch's current stream (b12x/_lib/utils.py:184-204)."""
    if stream is None:
        return None
    handle = getattr(stream, "cuda_stream", None)
    return int(handle) if handle is not None else int(stream)


def _stream_ptr(stream_int: int | None, device: torch.device) -> ctypes.c_void_p:
    if stream_int is None:
        stream_int = torch.cuda.current_stream(device).cuda_stream
    return ctypes.c_void_p(int(stream_int))


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] the kernels raise when a bounded wait runs out. Allocated once, on
    first use (call an op once before CUDA-graph capture, as with any warm-up)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    with _STATUS_LOCK:
        buf = _STATUS.get(index)
        if buf is None:
            buf = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", index))
            _STATUS[index] = buf
        return buf


def check_kernel_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a timed-out wait."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    buf = status_buffer(device)
    code = int(buf[0].item())
    if code != 0:
        buf.zero_()
        raise RuntimeError(f"b12x kernel status {code}: {KERNEL_STATUS_TEXT.get(code, 'unknown')}")


def _require_cuda(name: str, t: torch.Tensor) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be on CUDA")


def smallm_workspace(kind: int, m: int, n: int, k: int, device: torch.device,
                     sm_count: int = 0) -> torch.Tensor:
    """Per-device scratch of the decode-shape kernel (FP32 partial tiles + per-tile counters).
    Created zeroed and grown on demand, so the first call for a larger shape allocates (warm up
    before CUDA-graph capture). Every launch leaves the counters zero, and launches on one
    device share the buffer, so they must not overlap on the GPU (same stream, or ordered)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(index):
        need = int(_native.load().b12x_b200_gemm_smallm_workspace_bytes(kind, m, n, k, sm_count))
    if need < 0:
        raise _native.NativeLibraryError(f"no decode-shape plan for M={m}, N={n}, K={k}")
    with _STATUS_LOCK:
        buf = _WORKSPACE.get(index)
        if buf is None or buf.numel() < need:
            buf = torch.zeros(max(need, 1 << 20), dtype=torch.uint8,
                              device=torch.device("cuda", index))
            _WORKSPACE[index] = buf
        return buf


def gemm_blockscaled(kind: int, a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor,
                     sfb: torch.Tensor, c: torch.Tensor, alpha: torch.Tensor | None,
                     m: int, n: int, k: int, *, ldc: int | None = None, block_n: int = 0,
                     sm_count: int = 0, stream_int: int | None = None,
                     small_m: bool | None = None) -> None:
    """``c[M, ldc] = cvt(alpha * (a . sfa)(b . sfb)^T)`` for one group. ``a``/``b`` are row
    pointers to K-major code matrices, ``sfa``/``sfb`` point at the first scale atom.

    Decode shapes (M <= 128, unless ``small_m=False`` or a tile width is forced) go to the
    weight-streaming stream-K kernel, everything else to the persistent tiled kernel."""
    for name, t in (("a", a), ("b", b), ("sfa", sfa), ("sfb", sfb), ("c", c)):
        _require_cuda(name, t)
    if c.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported output dtype {c.dtype}")
    dev = a.device
    if small_m is None:
        small_m = m <= SMALL_M_AUTO and block_n == 0 and not _SMALL_M_DISABLED
    if small_m and 0 < m <= SMALL_M_MAX and n > 0:
        work = smallm_workspace(kind, m, n, k, dev, sm_count)
        with torch.cuda.device(dev):
            rc = _native.load().b12x_b200_gemm_blockscaled_smallm(
                kind, a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), c.data_ptr(),
                _DTYPE_CODE[c.dtype], alpha.data_ptr() if alpha is not None else None,
                m, n, k, ldc if ldc is not None else n, work.data_ptr(), work.numel(), sm_count,
                status_buffer(dev).data_ptr(), _stream_ptr(stream_int, dev))
        _native.check(rc, "b12x_b200_gemm_blockscaled_smallm")
        return
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_gemm_blockscaled(
            kind, a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), c.data_ptr(),
            _DTYPE_CODE[c.dtype], alpha.data_ptr() if alpha is not None else None,
            m, n, k, ldc if ldc is not None else n, block_n, sm_count,
            status_buffer(dev).data_ptr(), _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_gemm_blockscaled")


def gemm_block_fp8(a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor, sfb: torch.Tensor,
                   c: torch.Tensor, alpha: torch.Tensor | None, m: int, n: int, k: int, *,
                   ldc: int | None = None, sm_count: int = 0,
                   stream_int: int | None = None) -> None:
    """E4M3 operands with FP32 scales ``sfa [M, K/128]`` / ``sfb [N/128, K/128]``."""
    for name, t in (("a", a), ("b", b), ("sfa", sfa), ("sfb", sfb), ("c", c)):
        _require_cuda(name, t)
    dev = a.device
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_gemm_block_fp8(
            a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), c.data_ptr(),
            _DTYPE_CODE[c.dtype], alpha.data_ptr() if alpha is not None else None, m, n, k,
            ldc if ldc is not None else n, sm_count, status_buffer(dev).data_ptr(),
            _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_gemm_block_fp8")


def quantize_mxfp8_rows(src: torch.Tensor, values: torch.Tensor, scale_rows: torch.Tensor | None,
                        scale_mma: torch.Tensor | None, *, stream_int: int | None = None) -> None:
    _require_cuda("source", src)
    m, k = src.shape
    dev = src.device
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_quantize_mxfp8_rows(
            src.data_ptr(), _DTYPE_CODE[src.dtype], src.stride(0), values.data_ptr(),
            scale_rows.data_ptr() if scale_rows is not None else None,
            scale_mma.data_ptr() if scale_mma is not None else None, m, k,
            _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_quantize_mxfp8_rows")


def quantize_nvfp4_rows(src: torch.Tensor, global_scale: torch.Tensor, packed: torch.Tensor,
                        scale_mma: torch.Tensor, *, stream_int: int | None = None) -> None:
    _require_cuda("source", src)
    m, k = src.shape
    dev = src.device
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_quantize_nvfp4_rows(
            src.data_ptr(), _DTYPE_CODE[src.dtype], src.stride(0), global_scale.data_ptr(),
            packed.data_ptr(), scale_mma.data_ptr(), m, k, _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_quantize_nvfp4_rows")


__all__ = [
    "cuda_stream_to_int", "status_buffer", "check_kernel_status", "gemm_blockscaled",
    "gemm_block_fp8", "quantize_mxfp8_rows", "quantize_nvfp4_rows", "KERNEL_STATUS_TEXT",
]
