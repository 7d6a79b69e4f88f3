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
# (device index, stream handle) -> every decode workspace ever handed out for that stream, the
# newest last. Superseded buffers are kept: a captured CUDA graph or a kernel still in flight
# may hold their address.
_WORKSPACES: dict[tuple[int, int], list[torch.Tensor]] = {}
# device index -> zeroed workspaces not yet bound to a stream. A stream first seen during CUDA
# graph capture (torch captures on a side stream) takes one of these instead of allocating,
# which inside a capture would add a fill node to every replay.
_SPARE_WORKSPACES: dict[int, list[torch.Tensor]] = {}
_SPARES_PER_DEVICE = 2
SMALL_M_MAX = 128        # largest M the decode kernel accepts
SMALL_M_AUTO = 64        # largest M always routed to it
FUSED_QUANT_MAX_M = 16   # largest M of the decode kernel with the activation quantizer fused in
_WORKSPACE_MIN_BYTES = 8 << 20
_COUNTER_BYTES = 64 << 10  # counter block at the start of a decode workspace

_DTYPE_CODE = {torch.bfloat16: _native.DT_BF16, torch.float16: _native.DT_FP16,
               torch.float32: _native.DT_FP32}

import os as _os

# Debug aid, off by default: B12X_B200_CHECK_STATUS=1 makes every launcher synchronise and call
# check_kernel_status() after its kernel, so that a kernel that gave up a bounded wait (and left
# its output unwritten) raises at the call that launched it instead of going unnoticed. It
# serialises the host with the device and cannot be used under CUDA-graph capture.
_CHECK_AFTER_LAUNCH = _os.getenv("B12X_B200_CHECK_STATUS", "0") == "1"


def _after_launch(device: torch.device) -> None:
    if _CHECK_AFTER_LAUNCH and not torch.cuda.is_current_stream_capturing():
        check_kernel_status(device)

KERNEL_STATUS_TEXT = {
    1: "TMA producer timed out waiting for a free pipeline stage",
    2: "MMA issuer timed out waiting for operands or a free accumulator",
    3: "epilogue timed out waiting for a finished accumulator",
    4: "split-K reduction timed out waiting for its peers",
    5: "tensor memory was not allocated from column 0",
    6: "all-reduce over peer memory timed out waiting for another rank",
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


def _zeros_ready_for_any_stream(nbytes: int, index: int, dtype=torch.uint8) -> torch.Tensor:
    """Zero-filled device buffer whose fill has completed before it is handed to a kernel on
    some other stream. Under stream capture the fill is captured in order instead (the kernels
    that use the buffer are captured on the same stream) and nothing is synchronised."""
    device = torch.device("cuda", index)
    buf = torch.zeros(nbytes, dtype=dtype, device=device)
    if not torch.cuda.is_current_stream_capturing():
        torch.cuda.current_stream(device).synchronize()
    return buf


def _top_up_spares(index: int, size: int) -> None:
    """Keep a few zeroed workspaces of at least ``size`` bytes ready for streams that first
    show up inside a capture. Called with the lock held, outside any capture."""
    spares = _SPARE_WORKSPACES.setdefault(index, [])
    spares[:] = [b for b in spares if b.numel() >= size]
    while len(spares) < _SPARES_PER_DEVICE:
        spares.append(_zeros_ready_for_any_stream(size, index))


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] the kernels raise when a bounded wait runs out. Allocated once, on
    first use (call an op once before CUDA-graph capture, as with any warm-up)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    with _STATUS_LOCK:
        buf = _STATUS.get(index)
        if buf is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("call the op once on this device before capturing it into a "
                                   "CUDA graph (the kernel status word is created on first use)")
            buf = _zeros_ready_for_any_stream(4, index, torch.int32)
            _STATUS[index] = buf
        return buf


def check_kernel_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a timed-out wait. A kernel
    that gave up may have left per-tile counters of a decode workspace non-zero, so those are
    cleared together with the status word before the exception leaves."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    index = device.index if device.index is not None else torch.cuda.current_device()
    buf = status_buffer(device)
    torch.cuda.synchronize(device)
    code = int(buf[0].item())
    if code != 0:
        buf.zero_()
        with _STATUS_LOCK:
            stale = [w for (dev, _), ws in _WORKSPACES.items() if dev == index for w in ws]
        for w in stale:
            w[:_COUNTER_BYTES].zero_()
        torch.cuda.synchronize(device)
        raise RuntimeError(f"b12x kernel status {code}: {KERNEL_STATUS_TEXT.get(code, 'unknown')}")


def _require_cuda(name: str, t: torch.Tensor) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be on CUDA")


def stream_workspace(need: int, device: torch.device, stream_int: int | None = None) -> torch.Tensor:
    """Scratch (counters + FP32 partial tiles) for the kernels that split work along K, for
    launches on one stream of one device. Launches on the same stream run in order and share a
    buffer; every stream has its own, so such kernels on different streams never meet in one. A
    buffer is created zeroed the first time a stream needs one, or a larger one (so warm up
    before CUDA-graph capture), and is never released while the process lives."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if stream_int is None:
        stream_int = torch.cuda.current_stream(torch.device("cuda", index)).cuda_stream
    key = (index, int(stream_int))
    capturing = torch.cuda.is_current_stream_capturing()
    with _STATUS_LOCK:
        bufs = _WORKSPACES.setdefault(key, [])
        if not bufs or bufs[-1].numel() < need:
            size = _WORKSPACE_MIN_BYTES
            while size < need:
                size *= 2
            spares = _SPARE_WORKSPACES.get(index, [])
            fit = next((b for b in spares if b.numel() >= size), None) if capturing else None
            if fit is not None:
                spares[:] = [b for b in spares if b is not fit]
                bufs.append(fit)
            else:
                bufs.append(_zeros_ready_for_any_stream(size, index))
        if not capturing:
            _top_up_spares(index, bufs[-1].numel())
        return bufs[-1]


def smallm_workspace(kind: int, m: int, n: int, k: int, device: torch.device,
                     sm_count: int = 0, stream_int: int | None = None) -> torch.Tensor:
    """:func:`stream_workspace` sized for the decode-shape kernel on (M, N, K)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(index):
        need = int(_native.load().b12x_b200_gemm_smallm_workspace_bytes(kind, m, n, k, sm_count))
    if need < 0:
        raise _native.NativeLibraryError(f"no decode-shape plan for M={m}, N={n}, K={k}")
    return stream_workspace(need, device, stream_int)


def route_to_decode_kernel(m: int, n: int, device: torch.device, sm_count: int = 0) -> bool:
    """Whether an unforced GEMM of ``m`` rows goes to the weight-streaming decode kernel: up to
    64 rows. With 65..128 rows the decode kernel (one issuing warp, 128 padded rows per stage)
    was measured far behind the tiled kernel even on a grid the tiled kernel fills less than
    half (128 x 4096 x 4096: 25 us against 9 us), so it is only used there on request."""
    return 0 < m <= SMALL_M_AUTO


class QuantizedC:
    """Where a decode GEMM also writes the MXFP8 re-quantization of its rounded output rows:
    ``values [M, total_cols]`` E4M3 (row pitch ``values.stride(0)``), ``scale_rows
    [M, total_cols / 32]`` and/or flat ``scale_mma`` atoms; this GEMM fills columns
    ``col0 .. col0 + N - 1`` of the ``total_cols``-wide matrix."""

    def __init__(self, values: torch.Tensor, scale_rows: torch.Tensor | None,
                 scale_mma: torch.Tensor | None, col0: int = 0, total_cols: int | None = None):
        self.values, self.scale_rows, self.scale_mma = values, scale_rows, scale_mma
        self.col0 = int(col0)
        self.total_cols = int(values.shape[-1] if total_cols is None else total_cols)


def _epilogue(c: torch.Tensor, n: int, bias: torch.Tensor | None,
              quantized_c: QuantizedC | None):
    """ctypes ``Epilogue`` (or None) after the checks only the host can make."""
    if bias is None and quantized_c is None:
        return None
    ep = _native.Epilogue()
    if bias is not None:
        _require_cuda("bias", bias)
        if bias.dtype != c.dtype or bias.ndim != 1 or bias.shape[0] != n or bias.stride(0) != 1:
            raise ValueError(f"a fused bias must be a contiguous [{n}] tensor of the output dtype "
                             f"{c.dtype}, got {bias.dtype} {tuple(bias.shape)}")
        ep.bias = bias.data_ptr()
    if quantized_c is not None:
        q = quantized_c
        _require_cuda("quantized-C values", q.values)
        if q.values.element_size() != 1 or q.values.stride(-1) != 1:
            raise ValueError("quantized-C values must be one-byte elements with unit column stride")
        ep.quant_values = q.values.data_ptr()
        ep.quant_scale_rows = q.scale_rows.data_ptr() if q.scale_rows is not None else None
        ep.quant_scale_mma = q.scale_mma.data_ptr() if q.scale_mma is not None else None
        ep.quant_ld = q.values.stride(0) if q.values.ndim > 1 and q.values.shape[0] > 1 else q.total_cols
        ep.quant_col0 = q.col0
        ep.quant_cols = q.total_cols
    return ep


def gemm_blockscaled(kind: int, a: torch.Tensor, sfa: torch.Tensor | None, b: torch.Tensor,
                     sfb: torch.Tensor | None, c: torch.Tensor, alpha: torch.Tensor | None,
                     m: int, n: int, k: int, *, ldc: int | None = None, block_n: int = 0,
                     sm_count: int = 0, stream_int: int | None = None,
                     small_m: bool | None = None, bias: torch.Tensor | None = None,
                     quantized_c: QuantizedC | None = None, groups: int = 1) -> None:
    """``c[M, ldc] = cvt(alpha * (a . sfa)(b . sfb)^T)``. ``a``/``b`` are row pointers to K-major
    code matrices, ``sfa``/``sfb`` point at the first scale atom. With ``groups > 1`` the
    tensors hold that many problems of the same shape group after group (operands ``[L, rows,
    K]``, each group's dense scale atoms, outputs ``[L, M, ldc]``) and all of them run in one
    launch.

    Decode shapes (see :func:`route_to_decode_kernel`; never when a tile width is forced, always
    with ``small_m=True``) go to the weight-streaming stream-K kernel, everything else to the
    persistent tiled kernels; ``block_n=_native.BLOCK_N_PAIR`` forces the CTA-pair kernel."""
    plain = kind == _native.KIND_FP8      # no block scales: sfa / sfb are not read
    for name, t in (("a", a), ("b", b), ("c", c)) + (() if plain else (("sfa", sfa), ("sfb", sfb))):
        _require_cuda(name, t)
    if c.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported output dtype {c.dtype}")
    dev = a.device
    ep = _epilogue(c, n, bias, quantized_c)
    if plain:
        if small_m or quantized_c is not None:
            raise ValueError("the unscaled FP8 recipe runs on the tiled kernels only")
        small_m = False
    if small_m is None:
        small_m = block_n == 0 and 0 < m <= SMALL_M_MAX and (
            quantized_c is not None or route_to_decode_kernel(m, n, dev, sm_count))
    lib = _native.load()
    decode = bool(small_m and 0 < m <= SMALL_M_MAX and n > 0)
    with torch.cuda.device(dev):
        # Decode kernel: counters and partial tiles. Tiled kernels: scratch for the CTA-pair
        # kernel's split leftover tiles (0 when the shape has none).
        need = int(lib.b12x_b200_gemm_grouped_workspace_bytes(
            kind, int(decode), m, n, k, groups, 0 if decode else block_n, sm_count))
    if need < 0:
        raise _native.NativeLibraryError(f"no kernel plan for M={m}, N={n}, K={k}, groups={groups}")
    work = stream_workspace(need, dev, stream_int) if need > 0 else None
    common_tail = (work.data_ptr() if work is not None else None,
                   work.numel() if work is not None else 0,
                   ctypes.byref(ep) if ep is not None else None)
    head = (kind, a.data_ptr(), None if plain else sfa.data_ptr(), b.data_ptr(),
            None if plain else sfb.data_ptr(), c.data_ptr(),
            _DTYPE_CODE[c.dtype], alpha.data_ptr() if alpha is not None else None,
            m, n, k, ldc if ldc is not None else n, groups)
    with torch.cuda.device(dev):
        if decode:
            rc = lib.b12x_b200_gemm_blockscaled_smallm_grouped(
                *head, *common_tail, sm_count, status_buffer(dev).data_ptr(),
                _stream_ptr(stream_int, dev))
        else:
            rc = lib.b12x_b200_gemm_blockscaled_grouped(
                *head, block_n, sm_count, *common_tail, status_buffer(dev).data_ptr(),
                _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_gemm_blockscaled_smallm_grouped" if decode
                  else "b12x_b200_gemm_blockscaled_grouped")
    _after_launch(dev)


def gemm_smallm_fused_quant(kind: int, x: torch.Tensor, global_scale: torch.Tensor | None,
                            w: torch.Tensor, sfw: torch.Tensor, c: torch.Tensor,
                            alpha: torch.Tensor | None, m: int, n: int, k: int, *,
                            ldc: int | None = None, sm_count: int = 0,
                            stream_int: int | None = None, bias: torch.Tensor | None = None,
                            quantized_c: QuantizedC | None = None, groups: int = 1,
                            inv_rope: tuple | None = None) -> None:
    """Decode GEMM that quantizes its BF16 activation rows ``x [M, K]`` (M <= 16) inside the
    kernel; bit for bit ``quantize rows`` followed by :func:`gemm_blockscaled`. With
    ``groups > 1``: ``x [M, groups, K]``, weights / scale atoms / output group-major, one
    launch. ``inv_rope = (positions, cos_sin_cache, head_dim, nope_dim, rope_dim)`` (MXFP8
    only) rotates the rotary part of every head back before the rows are quantized."""
    for name, t in (("x", x), ("w", w), ("sfw", sfw), ("c", c)):
        _require_cuda(name, t)
    if x.dtype != torch.bfloat16 or x.stride(-1) != 1:
        raise ValueError("fused activation quantization needs BF16 rows with unit column stride")
    if c.dtype not in _DTYPE_CODE:
        raise TypeError(f"unsupported output dtype {c.dtype}")
    dev = x.device
    ep = _epilogue(c, n, bias, quantized_c)
    if groups == 1:
        work = smallm_workspace(kind, m, n, k, dev, sm_count, stream_int)
        row_stride, group_stride = (x.stride(0) if m > 1 else k), 0
    else:
        # x is [M, groups, K]: rows `x.stride(0)` apart, groups `x.stride(1)` apart.
        with torch.cuda.device(dev):
            need = int(_native.load().b12x_b200_gemm_grouped_workspace_bytes(
                kind, 1, m, n, k, groups, 0, sm_count))
        if need < 0:
            raise _native.NativeLibraryError(
                f"no decode-shape plan for M={m}, N={n}, K={k}, groups={groups}")
        work = stream_workspace(need, dev, stream_int)
        row_stride, group_stride = (x.stride(0) if m > 1 else groups * k), x.stride(1)
    if inv_rope is not None:
        positions, cache, head_dim, nope_dim, rope_dim = inv_rope
        _require_cuda("positions", positions)
        _require_cuda("cos_sin_cache", cache)
        if kind != _native.KIND_MXFP8 or ep is not None:
            raise ValueError("the inverse-RoPE prologue exists for MXFP8 without epilogue only")
        with torch.cuda.device(dev):
            rc = _native.load().b12x_b200_gemm_smallm_fused_quant_grouped_inv_rope(
                x.data_ptr(), row_stride, group_stride, positions.data_ptr(),
                1 if positions.dtype == torch.int64 else 0, cache.data_ptr(),
                1 if cache.dtype == torch.float32 else 0, head_dim, nope_dim, rope_dim,
                w.data_ptr(), sfw.data_ptr(), c.data_ptr(), _DTYPE_CODE[c.dtype],
                alpha.data_ptr() if alpha is not None else None, m, n, k,
                ldc if ldc is not None else n, groups, work.data_ptr(), work.numel(), sm_count,
                status_buffer(dev).data_ptr(), _stream_ptr(stream_int, dev))
        _native.check(rc, "b12x_b200_gemm_smallm_fused_quant_grouped_inv_rope")
        _after_launch(dev)
        return
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_gemm_smallm_fused_quant_grouped(
            kind, x.data_ptr(), row_stride, group_stride,
            global_scale.data_ptr() if global_scale is not None else None, w.data_ptr(),
            sfw.data_ptr(), c.data_ptr(), _DTYPE_CODE[c.dtype],
            alpha.data_ptr() if alpha is not None else None, m, n, k,
            ldc if ldc is not None else n, groups, work.data_ptr(), work.numel(),
            ctypes.byref(ep) if ep is not None else None, sm_count,
            status_buffer(dev).data_ptr(), _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_gemm_smallm_fused_quant_grouped")
    _after_launch(dev)


def gemm_smallm_timeline(kind: int, a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor,
                         sfb: torch.Tensor, c: torch.Tensor, alpha: torch.Tensor | None,
                         m: int, n: int, k: int, stamps: torch.Tensor, *,
                         stream_int: int | None = None) -> None:
    """Decode GEMM that also writes its per-CTA time stamps into ``stamps`` (int64, 8 per SM)."""
    dev = a.device
    work = smallm_workspace(kind, m, n, k, dev, 0, stream_int)
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_gemm_smallm_timeline(
            kind, a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), c.data_ptr(),
            _DTYPE_CODE[c.dtype], alpha.data_ptr() if alpha is not None else None, m, n, k, n,
            work.data_ptr(), work.numel(), 0, stamps.data_ptr(), stamps.numel(),
            status_buffer(dev).data_ptr(), _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_gemm_smallm_timeline")


def selftest_wait_timeout(device: torch.device, max_polls: int = 4096) -> None:
    """Launch the library's wait self-test: one warp gives up a bounded wait and raises the
    device's status word like a GEMM kernel would (see :func:`check_kernel_status`)."""
    with torch.cuda.device(device):
        rc = _native.load().b12x_b200_selftest_wait_timeout(
            status_buffer(device).data_ptr(), max_polls, _stream_ptr(None, device))
    _native.check(rc, "b12x_b200_selftest_wait_timeout")


def gemm_block_fp8(a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor, sfb: torch.Tensor,
                   c: torch.Tensor, alpha: torch.Tensor | None, m: int, n: int, k: int, *,
                   ldc: int | None = None, sm_count: int = 0,
                   stream_int: int | None = None, bias: torch.Tensor | None = None) -> None:
    """E4M3 operands with FP32 scales ``sfa [M, K/128]`` / ``sfb [N/128, K/128]``."""
    for name, t in (("a", a), ("b", b), ("sfa", sfa), ("sfb", sfb), ("c", c)):
        _require_cuda(name, t)
    dev = a.device
    ep = _epilogue(c, n, bias, None)
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_gemm_block_fp8_ex(
            a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), c.data_ptr(),
            _DTYPE_CODE[c.dtype], alpha.data_ptr() if alpha is not None else None, m, n, k,
            ldc if ldc is not None else n, sm_count, ctypes.byref(ep) if ep is not None else None,
            status_buffer(dev).data_ptr(), _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_gemm_block_fp8_ex")
    _after_launch(dev)


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


def gemm_blockscaled_scatter(kind: int, a: torch.Tensor, sfa: torch.Tensor | None, b: torch.Tensor,
                             sfb: torch.Tensor | None, destination_ptrs: list[int], rank: int,
                             dtype: torch.dtype, alpha: torch.Tensor | None, m: int, n: int, k: int,
                             *, ld: int | None = None, sm_count: int = 0,
                             stream_int: int | None = None) -> None:
    """The CTA-pair GEMM with its output scattered by row slab over ``destination_ptrs`` (every
    rank's ``[M, ld]`` receive buffer as mapped in this process): this rank's partial of slab
    ``s`` lands in slot ``rank`` of destination ``s``. ``M % (256 * world) == 0``."""
    plain = kind == _native.KIND_FP8
    for name, t in (("a", a), ("b", b)) + (() if plain else (("sfa", sfa), ("sfb", sfb))):
        _require_cuda(name, t)
    dev = a.device
    world = len(destination_ptrs)
    lib = _native.load()
    with torch.cuda.device(dev):
        need = int(lib.b12x_b200_gemm_grouped_workspace_bytes(kind, 0, m, n, k, 1,
                                                              _native.BLOCK_N_PAIR, sm_count))
    work = stream_workspace(need, dev, stream_int) if need > 0 else None
    dsts = (ctypes.c_void_p * world)(*destination_ptrs)
    with torch.cuda.device(dev):
        rc = lib.b12x_b200_gemm_blockscaled_scatter(
            kind, a.data_ptr(), None if plain else sfa.data_ptr(), b.data_ptr(),
            None if plain else sfb.data_ptr(), dsts, world, rank,
            _DTYPE_CODE[dtype], alpha.data_ptr() if alpha is not None else None, m, n, k,
            ld if ld is not None else n, sm_count, work.data_ptr() if work is not None else None,
            work.numel() if work is not None else 0, status_buffer(dev).data_ptr(),
            _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_gemm_blockscaled_scatter")
    _after_launch(dev)


def pack_block_fp8_weight_mxfp8(codes: torch.Tensor, scale: torch.Tensor, out_codes: torch.Tensor,
                                scale_rows: torch.Tensor | None, scale_mma: torch.Tensor | None,
                                m: int, k: int, groups: int, requantize: bool, *,
                                stream_int: int | None = None) -> None:
    """Block-scaled FP8 checkpoint weight ``[groups, M, K]`` + FP32 128x128 block scales ->
    MXFP8 codes, row-major UE8M0 bytes and scale atoms (one launch, load time)."""
    for name, t in (("codes", codes), ("scale", scale), ("out_codes", out_codes)):
        _require_cuda(name, t)
    if scale.dtype != torch.float32 or not scale.is_contiguous():
        raise ValueError("block scales must be contiguous float32")
    dev = codes.device
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_pack_block_fp8_weight_mxfp8(
            codes.data_ptr(), scale.data_ptr(), out_codes.data_ptr(),
            scale_rows.data_ptr() if scale_rows is not None else None,
            scale_mma.data_ptr() if scale_mma is not None else None, m, k, groups,
            1 if requantize else 0, _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_pack_block_fp8_weight_mxfp8")


def bmm_mxfp8(a: torch.Tensor, w_values: torch.Tensor, w_scales: torch.Tensor, out: torch.Tensor,
              *, n_major: bool, batch: int, m: int, n: int, k: int,
              stream_int: int | None = None) -> None:
    """``out[b] = a[b] @ dequant(w[b])``: BF16 ``a [B, M, K]`` (M <= 32), rowwise-MXFP8 weights
    (``[B, N, K]`` K-major or ``[B, K, N]`` N-major, one UE8M0 byte per 32 codes of the inner
    axis), BF16 ``out [B, M, N]``. The tensors may be strided views; inner axes are contiguous."""
    for name, t in (("a", a), ("w_values", w_values), ("w_scales", w_scales), ("out", out)):
        _require_cuda(name, t)
    dev = a.device
    with torch.cuda.device(dev):
        rc = _native.load().b12x_b200_bmm_mxfp8(
            a.data_ptr(), a.stride(0), a.stride(1),
            w_values.data_ptr(), w_values.stride(0), w_values.stride(1),
            w_scales.data_ptr(), w_scales.stride(0), w_scales.stride(1),
            out.data_ptr(), out.stride(0), out.stride(1), 1 if n_major else 0,
            batch, m, n, k, _stream_ptr(stream_int, dev))
    _native.check(rc, "b12x_b200_bmm_mxfp8")


def allreduce_peer_signal_bytes() -> int:
    return int(_native.load().b12x_b200_allreduce_peer_signal_bytes())


def allreduce_peer(buffer_ptrs: list[int], signal_ptrs: list[int], rank: int, dtype: torch.dtype,
                   rows: int, cols: int, ld: int, device: torch.device, *, blocks: int = 0,
                   max_polls: int = 0, stream_int: int | None = None,
                   output_ptrs: list[int] | None = None) -> None:
    """Sum of all ranks' ``[rows, ld]`` partials over peer memory. ``buffer_ptrs`` /
    ``signal_ptrs``: every rank's buffer and signal block as mapped in this process. Without
    ``output_ptrs`` every rank's buffer holds its whole partial and receives the sum in place;
    with them the buffers hold scattered partials (see :func:`gemm_blockscaled_scatter`) and the
    sum goes to every rank's output. ``rank = -1`` rehearses all ranks in one grid on ``device``
    (tests)."""
    world = len(buffer_ptrs)
    if len(signal_ptrs) != world or (output_ptrs is not None and len(output_ptrs) != world):
        raise ValueError("one signal block (and one output) per buffer")
    bufs = (ctypes.c_void_p * world)(*buffer_ptrs)
    sigs = (ctypes.c_void_p * world)(*signal_ptrs)
    tail = (world, rank, _DTYPE_CODE[dtype], rows, cols, ld, blocks, max_polls)
    with torch.cuda.device(device):
        if output_ptrs is None:
            name = "b12x_b200_allreduce_peer"
            rc = _native.load().b12x_b200_allreduce_peer(
                bufs, sigs, *tail, status_buffer(device).data_ptr(), _stream_ptr(stream_int, device))
        else:
            name = "b12x_b200_allreduce_peer_scattered"
            outs = (ctypes.c_void_p * world)(*output_ptrs)
            rc = _native.load().b12x_b200_allreduce_peer_scattered(
                bufs, outs, sigs, *tail, status_buffer(device).data_ptr(),
                _stream_ptr(stream_int, device))
    _native.check(rc, name)
    _after_launch(device)


__all__ = [
    "allreduce_peer", "allreduce_peer_signal_bytes", "pack_block_fp8_weight_mxfp8", "gemm_blockscaled_scatter", "cuda_stream_to_int", "status_buffer", "check_kernel_status", "gemm_blockscaled", "QuantizedC",
    "gemm_block_fp8", "gemm_smallm_fused_quant", "gemm_smallm_timeline", "selftest_wait_timeout",
    "route_to_decode_kernel", "smallm_workspace", "stream_workspace", "quantize_mxfp8_rows",
    "quantize_nvfp4_rows",
    "KERNEL_STATUS_TEXT",
]
