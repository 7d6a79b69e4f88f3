"""Dense block-scaled GEMM entry points: ``C = cvt(alpha * (A . SFA) @ (B . SFB)^T)``.

Drop-in for the reference's ``dense_gemm`` / ``dense_gemm_fused_quant_a`` and the torch
custom ops ``b12x::dense_gemm_launch`` / ``b12x::dense_gemm_launch_functional``
(b12x/_lib/dense_gemm.py:7068-7777, 6897-7051, 6335-6373, 6494-6532). Same names, argument
meaning and host-side errors; the device work is the sm_100a tcgen05 kernel behind the C
ABI. Tuning keywords of the reference's SM120 kernel (``load_path``, ``swap_ab``,
``cluster_shape_mn``, ``sfb_k_replicated``, the policy booleans of the custom ops) are
accepted and ignored; ``mma_tiler_mn`` selects a kernel when it names a tile one of them has:
``(128, 64/128/192/256)`` the single-CTA kernel with that tile width, ``(256, 256)`` the
CTA-pair kernel.

Operand contract (same as the reference): ``lhs = (A[M, Kp, L], SFA)``, ``rhs = (B[N, Kp, L],
SFB)``, K-major, ``Kp = K/2`` bytes for ``float4_e2m1fn`` (two codes per byte, low nibble
first) or ``K`` for ``float8_e4m3fn``; the scale tensors are the 6-D MMA views
``(32, 4, row_tiles, 4, k_tiles, L)`` over dense atom storage. Output is ``[M, N, L]`` backed by
physical ``[L, M, N]`` storage.
"""

from __future__ import annotations

import os
import logging
import time
from typing import Literal, Optional, Tuple

import torch

from .. import _native
from . import launch
from .launch import cuda_stream_to_int
from .layout import mma_view_is_canonical

logger = logging.getLogger(__name__)
_B12X_TIMING = os.getenv("B12X_TIMING", "0") == "1"
_B12X_TIMING_THRESHOLD_MS = float(os.getenv("B12X_TIMING_THRESHOLD_MS", "0"))

_DENSE_LOAD_PATHS = ("tma", "cpasync")
_AB_DTYPES = ("float4_e2m1fn", "float8_e4m3fn")
_MXFP6_AB_DTYPES = ("float6_e3m2fn", "float6_e2m3fn")
_C_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}
_KERNEL_BLOCK_N = (64, 128, 192, 256)
_ALPHA_ONE_CACHE: dict[tuple[str, int | None], torch.Tensor] = {}


def get_num_sm(device: torch.device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def _cached_alpha_one(device: torch.device | str) -> torch.Tensor:
    """Per-device FP32 one, so the default-alpha path allocates only on first use."""
    resolved = torch.device(device)
    if resolved.type == "cuda" and resolved.index is None:
        resolved = torch.device("cuda", torch.cuda.current_device())
    key = (resolved.type, resolved.index)
    alpha = _ALPHA_ONE_CACHE.get(key)
    if alpha is None:
        alpha = torch.ones((1,), dtype=torch.float32, device=resolved)
        _ALPHA_ONE_CACHE[key] = alpha
    return alpha


def _empty_dense_gemm_output(m: int, n: int, l: int, *, dtype: torch.dtype,
                             device: torch.device | str) -> torch.Tensor:
    """``[M, N, L]`` output in the layout the kernel writes: physical ``[L, M, N]``."""
    if l > 1:
        return torch.empty((l, m, n), dtype=dtype, device=device).as_strided(
            (m, n, l), (n, 1, m * n))
    return torch.empty((m, n, l), dtype=dtype, device=device)


def _kind_of(ab_dtype: str, sf_dtype: str, sf_vec_size: int) -> int:
    if ab_dtype == "float4_e2m1fn":
        if sf_dtype == "float8_e4m3fn" and sf_vec_size == 16:
            return _native.KIND_NVFP4
        if sf_dtype == "float8_e8m0fnu" and sf_vec_size == 32:
            return _native.KIND_MXFP4
        raise ValueError(
            "float4_e2m1fn operands need sf_dtype='float8_e4m3fn' with sf_vec_size=16 (NVFP4) or "
            f"sf_dtype='float8_e8m0fnu' with sf_vec_size=32 (MXFP4); got sf_dtype={sf_dtype!r}, "
            f"sf_vec_size={sf_vec_size}")
    if sf_dtype == "float8_e8m0fnu" and sf_vec_size == 32:
        return _native.KIND_MXFP8
    raise ValueError(
        "float8_e4m3fn operands need sf_dtype='float8_e8m0fnu' with sf_vec_size=32 "
        f"(or block_fp8=True); got sf_dtype={sf_dtype!r}, sf_vec_size={sf_vec_size}")


def _check_operand(name: str, t: torch.Tensor, rows: int, row_bytes: int, l: int) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be on CUDA")
    if t.element_size() != 1:
        raise TypeError(f"{name} must hold one byte per element, got {t.dtype}")
    if tuple(t.shape) != (rows, row_bytes, l):
        raise ValueError(f"{name} must have shape {(rows, row_bytes, l)}, got {tuple(t.shape)}")
    want = (row_bytes, 1, rows * row_bytes)
    if any(t.shape[i] > 1 and t.stride(i) != want[i] for i in range(3)):
        raise ValueError(
            f"{name} must be K-major over physical [L, rows, K] storage (strides {want}), "
            f"got {t.stride()}")
    if t.data_ptr() % 16 != 0 or row_bytes % 16 != 0:
        raise ValueError(f"{name} rows must be 16-byte aligned")


def _dense_gemm_launch_flat(a, b, sfa, sfb, c, alpha, *, n: int, k: int, l: int, ab_dtype: str,
                            sf_dtype: str, sf_vec_size: int, mma_tile_n: int, sm_count: int,
                            alpha_is_one: bool, stream_int: Optional[int],
                            mma_tile_m: int = 128,
                            quantized_c: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None
                            ) -> None:
    kind = _kind_of(ab_dtype, sf_dtype, sf_vec_size)
    m = int(a.shape[0])
    row_bytes = k // 2 if kind in (_native.KIND_NVFP4, _native.KIND_MXFP4) else k
    _check_operand("A", a, m, row_bytes, l)
    _check_operand("B", b, n, row_bytes, l)
    if not mma_view_is_canonical(sfa, m, k, sf_vec_size, l):
        raise ValueError("SFA must be the (32,4,m_tiles,4,k_tiles,L) view over dense atom storage")
    if not mma_view_is_canonical(sfb, n, k, sf_vec_size, l):
        raise ValueError("SFB must be the (32,4,n_tiles,4,k_tiles,L) view over dense atom storage")
    if tuple(c.shape) != (m, n, l):
        raise ValueError(f"out must have shape {(m, n, l)}, got {tuple(c.shape)}")
    if c.stride(1) != 1 or (l > 1 and c.stride(2) != m * n) or (m > 1 and c.stride(0) < n):
        raise ValueError(f"out must be backed by physical [L, M, N] storage, got strides {c.stride()}")
    if alpha is not None and (alpha.dtype != torch.float32 or alpha.numel() != 1):
        raise ValueError("alpha must be a float32 tensor with one element")
    if m == 0 or n == 0:
        return
    block_n = mma_tile_n if mma_tile_n in _KERNEL_BLOCK_N else 0
    if mma_tile_m == 256 and mma_tile_n == 256:
        block_n = _native.BLOCK_N_PAIR
    k_tiles = -(-(-(-k // sf_vec_size)) // 4)
    sfa_group = (-(-m // 128)) * k_tiles * 512
    sfb_group = (-(-n // 128)) * k_tiles * 512
    sfa_flat = sfa.view(torch.uint8) if sfa.dtype != torch.uint8 else sfa
    sfb_flat = sfb.view(torch.uint8) if sfb.dtype != torch.uint8 else sfb
    sfa_base = torch.as_strided(sfa_flat, (l * sfa_group,), (1,))
    sfb_base = torch.as_strided(sfb_flat, (l * sfb_group,), (1,))
    ldc = c.stride(0) if m > 1 else n
    if l > 1 and ldc != n:
        raise ValueError("a grouped output must be dense [L, M, N] storage")
    # One launch for all L groups: the operands are physical [L, rows, K] stacks, and the tiles
    # of every group go into one work list on the device. Quantized C: group g fills columns
    # [g * N, (g + 1) * N) of the [M, N * L] MXFP8 matrix.
    qc = None if quantized_c is None else launch.QuantizedC(
        quantized_c[0], quantized_c[1], quantized_c[2], col0=0, total_cols=n * l)
    launch.gemm_blockscaled(
        kind, a, sfa_base, b, sfb_base, c, None if alpha_is_one else alpha, m, n, k, ldc=ldc,
        block_n=block_n, sm_count=sm_count, stream_int=stream_int, quantized_c=qc, groups=l)


@torch.library.custom_op("b12x::dense_gemm_launch", mutates_args=("c_tensor_gpu",))
def _dense_gemm_launch_op(
    a_tensor_gpu: torch.Tensor, b_tensor_gpu: torch.Tensor, sfa_tensor_gpu: torch.Tensor,
    sfb_tensor_gpu: torch.Tensor, c_tensor_gpu: torch.Tensor, alpha_tensor_gpu: torch.Tensor,
    n: int, k: int, l: int, c_l: int, ab_dtype: str, sf_dtype: str, c_dtype: str,
    alpha_dtype: str, sf_vec_size: int, mma_k: int, tile_k: int, mma_tile_m: int,
    mma_tile_n: int, cluster_shape_m: int, cluster_shape_n: int, sm_count: int,
    single_work_tile_per_cta: bool, direct_one_m_tile_scheduler: bool, use_m1_non_tma: bool,
    split_k_slices: int, split_k_atomic_bf16: bool, large_m_unroll: bool, load_path: str,
    swap_ab: bool, sfb_k_reuse: bool, alpha_is_one: bool, stream_int: Optional[int],
) -> None:
    _dense_gemm_launch_flat(
        a_tensor_gpu, b_tensor_gpu, sfa_tensor_gpu, sfb_tensor_gpu, c_tensor_gpu,
        alpha_tensor_gpu, n=n, k=k, l=l, ab_dtype=ab_dtype, sf_dtype=sf_dtype,
        sf_vec_size=sf_vec_size, mma_tile_n=mma_tile_n, sm_count=sm_count,
        alpha_is_one=alpha_is_one, stream_int=stream_int, mma_tile_m=mma_tile_m)


@_dense_gemm_launch_op.register_fake
def _dense_gemm_launch_fake(*args, **kwargs) -> None:
    return None


@torch.library.custom_op("b12x::dense_gemm_launch_functional", mutates_args=())
def _dense_gemm_launch_functional_op(
    a_tensor_gpu: torch.Tensor, b_tensor_gpu: torch.Tensor, sfa_tensor_gpu: torch.Tensor,
    sfb_tensor_gpu: torch.Tensor, alpha_tensor_gpu: torch.Tensor, n: int, k: int, l: int,
    kernel_c_l: int, ab_dtype: str, sf_dtype: str, c_dtype: str, kernel_c_dtype: str,
    alpha_dtype: str, sf_vec_size: int, mma_k: int, tile_k: int, mma_tile_m: int,
    mma_tile_n: int, cluster_shape_m: int, cluster_shape_n: int, sm_count: int,
    single_work_tile_per_cta: bool, direct_one_m_tile_scheduler: bool, use_m1_non_tma: bool,
    split_k_slices: int, split_k_atomic_bf16: bool, large_m_unroll: bool, load_path: str,
    swap_ab: bool, sfb_k_reuse: bool, alpha_is_one: bool, stream_int: Optional[int],
) -> torch.Tensor:
    m = int(a_tensor_gpu.shape[0])
    out = _empty_dense_gemm_output(m, n, l, dtype=_C_DTYPES[c_dtype], device=a_tensor_gpu.device)
    _dense_gemm_launch_flat(
        a_tensor_gpu, b_tensor_gpu, sfa_tensor_gpu, sfb_tensor_gpu, out, alpha_tensor_gpu,
        n=n, k=k, l=l, ab_dtype=ab_dtype, sf_dtype=sf_dtype, sf_vec_size=sf_vec_size,
        mma_tile_n=mma_tile_n, sm_count=sm_count, alpha_is_one=alpha_is_one,
        stream_int=stream_int, mma_tile_m=mma_tile_m)
    return out


@_dense_gemm_launch_functional_op.register_fake
def _dense_gemm_launch_functional_fake(
    a_tensor_gpu, b_tensor_gpu, sfa_tensor_gpu, sfb_tensor_gpu, alpha_tensor_gpu, n, k, l,
    kernel_c_l, ab_dtype, sf_dtype, c_dtype, *rest,
) -> torch.Tensor:
    return _empty_dense_gemm_output(a_tensor_gpu.shape[0], n, l, dtype=_C_DTYPES[c_dtype],
                                    device=a_tensor_gpu.device)


def _select_default_mma_tiler_mn(m: int, n: int, sm_count: int) -> Tuple[int, int]:
    """Tile the kernel would pick for (m, n) on ``sm_count`` SMs: 128 rows by the width with
    the fewest waves x per-tile cost (same model as the C side)."""
    best, best_cost = 128, None
    tiles_m = -(-m // 128)
    for bn in (256, 192, 128, 64):
        waves = -(-(tiles_m * -(-n // bn)) // max(sm_count, 1))
        cost = waves * (128 + bn)
        if best_cost is None or cost < best_cost:
            best, best_cost = bn, cost
    return (128, best)


_UNIT_SCALE_CACHE: dict = {}


def _plain_fp8_launch(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor],
                      alpha: Optional[torch.Tensor], *, m: int, n: int, k: int, l: int,
                      c_dtype: str, mma_tiler_mn, sm_count: int, stream) -> torch.Tensor:
    """``dense_gemm(plain_fp8=True)`` on the tiled kernels: E4M3 x E4M3 with FP32 accumulation
    and ``alpha`` as the only scale (b12x/_lib/dense_gemm.py:7096-7139, 7225-7233; MMA :268-330 in the reference)."""
    _check_operand("A", a, m, k, l)
    _check_operand("B", b, n, k, l)
    if out is None:
        out = _empty_dense_gemm_output(m, n, l, dtype=_C_DTYPES[c_dtype], device=a.device)
    elif out.dtype != _C_DTYPES[c_dtype]:
        raise ValueError(f"out dtype {out.dtype} does not match c_dtype={c_dtype!r}")
    if tuple(out.shape) != (m, n, l):
        raise ValueError(f"out must have shape {(m, n, l)}, got {tuple(out.shape)}")
    if out.stride(1) != 1 or (l > 1 and out.stride(2) != m * n) or (m > 1 and out.stride(0) < n):
        raise ValueError(f"out must be backed by physical [L, M, N] storage, got strides {out.stride()}")
    if alpha is not None and (alpha.dtype != torch.float32 or alpha.numel() != 1):
        raise ValueError("alpha must be a float32 tensor with one element")
    if m == 0 or n == 0:
        return out
    block_n = 0
    if mma_tiler_mn is not None:
        tile_m, tile_n = int(mma_tiler_mn[0]), int(mma_tiler_mn[1])
        block_n = _native.BLOCK_N_PAIR if (tile_m, tile_n) == (256, 256) else (
            tile_n if tile_n in _KERNEL_BLOCK_N else 0)
    ldc = out.stride(0) if m > 1 else n
    if l > 1 and ldc != n:
        raise ValueError("a grouped output must be dense [L, M, N] storage")
    launch.gemm_blockscaled(_native.KIND_FP8, a, None, b, None, out, alpha, m, n, k, ldc=ldc,
                            block_n=block_n, sm_count=sm_count,
                            stream_int=cuda_stream_to_int(stream), groups=l)
    return out


def _unit_mxfp8_scales(device: torch.device, rows: int, k: int, groups: int) -> torch.Tensor:
    """Cached MMA-layout scale view with every UE8M0 byte at 127 (2^0), for plain FP8."""
    from .mxfp8_rows import pack_mxfp8_scales_for_dense_gemm

    key = (device.type, device.index, int(rows), int(k), int(groups))
    view = _UNIT_SCALE_CACHE.get(key)
    if view is None:
        ones = torch.full((groups, rows, k // 32), 127, dtype=torch.uint8, device=device)
        view = pack_mxfp8_scales_for_dense_gemm(ones, m=rows, k=k, num_groups=groups)
        _UNIT_SCALE_CACHE[key] = view
    return view


def dense_gemm(
    lhs: Tuple[torch.Tensor, torch.Tensor],
    rhs: Tuple[torch.Tensor, torch.Tensor],
    out: Optional[torch.Tensor] = None,
    *,
    ab_dtype: str,
    sf_dtype: str,
    c_dtype: str,
    sf_vec_size: int,
    sm_count: Optional[int] = None,
    mma_tiler_mn: Optional[Tuple[int, int]] = None,
    cluster_shape_mn: Tuple[int, int] = (1, 1),
    alpha: Optional[torch.Tensor] = None,
    alpha_dtype: Optional[str] = None,
    expected_m: Optional[int] = None,
    load_path: Optional[Literal["tma", "cpasync"]] = None,
    swap_ab: Optional[bool] = None,
    sfb_k_replicated: bool = False,
    rhs_values_tiled: Optional[torch.Tensor] = None,
    _quantized_c: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
    stream: object = None,
    a_preexpanded: bool = False,
    b_preexpanded: bool = False,
    b_packed: bool = False,
    a_fmt: Optional[str] = None,
    b_fmt: Optional[str] = None,
    x_bf16: Optional[torch.Tensor] = None,
    w_gscale: Optional[torch.Tensor] = None,
    plain_fp8: bool = False,
    block_fp8: bool = False,
) -> torch.Tensor:
    """Dense block-scaled GEMM for one batch stack; see the module docstring for layouts.

    ``expected_m`` is a regime hint in the reference; the sm_100a kernel chooses its tile from
    the live shape, so the hint is accepted and unused. ``alpha`` is a device FP32 scalar
    read by the kernel at run time (CUDA-graph replays see updated values).
    """
    a_torch, sfa_torch = lhs
    b_torch, sfb_torch = rhs
    if load_path is not None and load_path not in _DENSE_LOAD_PATHS:
        raise ValueError(
            f"dense_gemm load_path must be one of {_DENSE_LOAD_PATHS}, got {load_path!r}")
    if b_packed and b_preexpanded:
        raise ValueError("b_packed and b_preexpanded are mutually exclusive")
    if ab_dtype in _MXFP6_AB_DTYPES:
        raise NotImplementedError("MX-FP6 operands are outside the block-scaled GEMM path built here")
    if ab_dtype not in _AB_DTYPES:
        raise TypeError(f"dense_gemm unsupported ab_dtype: {ab_dtype}")
    if (a_preexpanded or b_preexpanded or b_packed or a_fmt is not None or b_fmt is not None
            or x_bf16 is not None or w_gscale is not None):
        raise ValueError(
            "a_preexpanded/b_preexpanded/a_fmt/b_fmt/x_bf16/w_gscale are only "
            f"supported with an MX-FP6 ab_dtype, got ab_dtype={ab_dtype!r}")
    if rhs_values_tiled is not None:
        raise NotImplementedError("a tile-major RHS belongs to the WO projection path")
    if c_dtype not in _C_DTYPES:
        raise KeyError(f"unsupported c_dtype string: {c_dtype!r}")

    m, k, l = a_torch.shape
    n = b_torch.shape[0]
    if ab_dtype == "float4_e2m1fn":
        k *= 2
        mma_k = 64
    else:
        mma_k = 32
    if sm_count is None:
        sm_count = get_num_sm(a_torch.device)
    if block_fp8:
        from .block_fp8_gemm import block_fp8_gemm

        return block_fp8_gemm(a_torch, sfa_torch, b_torch, sfb_torch, out, c_dtype=c_dtype,
                              sf_dtype=sf_dtype, sf_vec_size=sf_vec_size, alpha=alpha,
                              load_path=load_path, swap_ab=swap_ab,
                              sfb_k_replicated=sfb_k_replicated, sm_count=sm_count,
                              stream=stream)
    if plain_fp8 and (ab_dtype != "float8_e4m3fn" or sf_dtype != "float8_e8m0fnu"
                      or sf_vec_size != 32):
        # Per-tensor FP8 rides on the MXFP8 kernel: the caller passes unit block scales and
        # the one real scale as alpha (dense_gemm.py:7137-7139 in the reference).
        raise ValueError("plain_fp8 requires float8_e4m3fn operands with float8_e8m0fnu/32 scales")
    if plain_fp8 and (_quantized_c is not None or sfb_k_replicated):
        raise ValueError("plain_fp8 does not support tiled/quantized output or replicated scales")
    if plain_fp8:
        # The caller's scale storage is not read in this mode. Shapes of the tiled kernels run
        # the unscaled FP8 MMA (no scale bytes move at all); decode shapes stay on the
        # weight-streaming kernel, which is written for block scales, with every scale 2^0
        # (1/32 of the weight bytes on top).
        forced = mma_tiler_mn is not None and int(mma_tiler_mn[1]) in _KERNEL_BLOCK_N
        if _quantized_c is None and (forced or not launch.route_to_decode_kernel(
                m, n, a_torch.device, int(sm_count))):
            return _plain_fp8_launch(a_torch, b_torch, out, alpha, m=m, n=n, k=k, l=l,
                                     c_dtype=c_dtype, mma_tiler_mn=mma_tiler_mn,
                                     sm_count=int(sm_count), stream=stream)
        sfa_torch = _unit_mxfp8_scales(a_torch.device, m, k, l)
        sfb_torch = _unit_mxfp8_scales(a_torch.device, n, k, l)
    _kind_of(ab_dtype, sf_dtype, sf_vec_size)
    if mma_tiler_mn is None:
        # Tile width 0 in the op arguments means "the launcher chooses": the persistent tiled
        # kernel picks its width from the live shape and decode shapes go to the
        # weight-streaming kernel. A caller-supplied tile forces the tiled kernel.
        mma_tiler_mn = (128, 0)
    if alpha_dtype is None:
        alpha_dtype = "float32" if alpha is None else str(alpha.dtype).split(".")[-1]
    alpha_is_one = alpha is None
    if alpha is None:
        alpha = _cached_alpha_one(a_torch.device)
    stream_int = cuda_stream_to_int(stream)
    if _quantized_c is not None:
        # The GEMM also emits the MXFP8 re-quantization of its BF16 output rows (the decode
        # kernel's epilogue does it): restricted, as in the reference, to the small-M layout its
        # WO-A projection uses (b12x/_lib/dense_gemm.py:7497-7588).
        q_values, q_scale_rows, q_scale_mma = _quantized_c
        width = n * l
        if (swap_ab or c_dtype != "bfloat16" or m < 1 or m > 16 or n % 32 != 0 or width % 128 != 0
                or block_fp8 or plain_fp8
                or tuple(q_values.shape) != (m, width) or not q_values.is_contiguous()
                or q_values.dtype != torch.float8_e4m3fn
                or tuple(q_scale_rows.shape) != (m, width // 32) or not q_scale_rows.is_contiguous()
                or q_scale_rows.dtype != torch.float8_e8m0fnu
                or tuple(q_scale_mma.shape) != (32, 4, 1, 4, width // 128, 1)
                or q_scale_mma.dtype != torch.float8_e8m0fnu):
            raise ValueError("quantized C is restricted to the BF16 WO-A decode layout")
        if out is None:
            out = _empty_dense_gemm_output(m, n, l, dtype=torch.bfloat16, device=a_torch.device)
        _dense_gemm_launch_flat(
            a_torch, b_torch, sfa_torch, sfb_torch, out, alpha, n=n, k=k, l=l, ab_dtype=ab_dtype,
            sf_dtype=sf_dtype, sf_vec_size=sf_vec_size, mma_tile_n=0, sm_count=int(sm_count),
            alpha_is_one=alpha_is_one, stream_int=stream_int,
            quantized_c=(q_values, q_scale_rows, q_scale_mma))
        return out
    op_tail = (
        alpha_dtype, sf_vec_size, mma_k, sf_vec_size * 8 if ab_dtype == "float4_e2m1fn" else 128,
        int(mma_tiler_mn[0]), int(mma_tiler_mn[1]), int(cluster_shape_mn[0]),
        int(cluster_shape_mn[1]), int(sm_count), False, False, False, 1, False, False,
        load_path or "tma", bool(swap_ab), bool(sfb_k_replicated), alpha_is_one, stream_int,
    )
    t0 = time.perf_counter() if _B12X_TIMING else 0.0
    if _direct_launch_ok(a_torch):
        # Plain eager call on real CUDA tensors: what the custom op's body would do, without the
        # dispatcher round trip of a 33-argument op (about half of the host time of a call).
        # Tracing (torch.compile), fake tensors and meta tensors go through the ops below.
        if out is None:
            out = _empty_dense_gemm_output(m, n, l, dtype=_C_DTYPES[c_dtype], device=a_torch.device)
        elif out.dtype != _C_DTYPES[c_dtype]:
            raise ValueError(f"out dtype {out.dtype} does not match c_dtype={c_dtype!r}")
        _dense_gemm_launch_flat(
            a_torch, b_torch, sfa_torch, sfb_torch, out, alpha, n=n, k=k, l=l, ab_dtype=ab_dtype,
            sf_dtype=sf_dtype, sf_vec_size=sf_vec_size, mma_tile_n=int(mma_tiler_mn[1]),
            sm_count=int(sm_count), alpha_is_one=alpha_is_one, stream_int=stream_int,
            mma_tile_m=int(mma_tiler_mn[0]))
    elif out is None:
        out = torch.ops.b12x.dense_gemm_launch_functional(
            a_torch, b_torch, sfa_torch, sfb_torch, alpha, n, k, l, l, ab_dtype, sf_dtype,
            c_dtype, c_dtype, *op_tail)
    else:
        if out.dtype != _C_DTYPES[c_dtype]:
            raise ValueError(f"out dtype {out.dtype} does not match c_dtype={c_dtype!r}")
        torch.ops.b12x.dense_gemm_launch(
            a_torch, b_torch, sfa_torch, sfb_torch, out, alpha, n, k, l, l, ab_dtype, sf_dtype,
            c_dtype, *op_tail)
    if _B12X_TIMING:
        ms = (time.perf_counter() - t0) * 1000.0
        if ms >= _B12X_TIMING_THRESHOLD_MS:
            logger.warning("b12x_dense_gemm timing m=%d n=%d k=%d l=%d enqueue=%.3fms",
                           m, n, k, l, ms)
    return out


_DIRECT_LAUNCH = os.environ.get("B12X_B200_DIRECT_LAUNCH", "1") != "0"


def _direct_launch_ok(t: torch.Tensor) -> bool:
    """True for an ordinary eager call: a real CUDA tensor, nothing tracing."""
    return (_DIRECT_LAUNCH and type(t) is torch.Tensor and t.is_cuda
            and not torch.compiler.is_compiling())


def _fused_quant_rhs(name: str, b: torch.Tensor, sfb: torch.Tensor, row_bytes: int):
    if b.ndim != 3 or int(b.shape[1]) != row_bytes or int(b.shape[2]) != 1:
        raise ValueError(f"B must have shape [N,{row_bytes},1], got {tuple(b.shape)}")
    if b.element_size() != 1 or b.stride(1) != 1 or b.stride(0) != row_bytes:
        raise ValueError(f"{name}: B must be K-major one-byte codes")
    return b.select(2, 0), (sfb.view(torch.uint8) if sfb.dtype != torch.uint8 else sfb)


def dense_gemm_fused_quant_a(
    source: torch.Tensor,
    b: torch.Tensor,
    sfb: torch.Tensor,
    *,
    out: Optional[torch.Tensor] = None,
    expected_m: Optional[int] = None,
    sfb_k_replicated: bool = False,
    rhs_values_tiled: Optional[torch.Tensor] = None,
    a_inner_span: int = 0,
    mma_tiler_mn: Optional[Tuple[int, int]] = None,
    _atomic_output_precleared: bool = False,
    stream: object = None,
) -> torch.Tensor:
    """Small-M BF16 activations -> MXFP8 GEMM in one kernel (b12x/_lib/dense_gemm.py:6897-7051).

    The decode kernel's quantizer warps turn the BF16 rows into E4M3 codes and UE8M0/32 scales
    inside shared memory while the weight streams in; nothing is written to global memory but
    the output. Results equal ``quantize_rows`` followed by ``mm`` bit for bit.
    """
    if source.dtype != torch.bfloat16:
        raise ValueError("fused MXFP8 activation quantization requires BF16 A")
    if int(a_inner_span) != 0 or rhs_values_tiled is not None:
        raise NotImplementedError("L-blocked A and tile-major RHS belong to the WO projection path")
    if source.ndim != 2 or not source.is_contiguous():
        raise ValueError("fused MXFP8 activation quantization requires contiguous BF16 [M,K]")
    m, k = map(int, source.shape)
    if m < 1 or m > 8 or k % 128 != 0:
        raise ValueError(
            f"fused MXFP8 activation quantization requires 1<=M<=8 and K%128=0, got M={m}, K={k}")
    w, sfw = _fused_quant_rhs("mm_fused_quant_a", b, sfb, k)
    n = int(b.shape[0])
    if out is None:
        if _atomic_output_precleared:
            raise ValueError("a precleared fused-quant output must be caller-owned")
        out = torch.empty((m, n, 1), dtype=torch.bfloat16, device=source.device)
    if out.shape != (m, n, 1) or out.dtype != torch.bfloat16:
        raise ValueError(
            f"out must be BF16 with shape {(m, n, 1)}, got {out.dtype} {tuple(out.shape)}")
    launch.gemm_smallm_fused_quant(_native.KIND_MXFP8, source, None, w, sfw, out.select(2, 0),
                                   None, m, n, k, ldc=n, stream_int=cuda_stream_to_int(stream))
    return out


def dense_gemm_fused_quant_a_grouped(
    source: torch.Tensor,
    b: torch.Tensor,
    sfb: torch.Tensor,
    *,
    groups: int,
    out: Optional[torch.Tensor] = None,
    positions: Optional[torch.Tensor] = None,
    cos_sin_cache: Optional[torch.Tensor] = None,
    head_dim: int = 0,
    nope_dim: int = 0,
    rope_dim: int = 0,
    expected_m: Optional[int] = None,
    sfb_k_replicated: bool = False,
    mma_tiler_mn: Optional[Tuple[int, int]] = None,
    stream: object = None,
) -> torch.Tensor:
    """Grouped small-M BF16 activations -> MXFP8 GEMM in ONE launch
    (b12x/_lib/dense_gemm.py:5803-5944, the WO-A shape): ``source [M, groups, K]`` BF16 (rows
    may be strided, ``[groups, K]`` contiguous inside a row), per group ``[M, K] x [N, K]^T``
    into ``out [M, N, groups]``. Every group's rows are quantized inside the decode kernel,
    bit for bit as ``quantize_rows`` would. With ``positions`` / ``cos_sin_cache`` the trailing
    ``rope_dim`` elements of every ``head_dim`` block of a row are inverse-RoPE-rotated in FP32
    before quantization (``:5849-5882``; interleaved pairs, ``cos = cache[pos, j]``,
    ``sin = cache[pos, rope_dim / 2 + j]``)."""
    if source.dtype != torch.bfloat16 or source.ndim != 3:
        raise ValueError("fused grouped MXFP8 quantization requires BF16 [M, groups, K]")
    m, k = int(source.shape[0]), int(source.shape[2])
    if int(source.shape[1]) != groups:
        raise ValueError(f"source groups {int(source.shape[1])} != weight groups {groups}")
    if source.stride(2) != 1 or source.stride(1) != k:
        raise ValueError(
            f"fused grouped MXFP8 A needs contiguous [groups, K] rows, got strides {source.stride()}")
    row_stride = int(source.stride(0))
    if m < 1 or m > 8 or k % 128 != 0 or row_stride % 8 != 0:
        raise ValueError(
            f"fused grouped MXFP8 quantization requires 1<=M<=8, K%128=0, row stride%8=0; "
            f"got M={m}, K={k}, row_stride={row_stride}")
    if b.ndim != 3 or int(b.shape[1]) != k or int(b.shape[2]) != groups:
        raise ValueError(f"B must have shape [N,{k},{groups}], got {tuple(b.shape)}")
    inv_rope = None
    if positions is not None or cos_sin_cache is not None:
        if positions is None or cos_sin_cache is None:
            raise ValueError("inverse-RoPE needs both positions and cos_sin_cache")
        if positions.shape != (m,):
            raise ValueError(f"positions must have shape {(m,)}, got {tuple(positions.shape)}")
        if not positions.is_contiguous() or not cos_sin_cache.is_contiguous():
            raise ValueError("positions and cos_sin_cache must be contiguous")
        if cos_sin_cache.ndim != 2 or int(cos_sin_cache.shape[1]) != rope_dim:
            raise ValueError(
                f"cos_sin_cache must have shape [max_pos, {rope_dim}], got {tuple(cos_sin_cache.shape)}")
        if (head_dim <= 0 or nope_dim + rope_dim != head_dim or head_dim % 32 or nope_dim % 32
                or rope_dim % 32 or k % head_dim):
            raise ValueError(
                "fused inverse-RoPE requires 32-aligned head_dim = nope_dim + rope_dim "
                f"dividing K, got head={head_dim}, nope={nope_dim}, rope={rope_dim}, K={k}")
        if positions.dtype not in (torch.int32, torch.int64):
            raise ValueError(f"fused inv-RoPE positions must be int32/int64, got {positions.dtype}")
        if cos_sin_cache.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(
                f"fused inv-RoPE cos/sin cache must be bf16/fp32, got {cos_sin_cache.dtype}")
        inv_rope = (positions, cos_sin_cache, int(head_dim), int(nope_dim), int(rope_dim))
    n = int(b.shape[0])
    _check_operand("B", b, n, k, groups)
    if not mma_view_is_canonical(sfb, n, k, 32, groups):
        raise ValueError("SFB must be the (32,4,n_tiles,4,k_tiles,L) view over dense atom storage")
    if out is None:
        out = _empty_dense_gemm_output(m, n, groups, dtype=torch.bfloat16, device=source.device)
    if out.shape != (m, n, groups) or out.dtype != torch.bfloat16:
        raise ValueError(
            f"out must be BF16 with shape {(m, n, groups)}, got {out.dtype} {tuple(out.shape)}")
    if out.stride(1) != 1 or (groups > 1 and out.stride(2) != m * n) or (m > 1 and out.stride(0) != n):
        raise ValueError(f"out must be backed by physical [L, M, N] storage, got strides {out.stride()}")
    sfb_flat = sfb.view(torch.uint8) if sfb.dtype != torch.uint8 else sfb
    launch.gemm_smallm_fused_quant(_native.KIND_MXFP8, source, None, b, sfb_flat, out, None, m, n, k,
                                   ldc=n, stream_int=cuda_stream_to_int(stream), groups=groups,
                                   inv_rope=inv_rope)
    return out


def dense_gemm_fused_quant_a_nvfp4(
    source: torch.Tensor,
    global_scale: torch.Tensor,
    b: torch.Tensor,
    sfb: torch.Tensor,
    *,
    alpha: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    c_dtype: str = "bfloat16",
    stream: object = None,
) -> torch.Tensor:
    """NVFP4 counterpart of :func:`dense_gemm_fused_quant_a` (the reference fuses MXFP8 only):
    BF16 ``source [M, K]`` with ``M <= 16`` is quantized inside the decode kernel with the
    caller's ``global_scale`` (device FP32 scalar, read at run time) exactly as
    ``quantization.nvfp4.run`` would, then multiplied with the NVFP4 weight ``b [N, K/2, 1]`` /
    ``sfb``. ``alpha`` is normally ``1 / (global_scale_x * global_scale_w)``."""
    if source.dtype != torch.bfloat16 or source.ndim != 2 or not source.is_contiguous():
        raise ValueError("fused NVFP4 activation quantization requires contiguous BF16 [M,K]")
    m, k = map(int, source.shape)
    if m < 1 or m > launch.FUSED_QUANT_MAX_M or k % 64 != 0:
        raise ValueError(
            f"fused NVFP4 activation quantization requires 1<=M<={launch.FUSED_QUANT_MAX_M} and "
            f"K%64=0, got M={m}, K={k}")
    if global_scale.dtype != torch.float32 or global_scale.numel() != 1 or not global_scale.is_cuda:
        raise ValueError("global_scale must be a CUDA float32 tensor with one element")
    if alpha is not None and (alpha.dtype != torch.float32 or alpha.numel() != 1):
        raise ValueError("alpha must be a float32 tensor with one element")
    if c_dtype not in _C_DTYPES:
        raise KeyError(f"unsupported c_dtype string: {c_dtype!r}")
    w, sfw = _fused_quant_rhs("mm_fused_quant_a_nvfp4", b, sfb, k // 2)
    n = int(b.shape[0])
    if out is None:
        out = torch.empty((m, n, 1), dtype=_C_DTYPES[c_dtype], device=source.device)
    if out.shape != (m, n, 1) or out.dtype != _C_DTYPES[c_dtype]:
        raise ValueError(f"out must be {c_dtype} with shape {(m, n, 1)}, got {out.dtype} "
                         f"{tuple(out.shape)}")
    launch.gemm_smallm_fused_quant(_native.KIND_NVFP4, source, global_scale, w, sfw,
                                   out.select(2, 0), alpha, m, n, k, ldc=n,
                                   stream_int=cuda_stream_to_int(stream))
    return out


__all__ = ["dense_gemm", "dense_gemm_fused_quant_a", "dense_gemm_fused_quant_a_grouped",
           "dense_gemm_fused_quant_a_nvfp4", "get_num_sm"]
