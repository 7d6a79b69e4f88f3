"""``dense_gemm(..., block_fp8=True)``: E4M3 operands with compact FP32 scales.

Host side of the reference's block-FP8 mode (b12x/_lib/dense_gemm.py:7190-7224): activations
carry one FP32 scale per row and 128 columns (``[M, K/128]``), weights one per 128x128 block
(``[N/128, K/128]``); the oracle is ``_block_fp8_reference`` of
tests/gemm/test_gemm_stack.py:98-113. The same argument checks and error text apply.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import launch
from .launch import cuda_stream_to_int

_C_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def block_fp8_gemm(a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor, sfb: torch.Tensor,
                   out: Optional[torch.Tensor], *, c_dtype: str, sf_dtype: str, sf_vec_size: int,
                   alpha: Optional[torch.Tensor], load_path, swap_ab, sfb_k_replicated: bool,
                   sm_count: int, stream: object) -> torch.Tensor:
    m, k, l = a.shape
    n = b.shape[0]
    want_sfa, want_sfb = (m, k // 128), (n // 128, k // 128)
    if (sf_dtype != "float32" or sf_vec_size != 128 or l != 1 or n % 128 != 0 or k % 128 != 0
            or tuple(sfa.shape) != want_sfa or tuple(sfb.shape) != want_sfb
            or sfa.dtype != torch.float32 or sfb.dtype != torch.float32
            or not sfa.is_contiguous() or not sfb.is_contiguous()):
        raise ValueError(
            "block_fp8 requires L=1, N/K divisible by 128, sf_dtype='float32', "
            "sf_vec_size=128, and contiguous FP32 scales shaped "
            f"{want_sfa} and {want_sfb}")
    if load_path not in (None, "tma") or swap_ab not in (None, False) or sfb_k_replicated:
        raise ValueError(
            "block_fp8 currently requires unswapped TMA operands without tiled RHS, "
            "quantized output, or replicated weight scales")
    for name, t, rows in (("A", a, m), ("B", b, n)):
        if not t.is_cuda:
            raise ValueError(f"{name} must be on CUDA")
        if t.element_size() != 1 or tuple(t.shape) != (rows, k, 1) or t.stride(1) != 1 \
                or (rows > 1 and t.stride(0) != k):
            raise ValueError(f"{name} must be a K-major one-byte [{rows}, {k}, 1] tensor")
    if out is None:
        out = torch.empty((m, n, 1), dtype=_C_DTYPES[c_dtype], device=a.device)
    if tuple(out.shape) != (m, n, 1) or out.dtype != _C_DTYPES[c_dtype] or out.stride(1) != 1:
        raise ValueError(f"out must be {c_dtype} with shape {(m, n, 1)}")
    if alpha is not None and (alpha.dtype != torch.float32 or alpha.numel() != 1):
        raise ValueError("alpha must be a float32 tensor with one element")
    if m == 0:
        return out
    launch.gemm_block_fp8(a.select(2, 0), sfa, b.select(2, 0), sfb, out.select(2, 0), alpha,
                          m, n, k, ldc=out.stride(0) if m > 1 else n, sm_count=sm_count,
                          stream_int=cuda_stream_to_int(stream))
    return out
