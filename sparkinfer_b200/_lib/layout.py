"""Scale-factor layout helpers (pure torch views and copies).

The MMA layout is the one the reference stores (b12x/_lib/utils.py:384-519,
b12x/_lib/intrinsics.py:62-105): physical ``[L][row_tile][col_tile][32][4][4]`` bytes, seen
by callers as the strided 6-D view ``(32, 4, row_tiles, 4, col_tiles, L)``. A scale at
(row, col) sits at byte ``(row % 32) * 16 + ((row / 32) % 4) * 4 + col % 4`` of atom
``(row / 128, col / 4)``; the CUDA kernels read and write exactly these bytes.
"""

from __future__ import annotations

import math

import torch


def ceil_div(a: int, b: int) -> int:
    return (int(a) + int(b) - 1) // int(b)


def align_up(value: int, alignment: int) -> int:
    return ceil_div(value, alignment) * int(alignment)


def get_mma_sf_shape(m: int, k: int, num_groups: int = 1, sf_vec_size: int = 16):
    """6-D logical shape ``(32, 4, m_tiles, 4, k_tiles, num_groups)``."""
    return (32, 4, ceil_div(m, 128), 4, ceil_div(ceil_div(k, sf_vec_size), 4), num_groups)


def mma_sf_nbytes(m: int, k: int, sf_vec_size: int, num_groups: int = 1) -> int:
    shape = get_mma_sf_shape(m, k, num_groups, sf_vec_size)
    return math.prod(shape)


def convert_sf_to_mma_layout(sf: torch.Tensor, m: int, k: int, num_groups: int = 1,
                             sf_vec_size: int = 16) -> torch.Tensor:
    """Swizzled flat/2-D scale bytes -> strided 6-D MMA view (no copy)."""
    _, _, m_tiles, _, k_tiles, _ = get_mma_sf_shape(m, k, num_groups, sf_vec_size)
    expected = num_groups * m_tiles * k_tiles * 512
    if sf.numel() != expected:
        raise ValueError(
            f"Scale factor tensor has {sf.numel()} elements, expected {expected} "
            f"for m={m}, k={k}, num_groups={num_groups}")
    return sf.view(num_groups, m_tiles, k_tiles, 32, 4, 4).permute(3, 4, 1, 5, 2, 0)


def convert_sf_from_mma_layout(sf_6d: torch.Tensor, m: int, k: int, num_groups: int = 1,
                               sf_vec_size: int = 16) -> torch.Tensor:
    """6-D MMA view -> contiguous swizzled 2-D ``(L * M_pad, K_pad / vec)``."""
    _, _, m_tiles, _, k_tiles, _ = get_mma_sf_shape(m, k, num_groups, sf_vec_size)
    storage = sf_6d.permute(5, 2, 4, 0, 1, 3).contiguous()
    return storage.reshape(num_groups * m_tiles * 128, k_tiles * 4)


def swizzle_block_scale(scale: torch.Tensor, pad_value: int = 0) -> torch.Tensor:
    """Row-major ``[rows, cols]`` (or ``[L, rows, cols]``) scale bytes -> same-rank tensor whose
    memory is in atom order, rows padded to 128 and cols to 4 with ``pad_value``."""
    squeeze = scale.ndim == 2
    if squeeze:
        scale = scale.unsqueeze(0)
    if scale.ndim != 3:
        raise ValueError(f"scale must be 2D or 3D, got {tuple(scale.shape)}")
    batch, rows, cols = scale.shape
    rp, cp = align_up(rows, 128), align_up(cols, 4)
    as_u8 = scale.view(torch.uint8) if scale.dtype != torch.uint8 else scale
    padded = torch.full((batch, rp, cp), pad_value, dtype=torch.uint8, device=scale.device)
    padded[:, :rows, :cols] = as_u8
    out = padded.reshape(batch, rp // 128, 4, 32, cp // 4, 4).permute(0, 1, 4, 3, 2, 5)
    out = out.contiguous().reshape(batch, rp, cp)
    if scale.dtype != torch.uint8:
        out = out.view(scale.dtype)
    return out[0] if squeeze else out


def unswizzle_block_scale(mma_view: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """6-D MMA view -> row-major ``[L, rows, cols]`` scale bytes (uint8)."""
    groups = mma_view.shape[-1]
    rp, cp = align_up(rows, 128), align_up(cols, 4)
    storage = mma_view.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8)
    tiles = storage.reshape(groups, rp // 128, cp // 4, 32, 4, 4).permute(0, 1, 4, 3, 2, 5)
    return tiles.reshape(groups, rp, cp)[:, :rows, :cols].contiguous()


def mma_view_is_canonical(sf: torch.Tensor, m: int, k: int, sf_vec_size: int,
                          num_groups: int = 1) -> bool:
    """True when ``sf`` is the 6-D permuted view over dense ``[L][mt][kt][32][4][4]`` bytes
    (or a flat / contiguous tensor of exactly that many bytes)."""
    shape = get_mma_sf_shape(m, k, num_groups, sf_vec_size)
    nbytes = math.prod(shape)
    if sf.element_size() != 1:
        return False
    if sf.ndim == 6 and tuple(sf.shape) == shape:
        _, _, m_tiles, _, k_tiles, _ = shape
        want = (16, 4, k_tiles * 512, 1, 512, m_tiles * k_tiles * 512)
        return all(sf.shape[i] == 1 or sf.stride(i) == want[i] for i in range(6))
    return sf.is_contiguous() and sf.numel() == nbytes


__all__ = [
    "ceil_div", "align_up", "get_mma_sf_shape", "mma_sf_nbytes", "convert_sf_to_mma_layout",
    "convert_sf_from_mma_layout", "swizzle_block_scale", "unswizzle_block_scale",
    "mma_view_is_canonical",
]
