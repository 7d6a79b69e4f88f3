"""Generate the golden fixtures in this directory from the b12x reference's own torch code.

Run where the reference source tree is available:

    B12X_REFERENCE=/path/to/b12x-checkout python tests/golden/make_golden.py

It imports the reference's pure-torch functions (CPU), feeds them seeded inputs and stores
inputs and outputs as small ``.npz`` files. The tests load the files only; they never
import the reference. Nothing here runs a GPU kernel.

Reference functions used (path:line in the b12x tree):
  quantize_grouped_nvfp4_torch, swizzle_block_scale       b12x/_lib/intrinsics.py:62-193
  quantize_grouped_mxfp8_torch, pow2_ceil_ue8m0_torch     b12x/_lib/intrinsics.py:223-313
  _scale_u8_from_max_abs                                  b12x/gemm/_shared/wo_mxfp8.py:844-851
  ref_fp4_quant, dequantize_grouped_nvfp4,
  compute_global_scale, recover_grouped_e4m3_scales       tests/_reference/helpers.py:224-363
  _block_fp8_reference                                    tests/gemm/test_gemm_stack.py:98-113
  _dequant_physical, _logical_b (gemm.bmm's reference)    tests/gemm/test_bmm.py:74-84
  pack_fp8_block_scaled_weight_mxfp8 (re-quantization to UE8M0 block scales, expansion to
  per-row scales, MMA layout)                             b12x/gemm/_shared/wo_mxfp8.py:873-1187
    (these insist on CUDA tensors; the generator swaps the module's device check for a no-op
     in its own process so that the same torch code runs on CPU tensors)
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _bf16_inputs(seed: int, shape, scale: float = 1.0) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * scale).to(torch.bfloat16)


def _bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main() -> None:
    ref_root = os.environ.get("B12X_REFERENCE")
    if not ref_root:
        raise SystemExit("set B12X_REFERENCE to a checkout of the b12x reference")
    sys.path.insert(0, ref_root)
    from b12x._lib import intrinsics as ri  # noqa: E402
    from b12x.gemm._shared import wo_mxfp8 as rw  # noqa: E402
    from tests._reference import helpers as rh  # noqa: E402

    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---------------- NVFP4 quantizer: seeded randn, several shapes ----------------
    nv = {}
    for idx, (m, k, scale) in enumerate(
        [(128, 128, 1.0), (256, 512, 1.0), (128, 1024, 1.0), (384, 256, 0.02), (128, 192, 3.0)]
    ):
        x = _bf16_inputs(42 + idx, (m, k), scale)
        gs = rh.compute_global_scale(x)
        packed, scale_view = ri.quantize_grouped_nvfp4_torch(
            x.unsqueeze(0).float(), torch.tensor([m]), gs
        )
        q, s = rh.ref_fp4_quant(x.float(), gs)
        # Same bytes from the two reference quantizers.
        assert torch.equal(ri.pack_grouped_fp4_values(q.unsqueeze(0))[:, :, 0], packed[:, :, 0])
        swz = ri.swizzle_block_scale(s.to(torch.float8_e4m3fn).unsqueeze(0)).view(torch.uint8)
        deq = rh.dequantize_grouped_nvfp4(
            packed.permute(2, 0, 1).contiguous(), scale_view, k, gs
        )[0]
        nv[f"x{idx}"] = _bf16_bits(x)
        nv[f"gs{idx}"] = gs.numpy()
        nv[f"packed{idx}"] = packed[:, :, 0].contiguous().numpy()
        nv[f"scales{idx}"] = s.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        nv[f"swizzled{idx}"] = swz.reshape(-1).numpy()
        if idx == 0:
            nv["dequant0"] = deq.numpy()
    # Known-answer rows of tests/quantization/test_bf16_to_fp4_tma.py:485-560, gs = 1.
    block_values = torch.tensor(
        [0.0, 0.01171875, 0.03515625, 0.09375, 0.08740234375, 0.08837890625, 0.09912109375,
         0.10009765625],
        dtype=torch.bfloat16,
    )
    src = block_values.repeat_interleave(16).expand(128, 128).clone().contiguous()
    src[1, :16] = 0.001953125
    one = torch.ones((1,), dtype=torch.float32)
    packed, _ = ri.quantize_grouped_nvfp4_torch(src.unsqueeze(0).float(), torch.tensor([128]), one)
    _, s = rh.ref_fp4_quant(src.float(), one)
    nv["ka_x"] = _bf16_bits(src)
    nv["ka_packed"] = packed[:, :, 0].contiguous().numpy()
    nv["ka_scales"] = s.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.savez_compressed(HERE / "nvfp4_quant.npz", **nv)

    # ---------------- MXFP8 quantizer ----------------
    mx = {}
    for idx, (m, k, scale) in enumerate(
        [(128, 128, 1.0), (7, 256, 0.25), (256, 512, 1.0), (129, 160, 0.125), (16, 2048, 1.0)]
    ):
        x = _bf16_inputs(142 + idx, (m, k), scale)
        if idx == 1:
            x[3, 32:64] = 0  # an all-zero block
        blocked = x.float().reshape(m, k // 32, 32)
        max_abs = blocked.abs().amax(dim=-1)
        scale_u8 = rw._scale_u8_from_max_abs(max_abs)
        s = scale_u8.view(torch.float8_e8m0fnu).to(torch.float32)
        values = (
            (blocked / s[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).reshape(m, k)
        )
        # The CPU-safe twin in intrinsics.py must agree wherever the block is not all zero.
        twin_vals, _ = ri.quantize_grouped_mxfp8_torch(x.unsqueeze(0).float(), torch.tensor([m]))
        _, twin_byte = ri.pow2_ceil_ue8m0_torch(max_abs * (1.0 / 448.0))
        nz = max_abs > 0
        assert torch.equal(twin_byte[nz], scale_u8[nz])
        assert torch.equal(twin_vals[:, :, 0][nz.repeat_interleave(32, dim=1)],
                           values.view(torch.uint8)[nz.repeat_interleave(32, dim=1)])
        deq = (values.float().reshape(m, k // 32, 32) * s[..., None]).reshape(m, k)
        mx[f"x{idx}"] = _bf16_bits(x)
        mx[f"values{idx}"] = values.view(torch.uint8).numpy()
        mx[f"scale_rows{idx}"] = scale_u8.numpy()
        mx[f"swizzled{idx}"] = (
            ri.swizzle_block_scale(scale_u8.unsqueeze(0)).reshape(-1).numpy()
        )
        if idx == 0:
            mx["dequant0"] = deq.numpy()
    # Every positive finite BF16 amax: the UE8M0 byte table.
    all_bf16 = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    mx["amax_table_bits"] = _bf16_bits(all_bf16)
    mx["amax_table_byte"] = rw._scale_u8_from_max_abs(all_bf16.float()).numpy()
    np.savez_compressed(HERE / "mxfp8_quant.npz", **mx)

    # ---------------- GEMM references (dequantize -> FP32 matmul) ----------------
    gm = {}
    a = _bf16_inputs(1042, (128, 256))
    b = _bf16_inputs(1043, (192, 256), 0.02)
    gsa, gsb = rh.compute_global_scale(a), rh.compute_global_scale(b)
    pa, sva = ri.quantize_grouped_nvfp4_torch(a.unsqueeze(0).float(), torch.tensor([128]), gsa)
    pb, svb = ri.quantize_grouped_nvfp4_torch(b.unsqueeze(0).float(), torch.tensor([192]), gsb)
    da = rh.dequantize_grouped_nvfp4(pa.permute(2, 0, 1).contiguous(), sva, 256, gsa)[0]
    db = rh.dequantize_grouped_nvfp4(pb.permute(2, 0, 1).contiguous(), svb, 256, gsb)[0]
    gm["nv_a"], gm["nv_b"] = _bf16_bits(a), _bf16_bits(b)
    gm["nv_gsa"], gm["nv_gsb"] = gsa.numpy(), gsb.numpy()
    gm["nv_out"] = (da @ db.T).numpy()
    # Block-FP8 with FP32 scales: the reference's own test reference
    # (tests/gemm/test_gemm_stack.py:98-113, BF16 out), imported, plus the same dequantized
    # product kept in FP32 for the tight error bound.
    import importlib

    block_fp8_reference = importlib.import_module("tests.gemm.test_gemm_stack")._block_fp8_reference
    m, n, k = 64, 256, 256
    gen = torch.Generator().manual_seed(3042)
    a8 = torch.randn((m, k), generator=gen).clamp(-3, 3).to(torch.float8_e4m3fn)
    b8 = torch.randn((n, k), generator=gen).clamp(-3, 3).to(torch.float8_e4m3fn)
    sa = torch.rand((m, k // 128), generator=gen) + 0.5
    sb = torch.rand((n // 128, k // 128), generator=gen) + 0.5
    a_d = (a8.float().view(m, k // 128, 128) * sa[:, :, None]).reshape(m, k)
    b_d = (b8.float().view(n // 128, 128, k // 128, 128) * sb[:, None, :, None]).reshape(n, k)
    gm["bf8_out_bf16_bits"] = _bf16_bits(block_fp8_reference(a8, b8, sa, sb))
    gm["bf8_a"] = a8.view(torch.uint8).numpy()
    gm["bf8_b"] = b8.view(torch.uint8).numpy()
    gm["bf8_sa"], gm["bf8_sb"] = sa.numpy(), sb.numpy()
    gm["bf8_out"] = (a_d @ b_d.T).numpy()
    np.savez_compressed(HERE / "gemm_ref.npz", **gm)

    # ---------------- weight packers (checkpoint block-FP8 -> MXFP8 rows) ----------------
    import b12x.gemm._shared.wo_mxfp8 as rw  # noqa: E402

    rw._check_gpu_tensor = lambda name, tensor: None  # CPU run of device-agnostic torch code
    pk = {}
    for idx, (n_rows, k_cols, groups, seed, pow2) in enumerate([
            (256, 384, 1, 4042, False), (128, 256, 2, 4043, False), (200, 128, 1, 4044, False),
            (128, 256, 1, 4045, True)]):
        gen = torch.Generator().manual_seed(seed)
        w = (torch.randn((groups * n_rows, k_cols), generator=gen) * 100).clamp(-448, 448)
        w8 = w.to(torch.float8_e4m3fn)
        blocks = (groups, -(-n_rows // 128), k_cols // 128)
        if pow2:
            sc = torch.pow(2.0, torch.randint(-6, 3, blocks, generator=gen).float())
        else:
            sc = torch.rand(blocks, generator=gen) * 0.01 + 1e-4
        sc = sc[0] if groups == 1 else sc
        rows = rw.pack_fp8_block_scaled_weight_mxfp8(w8, sc, m=n_rows, k=k_cols, num_groups=groups)
        pk[f"w{idx}"] = w8.view(torch.uint8).numpy()
        pk[f"scale{idx}"] = sc.numpy()
        pk[f"shape{idx}"] = np.array([n_rows, k_cols, groups], dtype=np.int64)
        vals = rows.values if rows.values.ndim == 2 else rows.values.permute(2, 0, 1)
        pk[f"values{idx}"] = vals.contiguous().view(torch.uint8).numpy()
        pk[f"scale_rows{idx}"] = rows.scale_rows.contiguous().view(torch.uint8).numpy()
        # Physical bytes of the MMA-layout scale tensor: [L][row_tile][k_tile][32][4][4].
        pk[f"scale_mma{idx}"] = (rows.scale_mma.permute(5, 2, 4, 0, 1, 3).contiguous()
                                 .view(torch.uint8).numpy().reshape(-1))
    np.savez_compressed(HERE / "weight_pack.npz", **pk)

    # ---------------- gemm.bmm: the reference test module's own torch reference ----------------
    import importlib

    tb = importlib.import_module("tests.gemm.test_bmm")
    bm = {}
    for idx, (major, batch, m, n, k, seed) in enumerate([
            ("k", 3, 5, 48, 96, 5101), ("n", 2, 7, 64, 40, 5102), ("k", 2, 32, 40, 64, 5103)]):
        gen = torch.Generator().manual_seed(seed)
        rows, inner = (k, n) if major == "n" else (n, k)
        values = (torch.randn((batch, rows, inner), generator=gen) * 0.3).to(torch.float8_e4m3fn)
        scales = torch.randint(100, 150, (batch, rows, inner // 32), generator=gen, dtype=torch.uint8)
        scales[0, 0, 0], scales[0, 1, 0], scales[1, 0, 0] = 0, 1, 254
        lhs = _bf16_inputs(seed + 50, (batch, m, k))
        physical = tb._dequant_physical((values, scales))
        logical = tb._logical_b((values, scales), major)
        bm[f"major{idx}"] = np.array([major == "n"])
        bm[f"values{idx}"] = values.view(torch.uint8).numpy()
        bm[f"scales{idx}"] = scales.numpy()
        bm[f"lhs_bits{idx}"] = _bf16_bits(lhs)
        bm[f"dequant_bits{idx}"] = _bf16_bits(physical)
        bm[f"product{idx}"] = torch.bmm(lhs.double(), logical.double()).numpy()
    np.savez_compressed(HERE / "bmm_ref.npz", **bm)

    for name in ("nvfp4_quant.npz", "mxfp8_quant.npz", "gemm_ref.npz", "weight_pack.npz",
                 "bmm_ref.npz"):
        print(name, (HERE / name).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
