"""Row quantizers on the GPU against the CPU oracle: bit-exact codes and scale bytes.

Covers the reference's quantizer tests (tests/quantization/test_nvfp4.py:19-51,
test_bf16_to_fp4_tma.py:345-622, test_mxfp8.py:19-50,
tests/gemm/test_cute_migration_gemm_corpus.py:273-340): seeded shapes, known-answer scale
codes, zero blocks, zero global scale, no negative-zero nibbles, guard bytes around outputs,
CUDA-graph replay with mutated inputs at the same addresses, plus the decode shapes
(M = 1, 4, 16, 64) and the full-size activation of the MXFP8 prefill configuration.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN, bf16_bits_to_f32, seeded_bf16
from oracle import blockscaled_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from gpu_util import DEV

    return DEV


def _mx_outputs(m, k, dev, guard=64):
    """Outputs carved out of canary-filled buffers so out-of-range writes are caught."""
    natoms = -(-m // 128) * -(-k // 128)
    bufs = {}
    for name, n in (("values", m * k), ("scale_rows", m * (k // 32)), ("scale_mma", natoms * 512)):
        raw = torch.full((n + 2 * guard,), 0xA5, dtype=torch.uint8, device=dev)
        bufs[name] = (raw, raw[guard:guard + n])
    return bufs


def _assert_guards(bufs, guard=64):
    for name, (raw, view) in bufs.items():
        assert (raw[:guard] == 0xA5).all() and (raw[-guard:] == 0xA5).all(), f"{name} guard hit"


@pytest.mark.parametrize("m,k,scale,dtype", [
    (128, 128, 1.0, torch.bfloat16), (7, 256, 0.25, torch.bfloat16), (1, 4096, 1.0, torch.bfloat16),
    (8, 512, 4.0, torch.bfloat16), (9, 384, 1.0, torch.bfloat16), (129, 160, 0.125, torch.bfloat16),
    (300, 1024, 1.0, torch.float16), (512, 7168, 1.0, torch.bfloat16),
])
def test_mxfp8_rows_bit_exact(dev, m, k, scale, dtype):
    from sparkinfer_b200.quantization import mxfp8

    x = seeded_bf16(1000 + m + k, (m, k), scale).to(dtype)
    if m >= 7:
        x[3, 32:64] = 0  # all-zero block -> scale byte 127
    ref_values, ref_rows = O.quantize_mxfp8_rows(x.float().numpy())
    bufs = _mx_outputs(m, k, dev)
    values = bufs["values"][1].view(m, k).view(torch.float8_e4m3fn)
    scale_rows = bufs["scale_rows"][1].view(m, k // 32)
    scale_mma = bufs["scale_mma"][1]
    scale_mma.fill_(127)  # caller pre-fills padding lanes, as in the reference's tests
    mxfp8.quantize_rows(x.to(dev), values, scale_rows, scale_mma)
    torch.cuda.synchronize()
    assert np.array_equal(values.view(torch.uint8).cpu().numpy(), ref_values)
    assert np.array_equal(scale_rows.cpu().numpy(), ref_rows)
    assert np.array_equal(scale_mma.cpu().numpy(), O.swizzle_scales(ref_rows, 127))
    _assert_guards(bufs)


def test_mxfp8_rows_match_reference_fixture(dev):
    from sparkinfer_b200._lib.mxfp8_rows import empty_mxfp8_rows_for_dense_gemm, quantize_mxfp8_rows

    g = np.load(GOLDEN / "mxfp8_quant.npz")
    for idx in (0, 2, 4):
        bits = g[f"x{idx}"]
        x = torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).to(dev)
        m, k = x.shape
        out = empty_mxfp8_rows_for_dense_gemm(m, k, device=dev)
        quantize_mxfp8_rows(x, out.values, out.scale_rows, out.scale_mma)
        assert np.array_equal(out.values.view(torch.uint8).cpu().numpy(), g[f"values{idx}"])
        assert np.array_equal(out.scale_rows.view(torch.uint8)[0].cpu().numpy(), g[f"scale_rows{idx}"])


def test_mxfp8_rows_reject_bad_arguments(dev):
    from sparkinfer_b200.quantization import mxfp8

    x = torch.zeros((4, 128), dtype=torch.bfloat16, device=dev)
    v = torch.empty((4, 128), dtype=torch.uint8, device=dev)
    r = torch.empty((4, 4), dtype=torch.uint8, device=dev)
    s = torch.empty(512, dtype=torch.uint8, device=dev)
    with pytest.raises(TypeError):
        mxfp8.quantize_rows(x.float(), v, r, s)
    with pytest.raises(ValueError, match="contiguous"):
        mxfp8.quantize_rows(x.t(), v, r, s)
    with pytest.raises(ValueError, match="scale_mma"):
        mxfp8.quantize_rows(x, v, r, s[:100])
    with pytest.raises(ValueError, match="values"):
        mxfp8.quantize_rows(x, v[:2], r, s)


@pytest.mark.parametrize("m,k,scale", [
    (128, 128, 1.0), (256, 512, 0.02), (1, 4096, 1.0), (4, 4096, 1.0), (16, 4096, 1.0),
    (64, 4096, 1.0), (129, 192, 3.0), (384, 1024, 1.0),
])
def test_nvfp4_rows_bit_exact(dev, m, k, scale):
    from sparkinfer_b200.quantization import nvfp4

    x = seeded_bf16(2000 + m + k, (m, k), scale)
    xf = x.float().numpy()
    gs = O.nvfp4_global_scale(xf)
    ref_packed, ref_scales = O.quantize_nvfp4_rows(xf, gs)
    plan = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(plan, device=dev)
    outs.packed_a_storage.fill_(0xFF)
    outs.scale_storage.fill_(0xFF)
    nvfp4.run(plan=plan, x=x.to(dev), global_scale=torch.tensor([gs], device=dev), outputs=outs)
    torch.cuda.synchronize()
    packed = outs.packed_a_storage[0].cpu().numpy()
    assert np.array_equal(packed, ref_packed)
    assert np.array_equal(outs.scale_flat.cpu().numpy(), O.swizzle_scales(ref_scales, 0))
    assert not ((packed & 0x0F) == 0x08).any() and not ((packed >> 4) == 0x08).any()
    assert int(outs.scale_flat.max()) <= 0x7E


def test_nvfp4_rows_match_reference_fixture_and_known_answers(dev):
    from sparkinfer_b200.quantization import nvfp4

    g = np.load(GOLDEN / "nvfp4_quant.npz")
    for key_x, key_gs, key_p, key_s in [("x1", "gs1", "packed1", "swizzled1"),
                                        ("x3", "gs3", "packed3", "swizzled3")]:
        x = torch.from_numpy(g[key_x].view(np.int16)).view(torch.bfloat16).to(dev)
        plan = nvfp4.plan(*x.shape)
        outs = nvfp4.allocate_outputs(plan, device=dev)
        nvfp4.run(plan=plan, x=x, global_scale=torch.from_numpy(g[key_gs]).to(dev), outputs=outs)
        assert np.array_equal(outs.packed_a_storage[0].cpu().numpy(), g[key_p])
        assert np.array_equal(outs.scale_flat.cpu().numpy(), g[key_s])
    # Scale-boundary rows (tests/quantization/test_bf16_to_fp4_tma.py:485-560), gs = 1.
    x = torch.from_numpy(g["ka_x"].view(np.int16)).view(torch.bfloat16).to(dev)
    plan = nvfp4.plan(128, 128)
    outs = nvfp4.allocate_outputs(plan, device=dev)
    nvfp4.run(plan=plan, x=x, global_scale=torch.ones(1, device=dev), outputs=outs)
    scales = O.unswizzle_scales(outs.scale_flat.cpu().numpy(), 128, 8)
    assert scales[0].tolist() == [0, 1, 3, 8, 7, 8, 8, 9]
    assert int(outs.scale_flat[16]) == 0  # row 1, block 0 lives at byte 16 of the first atom
    assert int(outs.packed_a_storage[0, 1, :8].count_nonzero()) == 0
    assert np.array_equal(outs.packed_a_storage[0].cpu().numpy(), g["ka_packed"])


def test_nvfp4_graph_replay_reads_live_inputs_and_zero_global_scale(dev):
    """Capture once, then replay with the source and the global scale changed in place
    (tests/quantization/test_bf16_to_fp4_tma.py:382-482, 590-622)."""
    from sparkinfer_b200.quantization import nvfp4

    m, k = 128, 256
    x = seeded_bf16(77, (m, k)).to(dev)
    gs = torch.tensor([O.nvfp4_global_scale(x.float().cpu().numpy())], device=dev)
    plan = nvfp4.plan(m, k)
    outs = nvfp4.allocate_outputs(plan, device=dev)
    nvfp4.run(plan=plan, x=x, global_scale=gs, outputs=outs)  # warm-up
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        nvfp4.run(plan=plan, x=x, global_scale=gs, outputs=outs)
    x2 = seeded_bf16(78, (m, k), 2.0)
    x.copy_(x2.to(dev))
    gs2 = O.nvfp4_global_scale(x2.float().numpy())
    gs.fill_(float(gs2))
    outs.packed_a_storage.fill_(0xFF)
    outs.scale_storage.fill_(0xFF)
    graph.replay()
    torch.cuda.synchronize()
    ref_packed, ref_scales = O.quantize_nvfp4_rows(x2.float().numpy(), gs2)
    assert np.array_equal(outs.packed_a_storage[0].cpu().numpy(), ref_packed)
    assert np.array_equal(outs.scale_flat.cpu().numpy(), O.swizzle_scales(ref_scales, 0))
    gs.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert int(outs.packed_a_storage.count_nonzero()) == 0
    assert int(outs.scale_storage.count_nonzero()) == 0


def test_nvfp4_rejects_overlap_and_wrong_device(dev):
    from sparkinfer_b200.quantization import nvfp4

    plan = nvfp4.plan(128, 128)
    outs = nvfp4.allocate_outputs(plan, device=dev)
    x = torch.zeros((128, 128), dtype=torch.bfloat16, device=dev)
    gs = torch.ones(1, device=dev)
    big = torch.zeros(128 * 64 + 128 * 8, dtype=torch.uint8, device=dev)
    with pytest.raises(ValueError, match="overlap"):
        plan.launch(x, gs, big[:128 * 64], big[128 * 8:128 * 8 + 128 * 8])
    with pytest.raises(ValueError, match="contiguous"):
        plan.launch(x.t().contiguous().t(), gs, outs.packed_a_flat, outs.scale_flat)
    with pytest.raises(ValueError, match="shape"):
        plan.launch(x, gs, outs.packed_a_flat[:-2], outs.scale_flat)


def test_full_size_prefill_activation_rows(dev):
    """The 8192 x 7168 activation of the MXFP8 prefill configuration: exact on a sample of
    rows (the oracle takes seconds on 256 rows), and every scale byte follows from its own
    block's maximum."""
    from sparkinfer_b200._lib.mxfp8_rows import empty_mxfp8_rows_for_dense_gemm, quantize_mxfp8_rows

    m, k = 8192, 7168
    x = seeded_bf16(4242, (m, k))
    out = empty_mxfp8_rows_for_dense_gemm(m, k, device=dev)
    xd = x.to(dev)
    quantize_mxfp8_rows(xd, out.values, out.scale_rows, out.scale_mma)
    torch.cuda.synchronize()
    rows = np.r_[0:64, 4000:4064, 8128:8192]
    ref_values, ref_rows = O.quantize_mxfp8_rows(x[rows].float().numpy())
    assert np.array_equal(out.values.view(torch.uint8)[rows].cpu().numpy(), ref_values)
    assert np.array_equal(out.scale_rows.view(torch.uint8)[0][rows].cpu().numpy(), ref_rows)
    amax = xd.float().view(m, k // 32, 32).abs().amax(-1).cpu().numpy()
    assert np.array_equal(out.scale_rows.view(torch.uint8)[0].cpu().numpy(), O.ue8m0_from_amax(amax))


@pytest.mark.parametrize("m,k,ld", [(5, 256, 320), (130, 1056, 2048), (16, 4096, 4104)])
def test_row_quantizers_read_row_strided_sources_through_the_c_abi(dev, m, k, ld):
    """The C entry points take a leading dimension for the source (rows of a wider activation
    buffer, as the fused quantize-then-GEMM path passes them): same bytes as for a dense copy
    of the rows, for MXFP8 (with and without the row-major scale output) and NVFP4 (K a
    multiple of 16 but not of 64 in the second case)."""
    import ctypes

    from sparkinfer_b200 import _native

    lib = _native.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    wide = seeded_bf16(7000 + m + k, (m, ld), 0.5).to(dev)
    x = wide[:, :k]
    dense = x.contiguous().float().cpu().numpy()

    ref_values, ref_rows = O.quantize_mxfp8_rows(dense)
    values = torch.empty((m, k), dtype=torch.uint8, device=dev)
    rows = torch.empty((m, k // 32), dtype=torch.uint8, device=dev)
    atoms = (-(-m // 128)) * (-(-k // 128)) * 512
    mma = torch.full((atoms,), 127, dtype=torch.uint8, device=dev)
    for with_rows in (True, False):
        values.zero_()
        rc = lib.b12x_b200_quantize_mxfp8_rows(
            x.data_ptr(), _native.DT_BF16, ld, values.data_ptr(),
            rows.data_ptr() if with_rows else None, mma.data_ptr(), m, k, stream)
        _native.check(rc, "quantize_mxfp8_rows")
        torch.cuda.synchronize()
        assert np.array_equal(values.cpu().numpy(), ref_values)
        assert np.array_equal(mma.cpu().numpy(), O.swizzle_scales(ref_rows, 127))
    assert np.array_equal(rows.cpu().numpy(), ref_rows)

    gs = O.nvfp4_global_scale(dense)
    ref_packed, ref_scales = O.quantize_nvfp4_rows(dense, gs)
    packed = torch.empty((m, k // 2), dtype=torch.uint8, device=dev)
    sf = torch.zeros(((-(-m // 128)) * (-(-k // 64)) * 512,), dtype=torch.uint8, device=dev)
    gs_dev = torch.tensor([gs], dtype=torch.float32, device=dev)
    rc = lib.b12x_b200_quantize_nvfp4_rows(x.data_ptr(), _native.DT_BF16, ld, gs_dev.data_ptr(),
                                           packed.data_ptr(), sf.data_ptr(), m, k, stream)
    _native.check(rc, "quantize_nvfp4_rows")
    torch.cuda.synchronize()
    assert np.array_equal(packed.cpu().numpy(), ref_packed)
    assert np.array_equal(sf.cpu().numpy(), O.swizzle_scales(ref_scales, 0))
