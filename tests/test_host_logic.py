"""Host-side logic that needs no GPU: scratch plans and bindings on CPU tensors, layout
helpers against the oracle, argument validation, fake (meta) implementations of the custom
ops. Modelled on the reference's tests/gemm/test_block_fp8_linear_scratch_bindings.py and
tests/gemm/test_launch_custom_ops.py."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import blockscaled_oracle as O
from sparkinfer_b200._lib import layout
from sparkinfer_b200._lib.mxfp8_rows import MXFP8Rows
from sparkinfer_b200._lib.scratch import scratch_buffer_spec, scratch_tensor
from sparkinfer_b200.gemm import block_fp8_linear as bfl
from sparkinfer_b200.gemm import blockscaled
from sparkinfer_b200.gemm._shared import block_fp8 as block_impl
from sparkinfer_b200.quantization import nvfp4


def _packed_weight(*, in_features: int = 128, out_features: int = 256):
    weight = MXFP8Rows(
        values=torch.empty((out_features, in_features), dtype=torch.float8_e4m3fn),
        scale_rows=torch.empty((1, out_features, in_features // 32), dtype=torch.float8_e8m0fnu),
        scale_mma=torch.empty((32, 4, math.ceil(out_features / 128), 4,
                               math.ceil((in_features // 32) / 4), 1), dtype=torch.float8_e8m0fnu),
    )
    return bfl.Weight(weight=weight, in_features=in_features, out_features=out_features,
                      block_size=(128, 128))


def _cpu_plan(max_tokens=4):
    return bfl.plan(bfl.Caps(device="cpu", max_tokens=max_tokens, in_features=128, out_features=256))


def test_plan_exposes_one_opaque_uint8_scratch():
    plan = _cpu_plan()
    specs = plan.scratch_specs()
    assert len(specs) == 1 and specs[0].name == "block_fp8_linear.scratch"
    assert specs[0].dtype == torch.uint8 and specs[0].nbytes == specs[0].shape[0]
    assert specs[0].shape == plan.shapes_and_dtypes()[0][0]
    # align1024(T*K) + align1024(T*K/32) + ceil(T/128)*ceil(K/128)*512
    assert specs[0].shape[0] == 1024 + 1024 + 512


def test_bind_maps_scratch_views_without_allocating(monkeypatch):
    monkeypatch.setattr(block_impl, "_check_mxfp8_rows_storage", lambda *a, **k: None)
    plan = _cpu_plan()
    spec = plan.scratch_specs()[0]
    scratch = torch.empty(spec.shape, dtype=spec.dtype, device=spec.device)
    source = torch.empty((3, 128), dtype=torch.bfloat16)
    output = torch.empty((3, 256, 1), dtype=torch.bfloat16)
    packed = _packed_weight()
    binding = bfl.bind(plan, scratch=scratch, source=source, packed_weight=packed, output=output)
    assert isinstance(binding, bfl.Binding) and not hasattr(binding, "workspace")
    assert binding.source is source and binding.packed_weight is packed and binding.output is output
    assert binding.x_q.values.shape == (3, 128)
    assert binding.x_q.values.data_ptr() == scratch.data_ptr()
    assert binding.x_q.scale_rows.data_ptr() == scratch.data_ptr() + 1024
    assert binding.x_q.scale_mma.shape == (32, 4, 1, 4, 1, 1)
    assert (binding.x_q.scale_rows.view(torch.uint8) == 127).all()
    # mapping and sequence forms of the scratch argument
    bfl.bind(plan, scratch={"block_fp8_linear.scratch": scratch}, source=source,
             packed_weight=packed, output=output)
    bfl.bind(plan, scratch=[scratch], source=source, packed_weight=packed, output=output)


def test_bind_rejects_bad_arguments(monkeypatch):
    monkeypatch.setattr(block_impl, "_check_mxfp8_rows_storage", lambda *a, **k: None)
    plan = _cpu_plan()
    spec = plan.scratch_specs()[0]
    scratch = torch.empty(spec.shape, dtype=spec.dtype)
    packed = _packed_weight()
    good = dict(scratch=scratch, source=torch.empty((3, 128), dtype=torch.bfloat16),
                packed_weight=packed, output=torch.empty((3, 256, 1), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="exceed"):
        bfl.bind(plan, **{**good, "source": torch.empty((5, 128), dtype=torch.bfloat16)})
    with pytest.raises(ValueError, match="in_features"):
        bfl.bind(plan, **{**good, "source": torch.empty((3, 256), dtype=torch.bfloat16)})
    with pytest.raises(ValueError, match="dtype"):
        bfl.bind(plan, **{**good, "source": torch.empty((3, 128), dtype=torch.float16)})
    with pytest.raises(ValueError, match="requires"):
        bfl.bind(plan, **{**good, "scratch": scratch[:100]})
    with pytest.raises(TypeError):
        bfl.bind(plan, **{**good, "scratch": scratch.view(torch.int8)})
    with pytest.raises(ValueError, match="output must have shape"):
        bfl.bind(plan, **{**good, "output": torch.empty((3, 256), dtype=torch.bfloat16)})
    with pytest.raises(KeyError):
        bfl.bind(plan, **{**good, "scratch": {"other": scratch}})


def test_run_with_binding_rejects_duplicate_tensors(monkeypatch):
    monkeypatch.setattr(block_impl, "_check_mxfp8_rows_storage", lambda *a, **k: None)
    plan = _cpu_plan()
    spec = plan.scratch_specs()[0]
    source = torch.empty((3, 128), dtype=torch.bfloat16)
    binding = bfl.bind(plan, scratch=torch.empty(spec.shape, dtype=spec.dtype), source=source,
                       packed_weight=_packed_weight(),
                       output=torch.empty((3, 256, 1), dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="binding owns source"):
        bfl.run(source, binding=binding)
    with pytest.raises(TypeError):
        bfl.run()


def test_caps_validate():
    with pytest.raises(ValueError, match="multiple of 128"):
        bfl.Caps(device="cpu", max_tokens=4, in_features=160, out_features=256)
    with pytest.raises(ValueError, match="bf16/fp16"):
        bfl.Caps(device="cpu", max_tokens=4, in_features=128, out_features=256,
                 output_dtype=torch.float32)


def test_scratch_tensor_contract():
    spec = scratch_buffer_spec("s", nbytes=64, device=torch.device("cpu"))
    buf = torch.empty(64, dtype=torch.uint8)
    assert scratch_tensor(buf, (spec,), owner="t").shape == (64,)
    with pytest.raises(RuntimeError):
        scratch_tensor(buf, (spec, spec), owner="t")
    with pytest.raises(ValueError):
        scratch_tensor([buf, buf], (spec,), owner="t")


def test_layout_helpers_match_oracle_swizzle():
    rng = np.random.RandomState(1)
    for rows, cols in [(128, 4), (300, 10), (7, 8), (256, 56)]:
        scales = rng.randint(0, 255, size=(rows, cols)).astype(np.uint8)
        want = O.swizzle_scales(scales, pad_value=0)
        got = layout.swizzle_block_scale(torch.from_numpy(scales)).reshape(-1).numpy()
        assert np.array_equal(got, want)
        view = layout.convert_sf_to_mma_layout(torch.from_numpy(want), rows, cols * 16)
        assert view.shape == layout.get_mma_sf_shape(rows, cols * 16)
        assert layout.mma_view_is_canonical(view, rows, cols * 16, 16)
        back = layout.unswizzle_block_scale(view, rows, cols)[0].numpy()
        assert np.array_equal(back, scales)
        r, c = rows - 1, cols - 1
        assert view[r % 32, (r // 32) % 4, r // 128, c % 4, c // 4, 0] == scales[r, c]
        flat2d = layout.convert_sf_from_mma_layout(view, rows, cols * 16)
        assert np.array_equal(flat2d.reshape(-1).numpy(), want)
    assert not layout.mma_view_is_canonical(torch.zeros(7), 128, 64, 16)


def test_blockscaled_mm_validates_before_launch():
    a = torch.zeros((128, 64, 1), dtype=torch.uint8)
    sf = torch.zeros((32, 4, 1, 4, 2, 1), dtype=torch.uint8)
    kw = dict(sf_dtype="float8_e4m3fn", c_dtype="bfloat16", sf_vec_size=16, sm_count=148)
    with pytest.raises(TypeError, match="unsupported ab_dtype"):
        blockscaled.mm((a, sf), (a, sf), ab_dtype="int8", **kw)
    with pytest.raises(ValueError, match="load_path"):
        blockscaled.mm((a, sf), (a, sf), ab_dtype="float4_e2m1fn", load_path="ldg", **kw)
    with pytest.raises(ValueError, match="MX-FP6"):
        blockscaled.mm((a, sf), (a, sf), ab_dtype="float4_e2m1fn", a_fmt="e2m3", **kw)
    with pytest.raises(ValueError, match="mutually exclusive"):
        blockscaled.mm((a, sf), (a, sf), ab_dtype="float4_e2m1fn", b_packed=True,
                       b_preexpanded=True, **kw)
    with pytest.raises(ValueError, match=r"\(NVFP4\) or"):
        blockscaled.mm((a, sf), (a, sf), ab_dtype="float4_e2m1fn", sf_dtype="float8_e8m0fnu",
                       c_dtype="bfloat16", sf_vec_size=16, sm_count=148)
    with pytest.raises(ValueError, match="CUDA"):
        blockscaled.mm((a, sf), (a, sf), ab_dtype="float4_e2m1fn", **kw)


def test_nvfp4_plan_validates_shapes_and_tensors():
    with pytest.raises(ValueError, match="positive"):
        nvfp4.plan(0, 128)
    with pytest.raises(ValueError, match="multiple of 64"):
        nvfp4.plan(4, 100)
    plan = nvfp4.plan(4, 128)
    outs = nvfp4.allocate_outputs(plan, device="cpu")
    assert outs.packed_a_storage.shape == (1, 4, 64) and outs.scale_storage.numel() == 128 * 8
    assert outs.scale_mma_view(4, 128).shape == (32, 4, 1, 4, 2, 1)
    x = torch.zeros((4, 128), dtype=torch.bfloat16)
    gs = torch.ones(1)
    with pytest.raises(ValueError, match="dtype"):
        nvfp4.run(plan=plan, x=x.float(), global_scale=gs, outputs=outs)
    with pytest.raises(ValueError, match="shape"):
        nvfp4.run(plan=plan, x=x[:2], global_scale=gs, outputs=outs)
    with pytest.raises(ValueError, match="must be on"):
        nvfp4.run(plan=plan, x=x, global_scale=gs, outputs=outs)  # CPU tensors are refused


def test_custom_ops_have_fake_implementations():
    from torch._subclasses.fake_tensor import FakeTensorMode

    import sparkinfer_b200._lib.dense_gemm  # noqa: F401  (registers the ops)
    import sparkinfer_b200.gemm.mxfp8_linear._kernel  # noqa: F401

    with FakeTensorMode():
        src = torch.empty((5, 256), dtype=torch.bfloat16)
        w = torch.empty((64, 256), dtype=torch.float8_e4m3fn)
        srows = torch.empty((1, 64, 8), dtype=torch.float8_e8m0fnu)
        smma = torch.empty((32, 4, 1, 4, 2, 1), dtype=torch.float8_e8m0fnu)
        out = torch.ops.b12x.mxfp8_linear_fused(src, w, srows, smma, 256, 256, 64, 5, None)
        assert out.shape == (5, 64) and out.dtype == torch.bfloat16
        out = torch.ops.b12x.block_fp8_linear_mxfp8_fused(src, w, srows, smma, 256, 64, 0, None)
        assert out.shape == (5, 64)
        v, r, p = torch.ops.b12x.quantize_block_fp8_linear_input_mxfp8_alloc(src, 5, 256)
        assert v.shape == (5, 256) and r.shape == (1, 5, 8) and p.shape == (1, 1, 2, 32, 4, 4)
        a = torch.empty((128, 64, 1), dtype=torch.uint8)
        sf = torch.empty((32, 4, 1, 4, 2, 1), dtype=torch.uint8)
        alpha = torch.empty(1)
        tail = ("float32", 16, 64, 128, 128, 128, 1, 1, 148, False, False, False, 1, False, False,
                "tma", False, False, True, None)
        c = torch.ops.b12x.dense_gemm_launch_functional(
            a, a, sf, sf, alpha, 128, 128, 1, 1, "float4_e2m1fn", "float8_e4m3fn", "bfloat16",
            "bfloat16", *tail)
        assert c.shape == (128, 128, 1) and c.dtype == torch.bfloat16
        cc = torch.empty((128, 128, 1), dtype=torch.bfloat16)
        assert torch.ops.b12x.dense_gemm_launch(
            a, a, sf, sf, cc, alpha, 128, 128, 1, 1, "float4_e2m1fn", "float8_e4m3fn",
            "bfloat16", *tail) is None


@pytest.mark.parametrize("idx", [0, 1, 2, 3])
def test_weight_packers_match_reference_fixture(monkeypatch, idx):
    """pack_fp8_block_scaled_weight_mxfp8 (load-time torch code, device-agnostic apart from
    its CUDA-tensor check, which is lifted here) against outputs of the reference's own
    function on the same checkpoint-style inputs: re-quantized codes, per-row scale bytes and
    the physical bytes of the MMA-layout scale tensor, one and two groups, ragged row count,
    power-of-two scales passed through."""
    from conftest import GOLDEN
    from sparkinfer_b200._lib import mxfp8_rows as mr

    monkeypatch.setattr(mr, "_check_gpu_tensor", lambda name, tensor: None)
    g = np.load(GOLDEN / "weight_pack.npz")
    m, k, groups = (int(v) for v in g[f"shape{idx}"])
    weight = torch.from_numpy(g[f"w{idx}"]).view(torch.float8_e4m3fn)
    scale = torch.from_numpy(g[f"scale{idx}"])
    rows = mr.pack_fp8_block_scaled_weight_mxfp8(weight, scale, m=m, k=k, num_groups=groups)
    values = rows.values if rows.values.ndim == 2 else rows.values.permute(2, 0, 1)
    assert np.array_equal(values.contiguous().view(torch.uint8).numpy(), g[f"values{idx}"])
    assert np.array_equal(rows.scale_rows.contiguous().view(torch.uint8).numpy(),
                          g[f"scale_rows{idx}"])
    physical = rows.scale_mma.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8)
    assert np.array_equal(physical.numpy().reshape(-1), g[f"scale_mma{idx}"])


def test_tensor_fp8_linear_fake_op_and_host_validation():
    """The per-tensor FP8 linear's custom op has a fake (meta) implementation, and its host
    checks fire before anything touches a GPU (tests/gemm/test_tensor_fp8_linear.py and the
    argument checks of b12x/gemm/tensor_fp8_linear/_kernel.py:120-150, 232-268)."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    from sparkinfer_b200.gemm import tensor_fp8_linear
    from sparkinfer_b200.gemm.tensor_fp8_linear import _kernel  # noqa: F401  (registers the op)

    with FakeTensorMode():
        src = torch.empty((5, 160), dtype=torch.float8_e4m3fn)
        w = torch.empty((40, 256), dtype=torch.float8_e4m3fn)
        smma = torch.empty((32, 4, 1, 4, 2, 1), dtype=torch.float8_e8m0fnu)
        scale = torch.empty(1)
        out = torch.ops.b12x.tensor_fp8_linear_fused(src, w, smma, scale, 256, 40, 5,
                                                     torch.float16, None)
        assert out.shape == (5, 40) and out.dtype == torch.float16

    w_cpu = torch.zeros((64, 128), dtype=torch.float8_e4m3fn)
    with pytest.raises((ValueError, TypeError)):
        tensor_fp8_linear.pack_weight(w_cpu, torch.ones(1))  # CPU tensors are refused
    with pytest.raises(ValueError, match="CUDA"):
        tensor_fp8_linear.mm(w_cpu, object())  # the device check comes first, as in the reference
    assert isinstance(tensor_fp8_linear.is_supported(), bool)
    assert "tensor_fp8_linear" in {m.name for m in __import__("sparkinfer_b200").list_ops()}


def test_grouped_fused_quant_host_checks_fire_before_any_launch():
    """Argument errors of mm_fused_quant_a_grouped (b12x/_lib/dense_gemm.py:5803-5944) are host
    checks: they need no GPU and raise the reference's messages."""
    from sparkinfer_b200.gemm import blockscaled

    k, groups, n = 256, 3, 128
    src = torch.zeros((4, groups, k), dtype=torch.bfloat16)
    b = torch.zeros((groups, n, k), dtype=torch.uint8).permute(1, 2, 0)
    sfb = torch.zeros(1, dtype=torch.uint8)
    with pytest.raises(ValueError, match=r"requires BF16 \[M, groups, K\]"):
        blockscaled.mm_fused_quant_a_grouped(src.float(), b, sfb, groups=groups)
    with pytest.raises(ValueError, match="source groups 3 != weight groups 4"):
        blockscaled.mm_fused_quant_a_grouped(src, b, sfb, groups=4)
    with pytest.raises(ValueError, match="1<=M<=8"):
        blockscaled.mm_fused_quant_a_grouped(torch.zeros((9, groups, k), dtype=torch.bfloat16), b, sfb,
                                             groups=groups)
    with pytest.raises(ValueError, match="contiguous \\[groups, K\\] rows"):
        blockscaled.mm_fused_quant_a_grouped(
            torch.zeros((4, groups, 2 * k), dtype=torch.bfloat16)[:, :, :k], b, sfb, groups=groups)
    with pytest.raises(ValueError, match=r"B must have shape \[N,256,3\]"):
        blockscaled.mm_fused_quant_a_grouped(src, b[:, :128], sfb, groups=groups)
    positions = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(ValueError, match="needs both positions and cos_sin_cache"):
        blockscaled.mm_fused_quant_a_grouped(src, b, sfb, groups=groups, positions=positions)
    rope = dict(head_dim=128, nope_dim=96, rope_dim=32)
    with pytest.raises(ValueError, match=r"positions must have shape \(4,\)"):
        blockscaled.mm_fused_quant_a_grouped(src, b, sfb, groups=groups, positions=positions[:3],
                                             cos_sin_cache=torch.zeros((8, 32)), **rope)
    with pytest.raises(ValueError, match=r"cos_sin_cache must have shape \[max_pos, 32\]"):
        blockscaled.mm_fused_quant_a_grouped(src, b, sfb, groups=groups, positions=positions,
                                             cos_sin_cache=torch.zeros((8, 64)), **rope)
    with pytest.raises(ValueError, match=r"32-aligned head_dim = nope_dim \+ rope_dim"):
        blockscaled.mm_fused_quant_a_grouped(src, b, sfb, groups=groups, positions=positions,
                                             cos_sin_cache=torch.zeros((8, 32)), head_dim=128,
                                             nope_dim=80, rope_dim=32)
    with pytest.raises(ValueError, match="positions must be int32/int64"):
        blockscaled.mm_fused_quant_a_grouped(src, b, sfb, groups=groups,
                                             positions=positions.float(),
                                             cos_sin_cache=torch.zeros((8, 32)), **rope)
    with pytest.raises(ValueError, match="cache must be bf16/fp32"):
        blockscaled.mm_fused_quant_a_grouped(src, b, sfb, groups=groups, positions=positions,
                                             cos_sin_cache=torch.zeros((8, 32), dtype=torch.float16),
                                             **rope)
