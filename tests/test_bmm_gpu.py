"""``gemm.bmm`` (BF16 x rowwise-MXFP8, batched) against torch references, modelled on the
reference's tests/gemm/test_bmm.py: both weight layouts as zero-copy views of one allocation,
one-hot activations that read the dequantized weights back bit for bit, the E8M0 boundary
bytes, the error of a random product measured against FP64 next to cuBLAS's, determinism,
CUDA-graph replay into a strided output, a side stream, and torch.compile. The last test
drives the C-ABI launcher over geometries outside the qualified envelope."""

from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BATCH, PACK_ROWS = 16, 448
K_NMAJ, N_NMAJ = 192, 512
N_KMAJ, K_KMAJ = 256, 512
M_VALUES = (1, 2, 4, 8, 16, 25, 32)
BASE = dict(a_dtype="bfloat16", b_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu",
            c_dtype="bfloat16", sf_vec_size=32)


def _spec(major: str) -> dict:
    return {**BASE, "b_major": major, "sf_axis": major}


def _pack(seed: int, batch: int = BATCH):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    values = (torch.randn(batch * PACK_ROWS, K_KMAJ, device="cuda", generator=gen) * 0.1).to(
        torch.float8_e4m3fn)
    scales = torch.randint(118, 132, (batch * PACK_ROWS, K_KMAJ // 32), device="cuda",
                           generator=gen, dtype=torch.uint8)
    return values, scales


def _views(values, scales, batch: int = BATCH):
    v = values.view(batch, PACK_ROWS, K_KMAJ)
    s = scales.view(batch, PACK_ROWS, K_KMAJ // 32)
    return {"n": (v[:, :K_NMAJ, :], s[:, :K_NMAJ, :]),
            "k": (v[:, K_NMAJ:K_NMAJ + N_KMAJ, :], s[:, K_NMAJ:K_NMAJ + N_KMAJ, :])}


def _dequant(rhs) -> torch.Tensor:
    values, scales = rhs
    return values.to(torch.bfloat16) * scales.view(torch.float8_e8m0fnu).to(
        torch.bfloat16).repeat_interleave(32, dim=-1)


def _logical(rhs, major: str) -> torch.Tensor:
    d = _dequant(rhs)
    return d if major == "n" else d.transpose(1, 2)


def _dims(major: str):
    return (K_NMAJ, N_NMAJ) if major == "n" else (K_KMAJ, N_KMAJ)


def _strided_out(major: str, m: int, n: int, batch: int = BATCH):
    if major == "k":
        backing = torch.full((m, batch, n + 8), torch.nan, device="cuda", dtype=torch.bfloat16)
        return backing[..., :n].transpose(0, 1), backing[..., n:]
    return torch.empty(batch, m, n, device="cuda", dtype=torch.bfloat16), None


@pytest.fixture(scope="module")
def rhs_by_major():
    from sparkinfer_b200 import gemm

    views = _views(*_pack(7))
    for major, rhs in views.items():
        assert gemm.prewarm_bmm(rhs, M_VALUES, **_spec(major)) == len(M_VALUES)
    return views


def test_views_share_the_allocation():
    values, scales = _pack(11)
    views = _views(values, scales)
    for v, s in views.values():
        assert v.untyped_storage().data_ptr() == values.untyped_storage().data_ptr()
        assert s.untyped_storage().data_ptr() == scales.untyped_storage().data_ptr()
    assert views["n"][0].shape == (BATCH, K_NMAJ, N_NMAJ)
    assert views["k"][0].shape == (BATCH, N_KMAJ, K_KMAJ)
    assert views["k"][0].storage_offset() == K_NMAJ * K_KMAJ


@pytest.mark.parametrize("major", ["n", "k"])
def test_one_hot_rows_read_back_the_bf16_dequantization(rhs_by_major, major):
    from sparkinfer_b200 import gemm

    rhs = rhs_by_major[major]
    physical = _dequant(rhs)
    k, n = _dims(major)
    rows = torch.arange(32, device="cuda")
    for k0 in range(0, k, 32):
        lhs = torch.zeros(BATCH, 32, k, device="cuda", dtype=torch.bfloat16)
        lhs[:, rows, k0 + rows] = 1
        out = torch.empty(BATCH, 32, n, device="cuda", dtype=torch.bfloat16)
        returned = gemm.bmm(lhs, rhs, out, **_spec(major))
        expected = (physical[:, k0:k0 + 32, :] if major == "n"
                    else physical[:, :, k0:k0 + 32].transpose(1, 2))
        assert returned is out
        assert torch.equal(out, expected), f"dequantization differs at K={k0}"


@pytest.mark.parametrize("major", ["n", "k"])
def test_e8m0_boundary_bytes(rhs_by_major, major):
    from sparkinfer_b200 import gemm

    base_values, base_scales = rhs_by_major[major]
    values = torch.ones_like(base_values)
    scales = torch.full_like(base_scales, 127)
    k, n = _dims(major)
    lhs = torch.zeros(BATCH, 1, k, device="cuda", dtype=torch.bfloat16)
    lhs[:, :, 0] = 1
    for byte in (0, 1, 254, 255):
        scales.fill_(127)
        scales[:, :, 0] = byte
        out = torch.empty(BATCH, 1, n, device="cuda", dtype=torch.bfloat16)
        gemm.bmm(lhs, (values, scales), out, **_spec(major))
        physical = _dequant((values, scales))
        expected = physical[:, :1, :] if major == "n" else physical[:, :, :1].transpose(1, 2)
        nan = torch.isnan(expected)
        assert nan.any().item() == (byte == 255)
        assert torch.equal(torch.isnan(out), nan)
        assert torch.equal(out[~nan].contiguous().view(torch.uint16),
                           expected[~nan].contiguous().view(torch.uint16))


@pytest.mark.parametrize("major", ["n", "k"])
@pytest.mark.parametrize("m", M_VALUES)
def test_random_product_is_as_accurate_as_cublas(rhs_by_major, major, m):
    from sparkinfer_b200 import gemm

    rhs = rhs_by_major[major]
    logical = _logical(rhs, major)
    k, n = _dims(major)
    lhs = torch.randn(BATCH, m, k, device="cuda", dtype=torch.bfloat16)
    out = torch.full((BATCH, m, n), torch.nan, device="cuda", dtype=torch.bfloat16)
    gemm.bmm(lhs, rhs, out, **_spec(major))
    exact = torch.bmm(lhs.double(), logical.double())
    ours = (out.double() - exact).abs().max().item()
    cublas = (torch.bmm(lhs, logical).double() - exact).abs().max().item()
    assert torch.isfinite(out).all() and torch.count_nonzero(out) > 0
    assert ours <= cublas * 1.05 + 1e-12, (ours, cublas)
    # FP32 accumulation and one rounding: within half a BF16 step of the exact product.
    assert ((out.double() - exact).abs() <= exact.abs() * 2.0 ** -8 + 1e-3).all()


@pytest.mark.parametrize("major", ["n", "k"])
def test_repeated_launches_give_identical_bits(rhs_by_major, major):
    from sparkinfer_b200 import gemm

    rhs = rhs_by_major[major]
    k, n = _dims(major)
    lhs = torch.randn(BATCH, 8, k, device="cuda", dtype=torch.bfloat16)
    first = torch.empty(BATCH, 8, n, device="cuda", dtype=torch.bfloat16)
    second = torch.empty_like(first)
    gemm.bmm(lhs, rhs, first, **_spec(major))
    gemm.bmm(lhs, rhs, second, **_spec(major))
    assert torch.equal(first, second)


@pytest.mark.parametrize("major", ["n", "k"])
@pytest.mark.parametrize("m,batch", [(4, 16), (25, 16), (4, 8)])
def test_graph_replay_reads_fresh_input_and_keeps_the_padding(major, m, batch):
    from sparkinfer_b200 import gemm

    rhs = _views(*_pack(23, batch), batch)[major]
    k, n = _dims(major)
    assert gemm.can_implement_bmm(batch=batch, max_m=32, n=n, k=k, device="cuda", **_spec(major))
    lhs = torch.zeros(batch, m, k, device="cuda", dtype=torch.bfloat16)
    out, padding = _strided_out(major, m, n, batch)
    gemm.bmm(lhs, rhs, out, **_spec(major))     # nothing to compile: any M may be captured cold
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        assert gemm.bmm(lhs, rhs, out, **_spec(major)) is out
    fresh = torch.randn_like(lhs)
    lhs.copy_(fresh)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    eager = torch.empty(batch, m, n, device="cuda", dtype=torch.bfloat16)
    gemm.bmm(fresh, rhs, eager, **_spec(major))
    assert torch.equal(out, eager)
    if padding is not None:
        assert torch.isnan(padding).all()


@pytest.mark.parametrize("major", ["n", "k"])
def test_side_stream_launch(rhs_by_major, major):
    from sparkinfer_b200 import gemm

    rhs = rhs_by_major[major]
    k, n = _dims(major)
    side = torch.cuda.Stream()
    current = torch.cuda.current_stream()
    assert gemm.prewarm_bmm(rhs, (3,), stream=side, synchronize=False, **_spec(major)) == 1
    lhs = torch.randn(BATCH, 3, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(BATCH, 3, n, device="cuda", dtype=torch.bfloat16)
    side.wait_stream(current)
    assert gemm.bmm(lhs, rhs, out, stream=side, **_spec(major)) is out
    current.wait_stream(side)
    expected = torch.empty_like(out)
    gemm.bmm(lhs, rhs, expected, **_spec(major))
    assert torch.equal(out, expected)


@pytest.mark.parametrize("major", ["n", "k"])
def test_torch_compile_keeps_the_out_mutation(rhs_by_major, major):
    from sparkinfer_b200 import gemm

    rhs = rhs_by_major[major]
    k, n = _dims(major)

    def run(a, c):
        return gemm.bmm(a, rhs, c, **_spec(major))

    compiled = torch.compile(run, backend="aot_eager", fullgraph=True)
    for _ in range(2):
        lhs = torch.randn(BATCH, 2, k, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(BATCH, 2, n, device="cuda", dtype=torch.bfloat16)
        expected = torch.empty_like(out)
        gemm.bmm(lhs, rhs, expected, **_spec(major))
        assert compiled(lhs, out) is out
        assert torch.equal(out, expected)


def test_envelope_and_argument_errors(rhs_by_major):
    from sparkinfer_b200 import gemm

    rhs = rhs_by_major["n"]
    lhs = torch.zeros(BATCH, 1, K_NMAJ, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(BATCH, 1, N_NMAJ, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError, match="supports only"):
        gemm.bmm(lhs, rhs, out, **{**_spec("n"), "b_dtype": "bfloat16"})
    with pytest.raises(NotImplementedError, match="sf_axis to match b_major"):
        gemm.bmm(lhs, rhs, out, **{**_spec("n"), "sf_axis": "k"})
    with pytest.raises(ValueError, match="rhs values must be float8_e4m3fn"):
        gemm.bmm(lhs, (rhs[0].to(torch.bfloat16), rhs[1]), out, **_spec("n"))
    with pytest.raises(NotImplementedError, match="qualified"):
        gemm.bmm(lhs[:15], (rhs[0][:15], rhs[1][:15]), out[:15], **_spec("n"))
    shared = torch.zeros(BATCH * N_NMAJ, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="must not overlap lhs"):
        gemm.bmm(shared[: BATCH * K_NMAJ].view(BATCH, 1, K_NMAJ), rhs,
                 shared.view(BATCH, 1, N_NMAJ), **_spec("n"))
    kwargs = dict(batch=BATCH, max_m=32, n=N_NMAJ, k=K_NMAJ, device="cuda", **_spec("n"))
    assert gemm.can_implement_bmm(**kwargs)
    assert gemm.can_implement_bmm(**{**kwargs, "batch": 8})
    assert not gemm.can_implement_bmm(**{**kwargs, "max_m": 33})
    assert not gemm.can_implement_bmm(**{**kwargs, "batch": 15})
    assert not gemm.can_implement_bmm(**{**kwargs, "sf_axis": "k"})
    assert not gemm.can_implement_bmm(**{**kwargs, "b_dtype": "bfloat16"})


@pytest.mark.parametrize("idx", range(3))
def test_kernel_matches_the_oracle_on_the_golden_fixture(idx):
    """Inputs and FP64 product from the fixture generated with the reference test module's own
    torch reference; the oracle restates it; the kernel is the oracle's product accumulated in
    FP32 and rounded once to BF16."""
    from conftest import GOLDEN, bf16_bits_to_f32
    from oracle import blockscaled_oracle as O
    from sparkinfer_b200._lib import launch

    g = np.load(GOLDEN / "bmm_ref.npz")
    n_major = bool(g[f"major{idx}"][0])
    values = torch.from_numpy(g[f"values{idx}"]).cuda()
    scales = torch.from_numpy(g[f"scales{idx}"]).cuda()
    lhs = torch.from_numpy(g[f"lhs_bits{idx}"].view(np.int16)).cuda().view(torch.bfloat16)
    batch, m, k = lhs.shape
    n = values.shape[2] if n_major else values.shape[1]
    out = torch.full((batch, m, n), torch.nan, device="cuda", dtype=torch.bfloat16)
    launch.bmm_mxfp8(lhs, values.view(torch.float8_e4m3fn), scales, out, n_major=n_major,
                     batch=batch, m=m, n=n, k=k)
    torch.cuda.synchronize()
    exact = O.bmm_mxfp8(bf16_bits_to_f32(g[f"lhs_bits{idx}"]), g[f"values{idx}"],
                        g[f"scales{idx}"], n_major)
    np.testing.assert_allclose(exact, g[f"product{idx}"], rtol=1e-12, atol=0)
    got = out.float().cpu().numpy().astype(np.float64)
    # FP32 accumulation of exact products and one rounding to BF16: per output, 2^-8 of the
    # result plus 2^-20 of the sum of the products' magnitudes. Outputs whose partial sums can
    # leave the FP32 range (the fixture holds a 2^127 scale) are only required to be non-NaN.
    w = np.abs(O.dequantize_rowwise_mxfp8_bf16(g[f"values{idx}"], g[f"scales{idx}"])).astype(np.float64)
    magnitude = np.matmul(np.abs(bf16_bits_to_f32(g[f"lhs_bits{idx}"])).astype(np.float64),
                          w if n_major else np.swapaxes(w, -1, -2))
    safe = magnitude < 1.0e37
    assert safe.mean() > 0.75 and not np.isnan(got).any()
    bound = np.abs(exact) * 2.0 ** -8 + magnitude * 2.0 ** -20
    assert (np.abs(got - exact)[safe] <= bound[safe]).all()


def _launcher_cases():
    rng = np.random.default_rng(77)
    cases = []
    for i in range(16):
        n_major = bool(i % 2)
        batch = int(rng.choice([1, 3, 8, 16, 40]))
        m = int(rng.integers(1, 33))
        if n_major:
            n = 32 * int(rng.integers(1, 20))
            k = 8 * int(rng.integers(1, 90))
        else:
            n = int(rng.choice([1, 7, 32, 100, 256, 515]))
            k = 32 * int(rng.integers(1, 30))
        cases.append((i, n_major, batch, m, n, k))
    # K too long for the shared-memory-resident tensor-core kernel: the CUDA-core kernel.
    cases += [(16, False, 4, 5, 100, 2048), (17, True, 3, 32, 96, 1600), (18, False, 2, 19, 64, 4096),
              (19, True, 8, 12, 64, 2056)]
    return cases


@pytest.mark.parametrize("index,n_major,batch,m,n,k", _launcher_cases())
def test_launcher_handles_any_geometry_its_rules_allow(index, n_major, batch, m, n, k):
    """The C entry point is not limited to the qualified envelope: any batch, ragged N for
    K-major weights, K that leaves warps without work, padded strides."""
    from sparkinfer_b200._lib import launch

    gen = torch.Generator(device="cuda").manual_seed(500 + index)
    rows, inner = (k, n) if n_major else (n, k)
    pad = 16 * (index % 3)
    values = (torch.randn(batch, rows, inner + pad, device="cuda", generator=gen) * 0.5).to(
        torch.float8_e4m3fn)[:, :, :inner]
    scale_pad = 4 * (index % 2)
    scales = torch.randint(120, 131, (batch, rows, inner // 32 + scale_pad), device="cuda",
                           generator=gen, dtype=torch.uint8)[:, :, : inner // 32]
    lhs = torch.randn(batch, m, k + 8, device="cuda", generator=gen).to(torch.bfloat16)[:, :, :k]
    n_even = n + (n % 2)
    out = torch.full((batch, m, n_even + 2), torch.nan, device="cuda", dtype=torch.bfloat16)
    launch.bmm_mxfp8(lhs, values, scales, out, n_major=n_major, batch=batch, m=m, n=n, k=k)
    torch.cuda.synchronize()
    d = values.to(torch.bfloat16) * scales.view(torch.float8_e8m0fnu).to(
        torch.bfloat16).repeat_interleave(32, dim=-1)
    logical = d if n_major else d.transpose(1, 2)
    exact = torch.bmm(lhs.double(), logical.double())
    got = out[:, :, :n]
    assert torch.isnan(out[:, :, n:]).all(), "wrote past column N"
    assert torch.isfinite(got).all()
    tol = exact.abs() * 2.0 ** -8 + 2.0 ** -9 * float(exact.abs().max()) + 1e-6
    assert ((got.double() - exact).abs() <= tol).all()


def test_launcher_rejects_what_the_kernel_cannot_take():
    from sparkinfer_b200 import _native
    from sparkinfer_b200._lib import launch

    values = torch.zeros(2, 64, 64, device="cuda", dtype=torch.float8_e4m3fn)
    scales = torch.zeros(2, 64, 2, device="cuda", dtype=torch.uint8)
    out = torch.empty(2, 33, 64, device="cuda", dtype=torch.bfloat16)
    lhs = torch.zeros(2, 33, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(_native.NativeLibraryError):
        launch.bmm_mxfp8(lhs, values, scales, out, n_major=False, batch=2, m=33, n=64, k=64)
    with pytest.raises(_native.NativeLibraryError):   # rows of A off the 16-byte grid
        launch.bmm_mxfp8(lhs.view(-1)[1:1 + 2 * 4 * 64].view(2, 4, 64), values, scales,
                         out[:, :4], n_major=False, batch=2, m=4, n=64, k=64)
