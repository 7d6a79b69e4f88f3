"""Launch one kernel of the library a few times on seeded random operands.

    python profile_case.py <op> M N K [launches]
    python profile_case.py timeline_nvfp4 M N K [chain_length]

``op`` is one of ``mxfp8``, ``nvfp4`` (the tiled block-scaled GEMM, kernel and tile width chosen
by the library), ``pair_mxfp8``, ``pair_nvfp4`` (the CTA-pair kernel forced), ``mxfp4``,
``pair_mxfp4``, ``decode_mxfp4`` (E2M1 codes with UE8M0 scales per 32 elements), ``decode_nvfp4``,
``decode_mxfp8`` (the small-M stream-K kernel), ``fused_nvfp4``, ``fused_mxfp8`` (the same with
the activation quantizer fused in, M <= 16), ``block_fp8``, ``quant_mxfp8``, ``quant_nvfp4`` (row
quantizers; N is ignored), ``bmm_k``, ``bmm_n`` (the batched BF16 x MXFP8 product over 16 heads,
K-major or N-major weights, a different weight set each call). ``graph_<op>`` captures the
launches in one CUDA graph and prints the device time per call. The program is what a profiler is pointed at: few launches, nothing
else on the device, operands sized by the caller. It prints the CUDA-event time of the last
launch and exits non-zero if a kernel reported a timed-out wait.

``timeline_nvfp4`` instead replays a CUDA graph of ``chain_length`` decode GEMMs (each with its
own weight copy, back to back on one stream, as in a decode step) whose CTAs record global-timer
stamps, and prints where a GEMM's time goes: gap to the predecessor, set-up, dependency wait,
first operand bytes, the streaming phase, and the tail.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

from sparkinfer_b200 import _native  # noqa: E402
from sparkinfer_b200._lib import launch  # noqa: E402

OPS = ("mxfp8", "nvfp4", "pair_mxfp8", "pair_nvfp4", "decode_nvfp4", "decode_mxfp8",
       "fused_nvfp4", "fused_mxfp8", "fp8", "pair_fp8", "scatter2_nvfp4", "scatter4_nvfp4",
       "scatter8_nvfp4", "block_fp8", "quant_mxfp8", "quant_nvfp4", "mxfp4", "pair_mxfp4", "decode_mxfp4", "bmm_k", "bmm_n")


def build_case(op: str, m: int, n: int, k: int, device: torch.device):
    """Returns a zero-argument callable that launches ``op`` once on the current stream."""
    g = torch.Generator(device=device).manual_seed(1)

    def codes(shape):
        # Bit pattern 0x37 keeps every E4M3 byte and both E2M1 nibbles finite and small.
        raw = torch.randint(0, 256, shape, dtype=torch.uint8, device=device, generator=g)
        return raw & 0x37

    if op in ("fused_nvfp4", "fused_mxfp8"):
        kind = 0 if op.endswith("mxfp8") else 1
        row_bytes = k if kind == 0 else k // 2
        vec = 32 if kind == 0 else 16
        k_atoms = (k + vec * 4 - 1) // (vec * 4)
        x = torch.randn((m, k), device=device, generator=g).to(torch.bfloat16)
        b = codes((n, row_bytes))
        sfb = torch.full((((n + 127) // 128) * k_atoms * 512,), 127 if kind == 0 else 0x38,
                         dtype=torch.uint8, device=device)
        gs = torch.ones(1, device=device) if kind == 1 else None
        c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        return lambda: launch.gemm_smallm_fused_quant(kind, x, gs, b, sfb, c, None, m, n, k)
    if op in ("mxfp8", "nvfp4", "pair_mxfp8", "pair_nvfp4", "decode_nvfp4", "decode_mxfp8"):
        kind = 0 if op.endswith("mxfp8") else 1
        row_bytes = k if kind == 0 else k // 2
        vec = 32 if kind == 0 else 16
        k_atoms = (k + vec * 4 - 1) // (vec * 4)
        unit_scale = 127 if kind == 0 else 0x38  # 2^0 in UE8M0, 1.0 in E4M3
        a, b = codes((m, row_bytes)), codes((n, row_bytes))
        sfa = torch.full((((m + 127) // 128) * k_atoms * 512,), unit_scale, dtype=torch.uint8,
                         device=device)
        sfb = torch.full((((n + 127) // 128) * k_atoms * 512,), unit_scale, dtype=torch.uint8,
                         device=device)
        c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        small = op.startswith("decode")
        block_n = _native.BLOCK_N_PAIR if op.startswith("pair") else 0
        return lambda: launch.gemm_blockscaled(kind, a, sfa, b, sfb, c, None, m, n, k,
                                               block_n=block_n, small_m=small)
    if op in ("bmm_k", "bmm_n"):
        # 16 heads; 80 weight sets (160 MB, more than L2) taken in turn, as the layers of a
        # model would be.
        batch, sets, n_major = 16, 80, op == "bmm_n"
        rows, inner = (k, n) if n_major else (n, k)
        values = codes((sets, batch, rows, inner)).view(torch.float8_e4m3fn)
        scales = torch.full((sets, batch, rows, inner // 32), 127, dtype=torch.uint8, device=device)
        lhs = torch.randn((batch, m, k), device=device, generator=g).to(torch.bfloat16)
        out = torch.empty((batch, m, n), dtype=torch.bfloat16, device=device)
        turn = [0]

        def run():
            i = turn[0] = (turn[0] + 1) % sets
            launch.bmm_mxfp8(lhs, values[i], scales[i], out, n_major=n_major, batch=batch, m=m,
                             n=n, k=k)

        return run
    if op in ("mxfp4", "pair_mxfp4", "decode_mxfp4"):
        k_atoms = (k + 127) // 128
        a, b = codes((m, k // 2)), codes((n, k // 2))
        sfa = torch.full((((m + 127) // 128) * k_atoms * 512,), 127, dtype=torch.uint8, device=device)
        sfb = torch.full((((n + 127) // 128) * k_atoms * 512,), 127, dtype=torch.uint8, device=device)
        c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        block_n = _native.BLOCK_N_PAIR if op.startswith("pair") else 0
        return lambda: launch.gemm_blockscaled(_native.KIND_MXFP4, a, sfa, b, sfb, c, None, m, n, k,
                                               block_n=block_n, small_m=op.startswith("decode"))
    if op in ("fp8", "pair_fp8"):
        a, b = codes((m, k)), codes((n, k))
        c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        block_n = _native.BLOCK_N_PAIR if op.startswith("pair") else 0
        return lambda: launch.gemm_blockscaled(_native.KIND_FP8, a, None, b, None, c, None, m, n, k,
                                               block_n=block_n)
    if op in ("scatter2_nvfp4", "scatter4_nvfp4", "scatter8_nvfp4"):
        # The row-parallel GEMM of one rank with every slab owner's receive buffer on this GPU
        # (the scatter itself, without the links).
        world = int(op[7])
        k_atoms = (k + 63) // 64
        a, b = codes((m, k // 2)), codes((n, k // 2))
        sfa = torch.full((((m + 127) // 128) * k_atoms * 512,), 0x38, dtype=torch.uint8, device=device)
        sfb = torch.full((((n + 127) // 128) * k_atoms * 512,), 0x38, dtype=torch.uint8, device=device)
        recv = [torch.empty((m, n), dtype=torch.bfloat16, device=device) for _ in range(world)]
        ptrs = [t.data_ptr() for t in recv]

        def run(recv=recv):  # the closure keeps the receive buffers alive
            launch.gemm_blockscaled_scatter(1, a, sfa, b, sfb, ptrs, 0, torch.bfloat16, None, m, n, k)

        return run
    if op == "block_fp8":
        a, b = codes((m, k)), codes((n, k))
        sa = torch.rand((m, k // 128), device=device, generator=g) + 0.5
        sb = torch.rand(((n + 127) // 128, k // 128), device=device, generator=g) + 0.5
        c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        return lambda: launch.gemm_block_fp8(a, sa, b, sb, c, None, m, n, k)
    x = torch.randn((m, k), device=device, generator=g).to(torch.bfloat16)
    if op == "quant_mxfp8":
        v = torch.empty((m, k), dtype=torch.uint8, device=device)
        r = torch.empty((m, k // 32), dtype=torch.uint8, device=device)
        s = torch.empty((((m + 127) // 128) * ((k + 127) // 128) * 512,), dtype=torch.uint8,
                        device=device)
        return lambda: launch.quantize_mxfp8_rows(x, v, r, s)
    if op == "quant_nvfp4":
        gs = torch.ones(1, device=device)
        p = torch.empty((m, k // 2), dtype=torch.uint8, device=device)
        s = torch.empty((((m + 127) // 128) * ((k + 63) // 64) * 512,), dtype=torch.uint8,
                        device=device)
        return lambda: launch.quantize_nvfp4_rows(x, gs, p, s)
    raise SystemExit(f"unknown op {op!r}; expected one of {', '.join(OPS)}")


def timeline(m: int, n: int, k: int, chain: int, device: torch.device) -> int:
    """Replays a graph of `chain` decode GEMMs with per-CTA stamps and prints the medians."""
    g = torch.Generator(device=device).manual_seed(1)
    k_atoms = (k + 63) // 64
    x = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=device, generator=g) & 0x37
    sfx = torch.full((k_atoms * 512,), 0x38, dtype=torch.uint8, device=device)
    sfw = torch.full((((n + 127) // 128) * k_atoms * 512,), 0x38, dtype=torch.uint8, device=device)
    weights = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=g) & 0x37
               for _ in range(chain)]
    c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    stamps = torch.zeros((chain, sms * 8), dtype=torch.int64, device=device)

    def run():
        for i, w in enumerate(weights):
            launch.gemm_smallm_timeline(1, x, sfx, w, sfw, c, None, m, n, k, stamps[i])

    run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    rows = []
    for rep in range(5):
        flush.fill_(rep)
        stamps.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        t = stamps.view(chain, sms, 8).cpu().double()
        live = t[:, :, 0] > 0                      # CTAs that exist (grid may be smaller than the SMs)
        rows.append((start.elapsed_time(stop) * 1e3 / chain, t, live))
    launch.check_kernel_status(device)
    per_gemm_us, t, live = rows[-1]
    print(f"timeline_nvfp4 {m}x{n}x{k} chain={chain}: {per_gemm_us:.2f} us per GEMM (graph replay / chain), "
          f"{int(live[0].sum())} CTAs per GEMM")

    def med(v):
        return float(v.median()) / 1e3

    print("per GEMM i >= 1 (microseconds, medians over CTAs; 'first'/'last' over the whole grid):")
    print("  i  grid_start-prev_grid_end  entry->setup  setup->deps_done  entry->first_stage  "
          "first_stage->last_acc  last_acc->drained  drained->exit  grid_span")
    for i in range(1, chain):
        e, su, dd, fs, la, ex = (t[i, :, j][live[i]] for j in range(6))
        dr = t[i, :, 7][live[i]]
        prev_end = t[i - 1, :, 5][live[i - 1]].max()
        print(f"  {i}  {float(e.min() - prev_end) / 1e3:+8.2f}  {med(su - e):8.2f}  {med(dd - su):8.2f}  "
              f"{med(fs - e):8.2f}  {med(la - fs):8.2f}  {med(dr - la):8.2f}  {med(ex - dr):8.2f}  "
              f"{float(ex.max() - e.min()) / 1e3:8.2f}")
    e_all = [t[i, :, 0][live[i]].min() for i in range(chain)]
    period = [(float(e_all[i + 1] - e_all[i]) / 1e3) for i in range(chain - 1)]
    print("grid start to next grid start (us):", " ".join(f"{p:.2f}" for p in period))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 4:
        raise SystemExit(__doc__)
    op = argv[0]
    m, n, k = (int(v) for v in argv[1:4])
    launches = int(argv[4]) if len(argv) > 4 else 3
    device = torch.device("cuda:0")
    if op == "timeline_nvfp4":
        return timeline(m, n, k, max(launches, 2), device)
    graphed = op.startswith("graph_")
    fn = build_case(op[6:] if graphed else op, m, n, k, device)
    if graphed:
        # `launches` calls captured in one CUDA graph, replayed five times: device time per
        # call without the host's launch cost, for kernels of a few microseconds.
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(launches):
                fn()
        times = []
        for _ in range(5):
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / launches)
        launch.check_kernel_status(device)
        print(f"{op} {m}x{n}x{k} us_per_call={sorted(times)[2]:.2f} (median of 5 replays of "
              f"{launches} calls)")
        return 0
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    for i in range(launches):
        if i == launches - 1:
            start.record()
        fn()
    stop.record()
    torch.cuda.synchronize()
    launch.check_kernel_status(device)
    print(f"{op} {m}x{n}x{k} last_launch_ms={start.elapsed_time(stop):.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
