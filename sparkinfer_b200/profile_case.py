"""Launch one kernel of the library a few times on seeded random operands.

    python -m sparkinfer_b200.profile_case <op> M N K [launches]

``op`` is one of ``mxfp8``, ``nvfp4`` (the tiled block-scaled GEMM, tile width chosen by the
library), ``decode_nvfp4``, ``decode_mxfp8`` (the small-M stream-K kernel), ``block_fp8``,
``quant_mxfp8``, ``quant_nvfp4`` (row quantizers; N is ignored). The program is what a profiler
is pointed at: few launches, nothing else on the device, operands sized by the caller. It prints
the CUDA-event time of the last launch and exits non-zero if a kernel reported a timed-out wait.
"""
from __future__ import annotations

import sys

import torch

from ._lib import launch

OPS = ("mxfp8", "nvfp4", "decode_nvfp4", "decode_mxfp8", "block_fp8", "quant_mxfp8", "quant_nvfp4")


def build_case(op: str, m: int, n: int, k: int, device: torch.device):
    """Returns a zero-argument callable that launches ``op`` once on the current stream."""
    g = torch.Generator(device=device).manual_seed(1)

    def codes(shape):
        # Bit pattern 0x37 keeps every E4M3 byte and both E2M1 nibbles finite and small.
        raw = torch.randint(0, 256, shape, dtype=torch.uint8, device=device, generator=g)
        return raw & 0x37

    if op in ("mxfp8", "nvfp4", "decode_nvfp4", "decode_mxfp8"):
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
        return lambda: launch.gemm_blockscaled(kind, a, sfa, b, sfb, c, None, m, n, k,
                                               block_n=0, small_m=small)
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


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 4:
        raise SystemExit(__doc__)
    op = argv[0]
    m, n, k = (int(v) for v in argv[1:4])
    launches = int(argv[4]) if len(argv) > 4 else 3
    device = torch.device("cuda:0")
    fn = build_case(op, m, n, k, device)
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
