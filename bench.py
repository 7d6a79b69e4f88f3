#!/usr/bin/env python
"""Benchmark of the block-scaled GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0). A step is one pass of the hot path over one batch of
seeded synthetic operands of the named configuration. Timing: CUDA events on the launching
stream around every step, L2 flushed (a 256 MiB fill) between steps, max over ranks.

Workloads (the reference's configurations; seeds 42 + 1000*cfg + {0: A, 1: B}):
  cfg0_nvfp4_128x4096x4096         NVFP4 x NVFP4, BF16 out (pre-quantized operands)
  cfg1_nvfp4_decode_m{1,4,16,64}   activation quantize_rows + NVFP4 GEMM, N=14336 K=4096
  cfg2_mxfp8_prefill               quantize_rows + MXFP8 GEMM, 8192 x 7168 x 7168
  cfg3_block_fp8_colpar            E4M3 + FP32 block scales, 4096 x 18432 x 7168, N / gpus
  cfg4_nvfp4_rowpar                quantize_rows + NVFP4 GEMM + BF16 all-reduce,
                                   4096 x 7168 x 18432, K / gpus
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

NOMINAL = {"hbm_gbs": 8000.0, "fp8_tflops": 4500.0, "fp4_tflops": 9000.0}
DEFAULT_WORKLOAD = "cfg3_block_fp8_colpar"
L2_FLUSH_BYTES = 256 << 20

# DRAM bytes (read + write) of ONE launch of each workload's GEMM kernel on one GPU at the full
# size, from `ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum` captures of
# `python -m sparkinfer_b200.profile_case <op> M N K 3` (summaries under profiles/). Output
# bytes still held in the 126 MB L2 when the kernel ends are not in the write figure.
NCU_TRAFFIC_BYTES = {
    "cfg0_nvfp4_128x4096x4096": 9_763_584 + 0,
    "cfg1_nvfp4_decode_m16": 33_144_832 + 0,
    "cfg2_mxfp8_prefill": 268_549_632 + 98_470_400,
    "cfg3_block_fp8_colpar": 297_408_768 + 129_085_696,
    "cfg4_nvfp4_rowpar": 205_381_120 + 43_779_584,
}


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


# --------------------------------------------------------------------------------------
# Workload descriptions
# --------------------------------------------------------------------------------------
def workload_table() -> dict:
    t = {
        "cfg0_nvfp4_128x4096x4096": dict(cfg=0, kind="nvfp4", m=128, n=4096, k=4096, quant=False,
                                         shard=None, bound="hbm"),
        "cfg2_mxfp8_prefill": dict(cfg=2, kind="mxfp8", m=8192, n=7168, k=7168, quant=True,
                                   shard=None, bound="tensor"),
        "cfg3_block_fp8_colpar": dict(cfg=3, kind="block_fp8", m=4096, n=18432, k=7168,
                                      quant=False, shard="n", bound="tensor"),
        "cfg4_nvfp4_rowpar": dict(cfg=4, kind="nvfp4", m=4096, n=7168, k=18432, quant=True,
                                  shard="k", bound="tensor"),
    }
    for m in (1, 4, 16, 64):
        t[f"cfg1_nvfp4_decode_m{m}"] = dict(cfg=1, kind="nvfp4", m=m, n=14336, k=4096, quant=True,
                                            shard=None, bound="hbm")
    return t


def algorithmic_bytes(w: dict, n: int, k: int) -> int:
    """A + SFA + B + SFB + C of the GEMM (codes and scale bytes actually consumed)."""
    m = w["m"]
    if w["kind"] == "nvfp4":
        return m * k // 2 + m * k // 16 + n * k // 2 + n * k // 16 + m * n * 2
    if w["kind"] == "mxfp8":
        return m * k + m * k // 32 + n * k + n * k // 32 + m * n * 2
    return m * k + m * (k // 128) * 4 + n * k + (n // 128) * (k // 128) * 4 + m * n * 2


# --------------------------------------------------------------------------------------
# Clock sampling during the timed region
# --------------------------------------------------------------------------------------
class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) every ~2 ms from a thread
    while the timed region runs; falls back to one nvidia-smi query if NVML is unavailable."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.clocks: list[float] = []
        self.reason_bits = 0
        self.sm_max = None
        self._stop = threading.Event()
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    @staticmethod
    def _physical_index(index: int) -> int:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            try:
                return int(visible.split(",")[index])
            except (ValueError, IndexError):
                return index
        return index

    def _poll(self):
        if self._nvml is None:
            return
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.clocks.append(float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:
                break
            time.sleep(0.002)

    def stop(self) -> dict:
        self._stop.set()
        self.thread.join(timeout=1)
        if self._nvml is None or not self.clocks:
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", "--query-gpu=clocks.sm,clocks.max.sm",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10)
                a, b = [float(v) for v in out.stdout.strip().split(",")]
                return {"sm_mhz": a, "sm_max_mhz": b, "samples": 1, "reasons": [],
                        "note": "single nvidia-smi sample after the timed region"}
            except Exception:
                return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0,
                        "reasons": ["clock query unavailable"]}
        reasons = sorted(name for bit, name in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": float(np.median(self.clocks)), "sm_min_mhz": float(min(self.clocks)),
                "sm_max_mhz": self.sm_max, "samples": len(self.clocks), "reasons": reasons}


# --------------------------------------------------------------------------------------
# Synthetic operands (seeded, generated on the device, quantized by this package's ops or,
# for the block-FP8 recipe that has no quantizer op, by torch at set-up)
# --------------------------------------------------------------------------------------
def seeded_randn(seed: int, shape, scale: float, device) -> torch.Tensor:
    gen = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
    return (x * scale).to(torch.bfloat16)


def block_fp8_quantize(x: torch.Tensor, block_rows: int):
    """scales = amax / 448 over (block_rows x 128) blocks; codes = e4m3(v / s)."""
    r, c = x.shape
    t = x.float().view(r // block_rows, block_rows, c // 128, 128)
    amax = t.abs().amax(dim=(1, 3))
    s = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    codes = (t / s[:, None, :, None]).to(torch.float8_e4m3fn).view(r, c)
    return codes, s.contiguous()


class Step:
    """One configured step: device-resident operands plus the callable that runs the path."""

    def __init__(self, name: str, w: dict, rank: int, world: int, device, replicas: int = 1):
        from sparkinfer_b200.parallel import shard_range

        self.name, self.w, self.rank, self.world, self.device = name, w, rank, world, device
        m, n, k = w["m"], w["n"], w["k"]
        self.n_local, self.k_local = n, k
        n_shard = k_shard = None
        if w["shard"] == "n":
            n_shard = shard_range(n, world, rank)
            self.n_local = n_shard.size
        elif w["shard"] == "k":
            k_shard = shard_range(k, world, rank)
            self.k_local = k_shard.size
        seed = 42 + 1000 * w["cfg"]
        x = seeded_randn(seed, (m, k), 1.0, device)
        wt = seeded_randn(seed + 1, (n, k), 0.02 if w["kind"] != "block_fp8" else 1.0, device)
        self.kernels_per_step = 1
        self.h2d_bytes = self.d2h_bytes = 0
        self.group = 1          # consecutive steps captured together (HBM-bound workloads)
        self.replicas = replicas
        getattr(self, f"_setup_{w['kind']}")(x, wt, n_shard, k_shard)
        del x, wt
        torch.cuda.empty_cache()

    # ---- NVFP4: weights quantized once; activations quantized per call when quant=True ----
    def _setup_nvfp4(self, x, wt, n_shard, k_shard):
        from sparkinfer_b200.gemm import blockscaled
        from sparkinfer_b200.quantization import nvfp4
        from sparkinfer_b200.quantization.nvfp4._impl import BF16ToFP4TMAOutputs as BF16Outputs

        m, n, kl = self.w["m"], self.w["n"], self.k_local
        gs_x = (448.0 * 6.0 / x.float().abs().max()).reshape(1).float()
        gs_w = (448.0 * 6.0 / wt.float().abs().max()).reshape(1).float()
        if k_shard is not None:
            x = x[:, k_shard.begin:k_shard.end].contiguous()
            wt = wt[:, k_shard.begin:k_shard.end].contiguous()
        wplan = nvfp4.plan(n, kl)
        wq = nvfp4.allocate_outputs(wplan, device=self.device)
        nvfp4.run(plan=wplan, x=wt, global_scale=gs_w, outputs=wq)
        self.x, self.gs_x = x, gs_x
        self.xplan = nvfp4.plan(m, kl)
        self.xq = nvfp4.allocate_outputs(self.xplan, device=self.device)
        nvfp4.run(plan=self.xplan, x=x, global_scale=gs_x, outputs=self.xq)
        self.alpha = (1.0 / (gs_x * gs_w)).float()
        self.out = torch.empty((m, n, 1), dtype=torch.bfloat16, device=self.device)
        lhs = (self.xq.packed_a_view, self.xq.scale_mma_view(m, kl))
        kw = dict(ab_dtype="float4_e2m1fn", sf_dtype="float8_e4m3fn", sf_vec_size=16,
                  c_dtype="bfloat16", alpha=self.alpha)
        # HBM-bound workloads rotate over `replicas` copies of the weight (distinct addresses,
        # together larger than L2), so that consecutive steps in one graph all stream from HBM.
        self.group = max(1, self.replicas)
        rhs_list = []
        for r in range(self.group):
            codes = wq.packed_a_storage if r == 0 else wq.packed_a_storage.clone()
            scales = wq.scale_storage if r == 0 else wq.scale_storage.clone()
            rhs_list.append((codes.permute(1, 2, 0),
                             BF16Outputs(codes, scales).scale_mma_view(n, kl)))
        self.gemms = [(lambda rhs=rhs: blockscaled.mm(lhs, rhs, self.out, **kw)) for rhs in rhs_list]
        self.gemm = lambda: [g() for g in self.gemms]
        self.quant = (lambda: nvfp4.run(plan=self.xplan, x=self.x, global_scale=self.gs_x,
                                        outputs=self.xq)) if self.w["quant"] else None
        self.kernels_per_step = 2 if self.w["quant"] else 1
        self.host_in = x.cpu().pin_memory() if self.w["quant"] else None
        self.h2d_bytes = x.numel() * 2 if self.w["quant"] else (
            self.xq.packed_a_storage.numel() + self.xq.scale_storage.numel())
        self.d2h_bytes = self.out.numel() * 2

    def _setup_mxfp8(self, x, wt, n_shard, k_shard):
        from sparkinfer_b200._lib.mxfp8_rows import empty_mxfp8_rows_for_dense_gemm, quantize_mxfp8_rows
        from sparkinfer_b200.gemm import blockscaled

        m, n, k = self.w["m"], self.w["n"], self.w["k"]
        wq = empty_mxfp8_rows_for_dense_gemm(n, k, device=self.device)
        quantize_mxfp8_rows(wt, wq.values, wq.scale_rows, wq.scale_mma)
        self.x = x
        self.xq = empty_mxfp8_rows_for_dense_gemm(m, k, device=self.device)
        quantize_mxfp8_rows(x, self.xq.values, self.xq.scale_rows, self.xq.scale_mma)
        self.out = torch.empty((m, n, 1), dtype=torch.bfloat16, device=self.device)
        lhs = (self.xq.values.view(m, k, 1), self.xq.scale_mma)
        rhs = (wq.values.view(n, k, 1), wq.scale_mma)
        kw = dict(ab_dtype="float8_e4m3fn", sf_dtype="float8_e8m0fnu", sf_vec_size=32,
                  c_dtype="bfloat16")
        self.gemm = lambda: blockscaled.mm(lhs, rhs, self.out, **kw)
        self.quant = lambda: quantize_mxfp8_rows(self.x, self.xq.values, self.xq.scale_rows,
                                                 self.xq.scale_mma)
        self.kernels_per_step = 2
        self.host_in = x.cpu().pin_memory()
        self.h2d_bytes = x.numel() * 2
        self.d2h_bytes = self.out.numel() * 2

    def _setup_block_fp8(self, x, wt, n_shard, k_shard):
        from sparkinfer_b200.gemm import blockscaled

        m, k = self.w["m"], self.w["k"]
        if n_shard is not None:
            wt = wt[n_shard.begin:n_shard.end].contiguous()
        nl = wt.shape[0]
        a, sa = block_fp8_quantize(x, 1)
        b, sb = block_fp8_quantize(wt, 128)
        self.a, self.sa = a, sa
        self.out = torch.empty((m, nl, 1), dtype=torch.bfloat16, device=self.device)
        kw = dict(ab_dtype="float8_e4m3fn", sf_dtype="float32", sf_vec_size=128,
                  c_dtype="bfloat16", block_fp8=True)
        self.gemm = lambda: blockscaled.mm((a.view(m, k, 1), sa), (b.view(nl, k, 1), sb),
                                           self.out, **kw)
        self.quant = None
        self.host_in = None
        self.h2d_bytes = a.numel() + sa.numel() * 4
        self.d2h_bytes = self.out.numel() * 2

    def run(self):
        if self.group > 1:
            for g in self.gemms:
                if self.quant is not None:
                    self.quant()
                g()
            return
        if self.quant is not None:
            self.quant()
        self.gemm()
        if self.w["shard"] == "k" and self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(self.out)

    def flops(self) -> float:
        return 2.0 * self.w["m"] * self.w["n"] * self.w["k"]  # whole job, all ranks


# --------------------------------------------------------------------------------------
# Timing
# --------------------------------------------------------------------------------------
def capture(fn):
    """Capture ``fn`` (already warmed up) into a CUDA graph and return its replay; the
    reference times graph replays for the same reason (launch gaps dwarf micro-second
    kernels). Falls back to the eager callable if capture is refused."""
    try:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        torch.cuda.synchronize()
        return graph.replay
    except Exception:  # pragma: no cover - depends on the collective library
        torch.cuda.synchronize()
        return fn


def time_steps(fn, steps: int, warmup: int, flush: torch.Tensor, sync_ranks,
               use_graph: bool = True) -> list[float]:
    fn()
    if use_graph:
        fn = capture(fn)
    for _ in range(warmup):
        flush.fill_(1)
        fn()
    torch.cuda.synchronize()
    sync_ranks()
    begins = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.fill_(i & 1)  # evict operands and outputs from L2 between timed steps
        begins[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    sync_ranks()
    return [b.elapsed_time(e) for b, e in zip(begins, ends)]


def cpu_dequant_matmul(w: dict, sample_rows: int, seed: int = 7):
    """The oracle port of the reference's CPU path (dequantize to FP32, matmul) on a bounded
    sample: ``sample_rows`` rows of A against min(N, 2048) rows of B at full K. Returns
    (seconds, flops)."""
    from oracle import blockscaled_oracle as O

    rng = np.random.RandomState(seed)
    n = min(w["n"], 2048)
    k = w["k"]
    a = rng.standard_normal((sample_rows, k)).astype(np.float32)
    b = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if w["kind"] == "nvfp4":
        gsa, gsb = O.nvfp4_global_scale(a), O.nvfp4_global_scale(b)
        qa, qb = O.quantize_nvfp4_rows(a, gsa), O.quantize_nvfp4_rows(b, gsb)
        t0 = time.perf_counter()
        out = O.gemm_nvfp4(*qa, gsa, *qb, gsb)
    elif w["kind"] == "mxfp8":
        qa, qb = O.quantize_mxfp8_rows(a), O.quantize_mxfp8_rows(b)
        t0 = time.perf_counter()
        out = O.gemm_mxfp8(*qa, *qb)
    else:
        qa, qb = O.quantize_block_fp8(a, 1), O.quantize_block_fp8(b, 128)
        t0 = time.perf_counter()
        out = O.gemm_block_fp8(*qa, *qb)
    dt = time.perf_counter() - t0
    assert np.isfinite(out).all()
    return dt, 2.0 * sample_rows * n * k


def cpu_baseline(w: dict, limit_s: float = 12.0) -> dict:
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rows = min(w["m"], 256)
    dt, flops = cpu_dequant_matmul(w, rows)
    reps, total_t, total_f = 1, dt, flops
    while total_t < limit_s and reps < 8:
        dt, flops = cpu_dequant_matmul(w, rows, seed=7 + reps)
        total_t += dt
        total_f += flops
        reps += 1
    return {"value": total_f / total_t / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{reps} x ({rows} rows of A) x ({min(w['n'], 2048)} rows of B) x K={w['k']}, "
                      "oracle dequantize-to-FP32 + NumPy matmul (dequantize inside the timed region)"}


# --------------------------------------------------------------------------------------
# Main
# --------------------------------------------------------------------------------------
def run_reference_arm(args, w: dict, name: str, rank: int) -> None:
    if rank != 0:
        return
    vals = []
    for _ in range(args.warmup):
        cpu_dequant_matmul(w, min(w["m"], 256))
    t_all = 0.0
    for i in range(args.steps):
        dt, flops = cpu_dequant_matmul(w, min(w["m"], 256), seed=100 + i)
        vals.append(flops / dt / 1e12)
        t_all += dt
    value = float(np.mean(vals))
    cores = os.cpu_count() or 1
    sample = (f"each step: {min(w['m'], 256)} rows of A x {min(w['n'], 2048)} rows of B x "
              f"K={w['k']} of the {name} operands, oracle port of the reference's CPU "
              "dequantize-matmul")
    print(json.dumps({
        "impl": "reference", "metric": "block-scaled GEMM TFLOPS", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t_all / max(args.steps, 1) * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": w["kind"], "data": "synthetic",
        "config": {"workload": name, "m": w["m"], "n": w["n"], "k": w["k"]},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def measure(step: Step, args, flush, sync_ranks, reduce_max):
    """(ms per step, ms per GEMM launch). With a replica group, one timed graph replay holds
    `group` consecutive steps and `args.steps` is a multiple of it."""
    replays = max(1, args.steps // step.group)
    times = time_steps(step.run, replays, args.warmup, flush, sync_ranks)
    total_ms = reduce_max(sum(times))
    gemm_times = time_steps(step.gemm, max(1, min(args.steps, 20) // step.group), 3, flush, sync_ranks)
    gemm_ms = float(np.mean(gemm_times)) / step.group
    return total_ms / (replays * step.group), gemm_ms, times


def replicas_for(w: dict, steps: int) -> int:
    """Weight copies for an HBM-bound workload: the smallest divisor of `steps` whose copies
    together exceed 1.5x the 126 MB L2; 1 (flush between steps instead) if there is none."""
    if w["bound"] != "hbm":
        return 1
    weight_bytes = w["n"] * w["k"] // 2 * 1.125
    need = int(np.ceil(1.5 * 126e6 / weight_bytes))
    for r in range(need, min(steps, 4 * need) + 1):
        if steps % r == 0:
            return r
    return 1


def measure_e2e(step: Step, args, flush, sync_ranks, reduce_max) -> float:
    """Same step with HOST operands: pinned activation -> device, run, output -> host."""
    out_host = torch.empty(step.out.shape, dtype=step.out.dtype).pin_memory()
    if step.host_in is not None:
        dst = step.x

        def h2d():
            dst.copy_(step.host_in, non_blocking=True)
    elif step.w["kind"] == "block_fp8":
        ha, hs = step.a.cpu().pin_memory(), step.sa.cpu().pin_memory()

        def h2d():
            step.a.copy_(ha, non_blocking=True)
            step.sa.copy_(hs, non_blocking=True)
    else:
        hp = step.xq.packed_a_storage.cpu().pin_memory()
        hs = step.xq.scale_storage.cpu().pin_memory()

        def h2d():
            step.xq.packed_a_storage.copy_(hp, non_blocking=True)
            step.xq.scale_storage.copy_(hs, non_blocking=True)

    def fn():
        h2d()
        step.run()
        out_host.copy_(step.out, non_blocking=True)

    times = time_steps(fn, max(3, min(args.steps, 10)), 3, flush, sync_ranks, use_graph=False)
    return reduce_max(float(np.mean(times)))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the per-configuration table")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    table = workload_table()
    if args.workload not in table:
        raise SystemExit(f"unknown workload {args.workload!r}; choose from {sorted(table)}")
    w = table[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, w, args.workload, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for these ops)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    import torch.distributed as dist

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def sync_ranks():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(value: float) -> float:
        if world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peaks = measured_peaks()
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    step = Step(args.workload, w, rank, world, device, replicas=replicas_for(w, args.steps))
    step.run()
    sync_ranks()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_per_step, gemm_ms, _ = measure(step, args, flush, sync_ranks, reduce_max)
    clocks = sampler.stop() if sampler else None
    e2e_ms = measure_e2e(step, args, flush, sync_ranks, reduce_max)

    from sparkinfer_b200._lib.launch import check_kernel_status

    check_kernel_status(device)

    tensor_peak = peaks["bf16_tflops"] * (4 if w["kind"] == "nvfp4" else 2)
    nominal_tensor = NOMINAL["fp4_tflops"] if w["kind"] == "nvfp4" else NOMINAL["fp8_tflops"]
    flops_local = 2.0 * w["m"] * step.n_local * step.k_local
    bytes_local = algorithmic_bytes(w, step.n_local, step.k_local)
    traffic = NCU_TRAFFIC_BYTES.get(args.workload) if world == 1 else None
    if w["bound"] == "tensor":
        achieved = flops_local / gemm_ms / 1e9
        roofline = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak,
                    "unit": "TFLOP/s", "frac": achieved / tensor_peak, "traffic": traffic,
                    "peak_source": f"{peaks['source']} BF16 cuBLAS burst x"
                                   f"{4 if w['kind'] == 'nvfp4' else 2} (no FP8/FP4 figure is measured)",
                    "frac_of_nominal": achieved / nominal_tensor, "kernel_ms": gemm_ms,
                    "algorithmic_bytes": bytes_local}
    else:
        achieved = bytes_local / gemm_ms / 1e6
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                    "peak_source": f"{peaks['source']} copy bandwidth",
                    "frac_of_nominal": achieved / NOMINAL["hbm_gbs"], "kernel_ms": gemm_ms,
                    "algorithmic_bytes": bytes_local}

    extra = {}
    if world == 1 and not args.no_extra:
        for name, other in table.items():
            if name == args.workload:
                continue
            try:
                s = Step(name, other, 0, 1, device, replicas=replicas_for(other, 24))
                s.run()
                torch.cuda.synchronize()
                t_all = float(np.mean(time_steps(s.run, max(1, 24 // s.group), 3, flush, sync_ranks))) / s.group
                t_gemm = float(np.mean(time_steps(s.gemm, max(1, 24 // s.group), 3, flush, sync_ranks))) / s.group
                extra[name] = {
                    "ms_per_step": t_all, "gemm_ms": t_gemm,
                    "tflops": 2.0 * other["m"] * other["n"] * other["k"] / t_gemm / 1e9,
                    "gbs": algorithmic_bytes(other, other["n"], other["k"]) / t_gemm / 1e6,
                }
                del s
                torch.cuda.empty_cache()
            except Exception as exc:  # keep the headline line even if a side config fails
                extra[name] = {"error": str(exc)[:160]}

    if rank == 0:
        baseline = cpu_baseline(w) if world == 1 else None
        value = step.flops() / ms_per_step / 1e9
        line = {
            "metric": "block-scaled GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": max(1, args.steps // step.group) * step.group,
            "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if w["shard"] else "weak", "vs_baseline": None,
            "dtype": {"nvfp4": "fp4_e2m1 x ue4m3 -> f32", "mxfp8": "fp8_e4m3 x ue8m0 -> f32",
                      "block_fp8": "fp8_e4m3 x f32 scales -> f32"}[w["kind"]],
            "data": "synthetic",
            "config": {"workload": args.workload, "m": w["m"], "n": w["n"], "k": w["k"],
                       "sharding": {"n": "column-parallel N/gpus, no communication",
                                    "k": "row-parallel K/gpus + NCCL BF16 all-reduce",
                                    None: "single GPU"}[w["shard"]],
                       "step": ("activation quantize_rows + " if w["quant"] else "") + "GEMM"
                               + (" + all-reduce" if w["shard"] == "k" and world > 1 else ""),
                       "l2": ("256 MiB fill between timed steps" if step.group == 1 else
                              f"{step.group} rotating weight copies per graph replay (larger than "
                              "L2 together) + 256 MiB fill between replays")},
            "roofline": roofline,
            "e2e": {"value": step.flops() / e2e_ms / 1e9, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": step.h2d_bytes, "d2h_bytes_per_step": step.d2h_bytes,
                    "ms_per_step": e2e_ms},
            "gpu_launches": (max(1, args.steps // step.group) * step.group * step.kernels_per_step),
            "clocks": clocks,
            "pct_of_nominal_peak": 100.0 * value / world / nominal_tensor,
        }
        if baseline is not None:
            line["cpu_baseline"] = baseline
        if extra:
            line["configs"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
