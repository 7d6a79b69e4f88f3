#!/usr/bin/env python
"""Benchmark of the block-scaled GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0). A step is one pass of the hot path over one batch of
seeded synthetic operands of the named configuration. Timing: CUDA events on the launching
stream around every step, L2 flushed (a 256 MiB fill) between steps, max over ranks.

Operands are generated on the CPU (torch.Generator, seeds 42 + 1000*cfg + {0: A, 1: B}, FP32
randn cast to BF16) so that the GPU arm, the CPU arm (`--impl reference`, `cpu_baseline`) and
the oracle parity check in the line all see the same bits.

Workloads (the reference's configurations):
  cfg0_nvfp4_128x4096x4096         NVFP4 x NVFP4, BF16 out (pre-quantized operands)
  cfg1_nvfp4_decode_m{1,4,16,64}   activation quantize_rows + NVFP4 GEMM, N=14336 K=4096
  cfg1_nvfp4_decode_m{1,4,16}_fused  the same step as one kernel (quantizer fused in)
  cfg2_mxfp8_prefill               quantize_rows + MXFP8 GEMM, 8192 x 7168 x 7168
  cfg3_block_fp8_colpar            E4M3 + FP32 block scales, 4096 x 18432 x 7168, N / gpus
  cfg4_nvfp4_rowpar                quantize_rows + NVFP4 GEMM + BF16 sum over the ranks,
                                   4096 x 7168 x 18432, K / gpus. The sum is this package's
                                   own code over NVLink peer memory, fused into the GEMM's
                                   epilogue (B12X_BENCH_COLLECTIVE=fused, the default), or its
                                   stand-alone all-reduce kernel (=peer), or NCCL (=nccl);
                                   NCCL's time on the same bytes is reported beside it.
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
# Collective of the K-split (row-parallel) step on several GPUs: "fused" = the GEMM scatters its
# output tiles to the slab owners over NVLink peer memory while it runs and this package's
# reduction kernel adds and broadcasts the slabs; "peer" = plain GEMM, then this package's
# all-reduce kernel over peer memory; "nccl" = plain GEMM, then torch.distributed all_reduce.
COLLECTIVE = os.environ.get("B12X_BENCH_COLLECTIVE", "fused")
# Row pieces of the end-to-end (host buffers) measurement of the block-FP8 workload: 1 = copy
# everything in, multiply, copy everything out; more = the same work pipelined piece by piece.
E2E_ROW_CHUNKS = max(1, int(os.environ.get("B12X_BENCH_E2E_CHUNKS", "8")))

# DRAM bytes (read + write) of ONE launch of each workload's GEMM kernel on one GPU at the full
# size, from `ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum` captures of
# `python profile_case.py <op> M N K 3` (summaries under profiles/). Output
# bytes still held in the 126 MB L2 when the kernel ends are not in the write figure.
NCU_TRAFFIC_BYTES = {
    "cfg0_nvfp4_128x4096x4096": 9_762_816 + 0,
    "cfg1_nvfp4_decode_m16": 33_151_232 + 256,
    "cfg2_mxfp8_prefill": 286_378_496 + 115_882_496,
    "cfg3_block_fp8_colpar": 298_083_840 + 131_562_752,
    "cfg4_nvfp4_rowpar": 223_142_656 + 62_427_648,
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
    for m in (1, 4, 16):
        t[f"cfg1_nvfp4_decode_m{m}_fused"] = dict(cfg=1, kind="nvfp4", m=m, n=14336, k=4096,
                                                  quant=True, fused=True, shard=None, bound="hbm")
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
# Synthetic operands (seeded, generated on the CPU, quantized by this package's ops or, for
# the block-FP8 recipe that has no quantizer op, by torch at set-up)
# --------------------------------------------------------------------------------------
def seeded_randn_cpu(seed: int, shape, scale: float) -> torch.Tensor:
    """BF16 [rows, k] from a CPU generator: the first r rows of a larger tensor with the same
    seed and k are these r rows (the sampler fills in row order), which is what lets the CPU
    arm work on a leading block of the GPU arm's operands."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=gen, dtype=torch.float32)
    return (x * scale).to(torch.bfloat16)


def operand_scales(w: dict) -> tuple[float, float]:
    return 1.0, (0.02 if w["kind"] != "block_fp8" else 1.0)


PARITY_ROWS = 16
PARITY_COLS = 64


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
        sx, sw = operand_scales(w)
        x_cpu = seeded_randn_cpu(seed, (m, k), sx)
        wt_cpu = seeded_randn_cpu(seed + 1, (n, k), sw)
        # Leading rows of A and the rows of B behind this rank's leading output columns, kept on
        # the host (full K) for the oracle parity check of the output.
        n0 = n_shard.begin if n_shard is not None else 0
        self.parity_x = x_cpu[:min(PARITY_ROWS, m)].clone()
        self.parity_w = wt_cpu[n0:n0 + min(PARITY_COLS, self.n_local)].clone()
        self.amax_x = float(x_cpu.float().abs().max())
        self.amax_w = float(wt_cpu.float().abs().max())
        x, wt = x_cpu.to(device), wt_cpu.to(device)
        del x_cpu, wt_cpu
        self.kernels_per_step = 1
        self.reducer, self.collective = None, "none"
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
        self.x, self.gs_x, self.gs_w = x, gs_x, gs_w
        self.xplan = nvfp4.plan(m, kl)
        self.xq = nvfp4.allocate_outputs(self.xplan, device=self.device)
        nvfp4.run(plan=self.xplan, x=x, global_scale=gs_x, outputs=self.xq)
        self.alpha = (1.0 / (gs_x * gs_w)).float()
        self.out = self._output_buffer(m, n)
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
        self.fused = bool(self.w.get("fused"))
        if self.fused:
            # One kernel per step: the decode GEMM quantizes the BF16 rows itself.
            self.gemms = [(lambda rhs=rhs: blockscaled.mm_fused_quant_a_nvfp4(
                self.x, self.gs_x, rhs[0], rhs[1], alpha=self.alpha, out=self.out))
                for rhs in rhs_list]
        else:
            self.gemms = [(lambda rhs=rhs: blockscaled.mm(lhs, rhs, self.out, **kw))
                          for rhs in rhs_list]
        self.gemm = lambda: [g() for g in self.gemms]
        if self.reducer is not None and self.reducer.scatter:
            from sparkinfer_b200 import _native

            self.gemm = lambda: self.reducer.gemm(
                _native.KIND_NVFP4, self.xq.packed_a_storage, self.xq.scale_storage,
                wq.packed_a_storage, wq.scale_storage, self.alpha, kl)
        self.quant = (lambda: nvfp4.run(plan=self.xplan, x=self.x, global_scale=self.gs_x,
                                        outputs=self.xq)) if (self.w["quant"] and not self.fused) else None
        self.kernels_per_step = 2 if self.quant is not None else 1
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

    def _output_buffer(self, m: int, n: int) -> torch.Tensor:
        """Output of a K-split step on several GPUs: the peer-mapped buffer of this package's
        all-reduce kernel, so that the GEMM writes its partial where the kernel sums it. All
        ranks agree on whether the peer mapping came up; if it did not on any of them, the
        step uses NCCL and the line says so."""
        self.reducer = None
        self.collective = "none"
        if self.w["shard"] == "k" and self.world > 1:
            import torch.distributed as dist

            from sparkinfer_b200.parallel import PeerAllReduce

            self.collective = "nccl all_reduce"
            reducer, why = None, ""
            if COLLECTIVE in ("peer", "fused"):
                scatter = COLLECTIVE == "fused" and m % (256 * self.world) == 0
                try:
                    reducer = PeerAllReduce(m, n, torch.bfloat16, device=self.device, scatter=scatter)
                except Exception as exc:  # no symmetric memory on this box
                    why = f"{type(exc).__name__}: {str(exc)[:120]}"
            ok = torch.tensor([1 if reducer is not None else 0], device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 1:
                self.reducer = reducer
                self.collective = (
                    "b12x_b200_gemm_blockscaled_scatter + b12x_b200_allreduce_peer_scattered "
                    "(GEMM tiles scattered to slab owners over NVLink peer memory, own reduction kernel)"
                    if reducer.scatter else
                    "b12x_b200_allreduce_peer (own kernel, NVLink peer memory)")
                return reducer.result.view(m, n, 1)
            if COLLECTIVE in ("peer", "fused"):
                self.collective += f" (peer memory unavailable: {why or 'on another rank'})"
        return torch.empty((m, n, 1), dtype=torch.bfloat16, device=self.device)

    def all_reduce(self):
        if self.reducer is not None:
            self.reducer()
        else:
            import torch.distributed as dist

            dist.all_reduce(self.out)

    def _setup_block_fp8(self, x, wt, n_shard, k_shard):
        from sparkinfer_b200.gemm import blockscaled

        m, k = self.w["m"], self.w["k"]
        if n_shard is not None:
            wt = wt[n_shard.begin:n_shard.end].contiguous()
        nl = wt.shape[0]
        a, sa = block_fp8_quantize(x, 1)
        b, sb = block_fp8_quantize(wt, 128)
        self.a, self.sa, self.b, self.sb = a, sa, b, sb
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
            self.all_reduce()

    def flops(self) -> float:
        return 2.0 * self.w["m"] * self.w["n"] * self.w["k"]  # whole job, all ranks

    def parity(self) -> dict:
        """Leading PARITY_ROWS x PARITY_COLS block of the output of the last step against the
        oracle (quantize the same BF16 rows on the CPU, dequantize to FP32, matmul). The bar is
        the path's tolerance, max|err| <= 1e-2 * max|ref|; for row-parallel runs the output is
        the all-reduced sum of the ranks' BF16 partials and still has to meet it."""
        from oracle import blockscaled_oracle as O

        rows, cols = self.parity_x.shape[0], self.parity_w.shape[0]
        got = self.out[:rows, :cols, 0].float().cpu().numpy()
        xa, wb = self.parity_x.float().numpy(), self.parity_w.float().numpy()
        if self.w["kind"] == "nvfp4":
            gsx, gsw = np.float32(self.gs_x.item()), np.float32(self.gs_w.item())
            ref = (O.dequantize_nvfp4(*O.quantize_nvfp4_rows(xa, gsx), gsx)
                   @ O.dequantize_nvfp4(*O.quantize_nvfp4_rows(wb, gsw), gsw).T)
        elif self.w["kind"] == "mxfp8":
            ref = (O.dequantize_mxfp8(*O.quantize_mxfp8_rows(xa))
                   @ O.dequantize_mxfp8(*O.quantize_mxfp8_rows(wb)).T)
        else:
            # No quantizer op exists for this recipe: the codes and FP32 scales the GEMM consumed
            # are read back (whole 128-row weight blocks) and multiplied by the oracle.
            blk = -(-cols // 128)
            ref = O.gemm_block_fp8(self.a[:rows].view(torch.uint8).cpu().numpy(),
                                   self.sa[:rows].cpu().numpy(),
                                   self.b[:blk * 128].view(torch.uint8).cpu().numpy(),
                                   self.sb[:blk].cpu().numpy())[:, :cols]
        scale = float(np.abs(ref).max())
        err = float(np.abs(got - ref).max())
        return {"max_err": err, "max_ref": scale, "tolerance": 1e-2 * scale,
                "ok": bool(err <= 1e-2 * scale), "block": f"{rows}x{cols} leading block vs oracle"}


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


# --------------------------------------------------------------------------------------
# CPU arm: the reference's CPU-runnable path (dequantize to FP32, torch.matmul) on a leading
# block of the workload's own operands, dequantize and matmul timed separately
# --------------------------------------------------------------------------------------
E2M1_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


class CpuReference:
    """Threaded torch restatement of the reference's CPU dequantize-matmul
    (tests/_reference/helpers.py:324-341, b12x/gemm/_shared/wo_mxfp8.py:1921-1943,
    tests/gemm/test_gemm_stack.py:98-113) on the first `ra` rows of the workload's A and the
    first `rb` rows of its B at full K. The quantized sample is built outside the timed region
    by torch restatements of the oracle's quantizers; both directions are checked against the
    NumPy oracle on a few rows when the object is built.

    One `step()` times dequantize(A sample), dequantize(B sample) and the FP32 matmul
    separately. The whole-configuration time is extrapolated by rows:
        dequant_s = t_dequant_A * M / ra + t_dequant_B * N / rb
        matmul_s  = t_matmul * (M * N) / (ra * rb)
    and the reported rate is 2 * M * N * K / (dequant_s + matmul_s)."""

    def __init__(self, w: dict, name: str):
        from oracle import blockscaled_oracle as O

        self.w, self.name = w, name
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        m, n, k = w["m"], w["n"], w["k"]
        self.ra, self.rb = min(m, 2048), min(n, 4096)
        seed = 42 + 1000 * w["cfg"]
        sx, sw = operand_scales(w)
        x = seeded_randn_cpu(seed, (self.ra, k), sx).float()
        wt = seeded_randn_cpu(seed + 1, (self.rb, k), sw).float()
        kind = w["kind"]
        if kind == "nvfp4":
            # The global scales come from the sample's own maxima (the GPU arm derives them from
            # the whole tensors; timing does not depend on the value).
            self.gs = [float(448.0 * 6.0 / t.abs().max()) for t in (x, wt)]
            self.q = [self._quant_nvfp4(t, g) for t, g in zip((x, wt), self.gs)]
            for (codes, scales), g, t in zip(self.q, self.gs, (x, wt)):
                pa, sa = O.quantize_nvfp4_rows(t[:4].numpy(), np.float32(g))
                assert np.array_equal(codes[:4].numpy(), pa) and np.array_equal(
                    scales[:4].view(torch.uint8).numpy(), sa), "torch NVFP4 quantizer != oracle"
                assert np.array_equal(self._deq_nvfp4(codes[:4], scales[:4], g).numpy(),
                                      O.dequantize_nvfp4(pa, sa, np.float32(g)))
        elif kind == "mxfp8":
            self.q = [self._quant_mxfp8(t) for t in (x, wt)]
            for (codes, scales), t in zip(self.q, (x, wt)):
                va, sr = O.quantize_mxfp8_rows(t[:4].numpy())
                assert np.array_equal(codes[:4].view(torch.uint8).numpy(), va) and np.array_equal(
                    scales[:4].numpy(), sr), "torch MXFP8 quantizer != oracle"
                assert np.array_equal(self._deq_mxfp8(codes[:4], scales[:4]).numpy(),
                                      O.dequantize_mxfp8(va, sr))
        else:
            self.q = [block_fp8_quantize(x, 1), block_fp8_quantize(wt, 128)]
            a8, sa = self.q[0]
            b8, sb = self.q[1]
            ref = O.gemm_block_fp8(a8[:4].view(torch.uint8).numpy(), sa[:4].numpy(),
                                   b8[:128].view(torch.uint8).numpy(), sb[:1].numpy())
            mine = self._deq_block_fp8(a8[:4], sa[:4], 1) @ self._deq_block_fp8(b8[:128], sb[:1], 128).T
            assert np.abs(mine.numpy() - ref).max() <= 1e-5 * np.abs(ref).max(), \
                "torch block-FP8 dequantize-matmul != oracle"

    # ---- quantizers (set-up only) ----
    @staticmethod
    def _quant_nvfp4(x: torch.Tensor, gs: float):
        r, k = x.shape
        blocks = x.view(r, k // 16, 16)
        gs_t = torch.tensor(gs, dtype=torch.float32)
        s = gs_t * (blocks.abs().amax(-1) / 6.0)
        s_q = s.to(torch.float8_e4m3fn)
        t = s_q.float() * (torch.tensor(1.0) / gs_t)
        inv = torch.where(t == 0, torch.zeros_like(t), 1.0 / t)
        y = (blocks * inv[:, :, None]).clamp_(-6.0, 6.0)
        mag = y.abs()
        bounds = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
        ties_up = (0.75, 1.75, 3.5)  # round-to-nearest-even on the E2M1 grid
        idx = torch.zeros(mag.shape, dtype=torch.uint8)
        for b in bounds:
            idx += (mag >= b).to(torch.uint8) if b in ties_up else (mag > b).to(torch.uint8)
        codes = (idx | (((y < 0) & (idx > 0)).to(torch.uint8) << 3)).view(r, k // 2, 2)
        return (codes[..., 0] | (codes[..., 1] << 4)).contiguous(), s_q.contiguous()

    @staticmethod
    def _quant_mxfp8(x: torch.Tensor):
        r, k = x.shape
        blocks = x.view(r, k // 32, 32)
        amax = blocks.abs().amax(-1)
        mant, exp = torch.frexp(amax / 448.0)           # v = mant * 2^exp, mant in [0.5, 1)
        e = torch.where(mant > 0.5, exp, exp - 1).clamp_(-127, 127)
        byte = torch.where(amax > 0, e + 127, torch.full_like(e, 127)).to(torch.uint8)
        inv = torch.exp2(127.0 - byte.float())
        q = (blocks * inv[:, :, None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
        return q.view(r, k).contiguous(), byte.contiguous()

    # ---- dequantizers (timed) ----
    @staticmethod
    def _deq_nvfp4(packed: torch.Tensor, scales: torch.Tensor, gs: float) -> torch.Tensor:
        r, kb = packed.shape
        lut = torch.tensor(E2M1_VALUES, dtype=torch.float32)
        vals = torch.stack((lut[(packed & 0xF).long()], lut[(packed >> 4).long()]), dim=-1)
        # value * scale / global_scale, in that order (tests/_reference/helpers.py:324-341)
        sf = scales.float()
        return (vals.view(r, kb * 2 // 16, 16) * sf[:, :, None]
                / torch.tensor(gs, dtype=torch.float32)).view(r, kb * 2)

    @staticmethod
    def _deq_mxfp8(codes: torch.Tensor, scale_rows: torch.Tensor) -> torch.Tensor:
        r, k = codes.shape
        sf = torch.exp2(scale_rows.float() - 127.0)
        return (codes.float().view(r, k // 32, 32) * sf[:, :, None]).view(r, k)

    @staticmethod
    def _deq_block_fp8(codes: torch.Tensor, scale: torch.Tensor, block_rows: int) -> torch.Tensor:
        r, k = codes.shape
        return (codes.float().view(r // block_rows, block_rows, k // 128, 128)
                * scale[:, None, :, None]).view(r, k)

    def _dequant(self, which: int) -> torch.Tensor:
        kind = self.w["kind"]
        if kind == "nvfp4":
            return self._deq_nvfp4(*self.q[which], self.gs[which])
        if kind == "mxfp8":
            return self._deq_mxfp8(*self.q[which])
        return self._deq_block_fp8(*self.q[which], 1 if which == 0 else 128)

    def step(self) -> dict:
        t0 = time.perf_counter()
        a = self._dequant(0)
        t1 = time.perf_counter()
        b = self._dequant(1)
        t2 = time.perf_counter()
        out = a @ b.T
        t3 = time.perf_counter()
        assert bool(torch.isfinite(out).all())
        m, n, k = self.w["m"], self.w["n"], self.w["k"]
        dequant_s = (t1 - t0) * m / self.ra + (t2 - t1) * n / self.rb
        matmul_s = (t3 - t2) * (m * n) / (self.ra * self.rb)
        return {"dequant_s": dequant_s, "matmul_s": matmul_s, "sample_s": t3 - t0,
                "matmul_sample_tflops": 2.0 * self.ra * self.rb * k / (t3 - t2) / 1e12,
                "tflops": 2.0 * m * n * k / (dequant_s + matmul_s) / 1e12}

    def describe(self, reps: int) -> str:
        return (f"{reps} x [rows 0..{self.ra - 1} of A, rows 0..{self.rb - 1} of B, K={self.w['k']} of "
                f"the {self.name} operands (same seeds as the GPU arm)]: torch dequantize-to-FP32 of "
                f"each, then FP32 torch.matmul, on {self.cores} threads, timed separately; whole "
                "configuration = t_deqA*M/ra + t_deqB*N/rb + t_mm*M*N/(ra*rb)")


def cpu_baseline(w: dict, name: str, limit_s: float = 12.0, max_reps: int = 8) -> dict:
    ref = CpuReference(w, name)
    ref.step()  # warm-up (thread pool, page faults)
    runs, spent = [], 0.0
    while len(runs) < max_reps and (spent < limit_s or not runs):
        r = ref.step()
        runs.append(r)
        spent += r["sample_s"]
    return {"value": float(np.mean([r["tflops"] for r in runs])), "unit": "TFLOP/s",
            "cores": ref.cores, "kind": "port",
            "dequant_s": float(np.mean([r["dequant_s"] for r in runs])),
            "matmul_s": float(np.mean([r["matmul_s"] for r in runs])),
            "matmul_sample_tflops": float(np.mean([r["matmul_sample_tflops"] for r in runs])),
            "sample": ref.describe(len(runs))}


def config_dict(name: str, w: dict, world: int, steps: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    group = replicas_for(w, steps)
    return {"workload": name, "m": w["m"], "n": w["n"], "k": w["k"],
            "sharding": {"n": "column-parallel N/gpus, no communication",
                         "k": "row-parallel K/gpus + BF16 all-reduce (own peer-memory kernel; NCCL timed beside it)",
                         None: "single GPU"}[w["shard"]],
            "step": ("activation quantize_rows + " if w["quant"] else "") + "GEMM"
                    + (" (one fused kernel)" if w.get("fused") else "")
                    + (" + all-reduce" if w["shard"] == "k" and world > 1 else ""),
            "l2": ("256 MiB fill between timed steps" if group == 1 else
                   f"{group} rotating weight copies per graph replay (larger than "
                   "L2 together) + 256 MiB fill between replays")}


DTYPE_TEXT = {"nvfp4": "fp4_e2m1 x ue4m3 -> f32", "mxfp8": "fp8_e4m3 x ue8m0 -> f32",
              "block_fp8": "fp8_e4m3 x f32 scales -> f32"}


# --------------------------------------------------------------------------------------
# Main
# --------------------------------------------------------------------------------------
def run_reference_arm(args, w: dict, name: str, rank: int, world: int) -> None:
    """`--impl reference`: the CPU path alone, on rank 0's host cores."""
    if rank != 0:
        return
    ref = CpuReference(w, name)
    for _ in range(max(args.warmup, 1)):
        ref.step()
    runs = [ref.step() for _ in range(max(args.steps, 1))]
    value = float(np.mean([r["tflops"] for r in runs]))
    dequant_s = float(np.mean([r["dequant_s"] for r in runs]))
    matmul_s = float(np.mean([r["matmul_s"] for r in runs]))
    print(json.dumps({
        "impl": "reference", "metric": "block-scaled GEMM TFLOPS", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": (dequant_s + matmul_s) * 1e3, "higher_is_better": True,
        "scaling": "strong" if w["shard"] else "weak", "vs_baseline": None,
        "dtype": DTYPE_TEXT[w["kind"]], "data": "synthetic",
        "config": config_dict(name, w, world, args.steps),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": ref.cores, "kind": "port",
                         "dequant_s": dequant_s, "matmul_s": matmul_s,
                         "matmul_sample_tflops": float(np.mean([r["matmul_sample_tflops"] for r in runs])),
                         "sample": ref.describe(len(runs))},
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
        chunks = E2E_ROW_CHUNKS if step.w["m"] % (E2E_ROW_CHUNKS * 128) == 0 else 1
        if chunks > 1:
            # The caller's rows in `chunks` pieces, each copied in, multiplied and copied out on
            # its own: the copies of one piece run (on their own streams) under the GEMM and the
            # copies of its neighbours, as a host that feeds the GEMM from pinned memory would
            # arrange it. Same public call (`blockscaled.mm`) per piece, same bytes per step.
            step.e2e_chunks = chunks
            return _e2e_block_fp8_pipelined(step, ha, hs, out_host, chunks, args, flush,
                                            sync_ranks, reduce_max)

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


def _e2e_block_fp8_pipelined(step: Step, ha, hs, out_host, chunks: int, args, flush, sync_ranks,
                             reduce_max) -> float:
    from sparkinfer_b200.gemm import blockscaled

    m, k = step.w["m"], step.w["k"]
    nl = step.out.shape[1]
    rows = m // chunks
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    kw = dict(ab_dtype="float8_e4m3fn", sf_dtype="float32", sf_vec_size=128, c_dtype="bfloat16",
              block_fp8=True)
    b = (step.b.view(nl, k, 1), step.sb)
    pieces = []
    for i in range(chunks):
        r = slice(i * rows, (i + 1) * rows)
        pieces.append((step.a[r], ha[r], step.sa[r], hs[r], step.out[r], out_host[r],
                       torch.cuda.Event(), torch.cuda.Event()))

    def fn():
        s_in.wait_stream(cur)    # not before the step begins (and the previous step's GEMMs are done)
        s_out.wait_stream(cur)
        for a_dev, a_host, sa_dev, sa_host, out_dev, out_h, copied, computed in pieces:
            with torch.cuda.stream(s_in):
                a_dev.copy_(a_host, non_blocking=True)
                sa_dev.copy_(sa_host, non_blocking=True)
                copied.record(s_in)
            cur.wait_event(copied)
            blockscaled.mm((a_dev.view(rows, k, 1), sa_dev), b, out_dev, **kw)
            computed.record(cur)
            s_out.wait_event(computed)
            with torch.cuda.stream(s_out):
                out_h.copy_(out_dev, non_blocking=True)
        cur.wait_stream(s_out)   # the step ends when the last piece of the result is on the host

    times = time_steps(fn, max(3, min(args.steps, 10)), 3, flush, sync_ranks, use_graph=False)
    return reduce_max(float(np.mean(times)))


def time_components(step: Step, flush, sync_ranks, reduce_max) -> dict:
    """Device time of each part of a step, each timed alone (graph replays, L2 flushed)."""
    out = {}
    reps = max(1, 20 // step.group)
    out["gemm_ms"] = reduce_max(float(np.mean(time_steps(step.gemm, reps, 3, flush, sync_ranks)))) / step.group
    if step.quant is not None:
        out["quant_ms"] = reduce_max(float(np.mean(time_steps(step.quant, 20, 3, flush, sync_ranks))))
    if step.w["shard"] == "k" and step.world > 1:
        import torch.distributed as dist

        out["collective"] = step.collective
        out["allreduce_ms"] = reduce_max(float(np.mean(
            time_steps(step.all_reduce, 20, 3, flush, sync_ranks, use_graph=False))))
        if step.reducer is not None:  # the library collective on the same bytes, for comparison
            scratch = torch.empty_like(step.out)
            out["nccl_allreduce_ms"] = reduce_max(float(np.mean(
                time_steps(lambda: dist.all_reduce(scratch), 20, 3, flush, sync_ranks, use_graph=False))))
            del scratch
    return out


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
        run_reference_arm(args, w, args.workload, rank, world)
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

    def parity_over_ranks(step: Step) -> dict:
        sync_ranks()  # ranks leave the set-up of a step at different times
        step.run()
        torch.cuda.synchronize()
        par = step.parity()
        par["max_err"] = reduce_max(par["max_err"])
        par["ok"] = bool(par["max_err"] <= par["tolerance"])
        return par

    peaks = measured_peaks()
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    step = Step(args.workload, w, rank, world, device, replicas=replicas_for(w, args.steps))
    step.run()
    sync_ranks()
    parity = parity_over_ranks(step)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_per_step, gemm_ms, _ = measure(step, args, flush, sync_ranks, reduce_max)
    clocks = sampler.stop() if sampler else None
    e2e_ms = measure_e2e(step, args, flush, sync_ranks, reduce_max)
    e2e_pieces = getattr(step, "e2e_chunks", 1)
    h2d_d2h = (step.h2d_bytes, step.d2h_bytes)

    from sparkinfer_b200._lib.launch import check_kernel_status

    def kernel_status_over_ranks() -> str | None:
        """Highest kernel status word over the ranks (None when every bounded wait was met);
        every rank gets the same answer, so nobody leaves the others inside a collective."""
        try:
            check_kernel_status(device)
            code, text = 0.0, ""
        except RuntimeError as exc:
            code, text = 1.0, str(exc)
        if reduce_max(code) == 0.0:
            return None
        return text or "a kernel on another rank reported a timed-out wait"

    headline_status = kernel_status_over_ranks()

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

    # Every other configuration, timed the same way. On several GPUs only the configurations
    # that shard are run (column-parallel and row-parallel), so that a scaling run records both.
    extra = {}
    if not args.no_extra:
        del step
        torch.cuda.empty_cache()
        for name, other in table.items():
            if name == args.workload or (world > 1 and not other["shard"]):
                continue
            try:
                s = Step(name, other, rank, world, device, replicas=replicas_for(other, 24))
                par = parity_over_ranks(s)
                reps = max(1, 24 // s.group)
                t_all = reduce_max(float(np.mean(time_steps(s.run, reps, 3, flush, sync_ranks)))) / s.group
                parts = time_components(s, flush, sync_ranks, reduce_max)
                n_loc, k_loc = s.n_local, s.k_local
                extra[name] = {
                    "ms_per_step": t_all, **parts,
                    "tflops": 2.0 * other["m"] * other["n"] * other["k"] / t_all / 1e9,
                    "gemm_tflops_per_gpu": 2.0 * other["m"] * n_loc * k_loc / parts["gemm_ms"] / 1e9,
                    "gbs": algorithmic_bytes(other, n_loc, k_loc) / parts["gemm_ms"] / 1e6,
                    "parity_max_err": par["max_err"], "parity_tolerance": par["tolerance"],
                    "parity_ok": par["ok"],
                }
                del s
                torch.cuda.empty_cache()
            except Exception as exc:  # keep the headline line even if a side config fails
                extra[name] = {"error": str(exc)[:160]}
            status = kernel_status_over_ranks()
            if status is not None:
                extra.setdefault(name, {})["kernel_status"] = status

    if rank == 0:
        baseline = cpu_baseline(w, args.workload) if world == 1 else None
        flops = 2.0 * w["m"] * w["n"] * w["k"]
        value = flops / ms_per_step / 1e9
        group = replicas_for(w, args.steps)
        kernels_per_step = 2 if (w["quant"] and not w.get("fused")) else 1
        line = {
            "metric": "block-scaled GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": max(1, args.steps // group) * group,
            "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if w["shard"] else "weak", "vs_baseline": None,
            "dtype": DTYPE_TEXT[w["kind"]],
            "data": "synthetic",
            "config": config_dict(args.workload, w, world, args.steps),
            "roofline": roofline,
            "parity": parity,
            "kernel_status": headline_status or "ok",
            "e2e": {"value": flops / e2e_ms / 1e9, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d_d2h[0], "d2h_bytes_per_step": h2d_d2h[1],
                    "ms_per_step": e2e_ms, "row_pieces": e2e_pieces},
            "gpu_launches": max(1, args.steps // group) * group * kernels_per_step,
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
