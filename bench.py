#!/usr/bin/env python
"""Benchmark of the gern_b200 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of a fused kernel over one batch of seeded synthetic input.  The default
workload is the fused two-stage blur on an 8192 x 8192 fp32 image per GPU (row bands of a taller
image at N > 1, the 2-row halo read from the neighbour inside the timed region).  Other workloads:
softmax (65536 x 4096 fp32), gemm_bf16 (8192^3), attention (32768 x 4096 x 128), gemm_f32 (512^3).
Rank 0 prints one JSON line.  `--impl reference` times the reference's CPU path instead (the
compiled reference code under oracle/_ref when present, else the CPU restatement under oracle/).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


def load_traffic(kernel: str):
    """DRAM bytes per launch from the committed ncu summary (profiles/traffic.json), or None."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                return json.load(f).get(kernel)
        except Exception:
            return None
    return None


def mt19937_uniform(n, lo, hi):
    """std::mt19937(0) + std::uniform_real_distribution<float>(lo, hi): the stream the reference's
    MatrixCPU::random_fill produces (test/library/matrix/impl/cpu-matrix.h:71-81)."""
    bg = np.random.MT19937()
    bg._legacy_seeding(0)
    u = bg.random_raw(n).astype(np.uint32).astype(np.float32) * np.float32(2.0 ** -32)
    u = np.minimum(u, np.nextafter(np.float32(1.0), np.float32(0.0)))
    return (u * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------
class Workload:
    """One benchmarked fused kernel: device-resident run, host-buffer run, CPU sample."""
    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "hbm"
    kernel = ""

    def __init__(self, ctx, rank, world, torch):
        self.ctx, self.rank, self.world, self.torch = ctx, rank, world, torch

    def units_per_step(self) -> float:          # bytes or flops this rank processes per step
        raise NotImplementedError

    def launches_per_step(self) -> int:
        return 1

    def step(self, stream):
        raise NotImplementedError

    def e2e_setup(self):
        raise NotImplementedError

    def e2e_step(self):
        raise NotImplementedError

    def config(self) -> dict:
        raise NotImplementedError


class BlurWorkload(Workload):
    """8192 x 8192 input image per GPU; as in the reference's app (apps/blur/blur.cpp:28-44) the
    output is 8188 x 8188: the last two rows and columns of the stored image are padding."""
    name = "blur"
    metric = "fused two-stage blur, algorithmic HBM bytes per second"
    unit = "GB/s"
    dtype = "f32"
    kernel = "blur3x3_reg_kernel"
    N = 8192
    VARIANT = None      # --variant: a kernel variant of the library's test hook (N = 1 only)

    def __init__(self, ctx, rank, world, torch, dist=None):
        super().__init__(ctx, rank, world, torch)
        from gern_b200 import sharding
        self.sharding = sharding
        n = self.N
        # The job's image has world * 8192 stored rows (8192 per GPU: weak scaling); its last two
        # rows and columns are padding, so the valid image is (world * 8192 - 2) x 8190.
        self.band = sharding.blur_band(world * n - 2, world, rank)
        rows = self.band.band_rows
        self.oc = n - 4                                   # output columns
        self.out = torch.empty((self.band.out_rows, self.oc), device="cuda")
        self.dist = dist
        self.halo = None
        self.mode = "none"
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        if world > 1:
            # Preferred: the band lives in symmetric memory, and the kernel reads the two halo
            # rows straight out of the next rank's band over NVLink (plain loads, no collective
            # and no extra launch).  Fallback: NCCL send/recv into a local halo buffer each step.
            try:
                import torch.distributed._symmetric_memory as symm
                buf = symm.empty((n, n), dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
                hdl = symm.rendezvous(buf, dist.group.WORLD)
                self.x = buf[:rows]
                self.x.copy_(torch.rand((rows, n), generator=g, device="cuda"))
                if self.band.recvs_halo:
                    peer = hdl.get_buffer(rank + 1, (n, n), torch.float32)
                    self.halo = peer[0:2]
                self._symm = (buf, hdl)
                self.mode = "peer loads over NVLink (symmetric memory)"
            except Exception as e:  # noqa: BLE001
                self.mode = f"NCCL send/recv ({type(e).__name__})"
                self.x = torch.rand((rows, n), generator=g, device="cuda")
                self.halo = torch.empty((2, n), device="cuda") if self.band.recvs_halo else None
                self.side = torch.cuda.Stream()
        else:
            self.x = torch.rand((rows, n), generator=g, device="cuda")

    def units_per_step(self):
        n = self.N
        read = (self.band.band_rows + self.band.halo_rows) * n * 4
        write = self.band.out_rows * self.oc * 4
        if self.world == 1:
            read = n * n * 4      # the stored image, padding included
        return float(read + write)

    def step(self, stream):
        torch = self.torch
        n = self.N
        band = self.band
        if self.world == 1:
            self.ctx.blur3x3(self.x[:, : n - 2], self.out, stream=stream, variant=self.VARIANT)
            return
        if self.mode.startswith("NCCL"):
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                for w in self.sharding.exchange_blur_halo(self.dist, band, self.x[0:2], self.halo):
                    w.wait()
            torch.cuda.current_stream().wait_stream(self.side)
        # One launch: the last block row of the band reads the two halo rows through `halo`.
        halo = self.halo[:, : n - 2] if band.recvs_halo else None
        self.ctx.blur3x3_band(self.x[:, : n - 2], halo, self.out, stream=stream)

    def e2e_setup(self):
        torch = self.torch
        n = self.N
        self.h_in = torch.rand((n, n), dtype=torch.float32).pin_memory()
        self.h_out = torch.empty((n - 4, n - 4), dtype=torch.float32).pin_memory()
        return (n - 2) * (n - 2) * 4, (n - 4) * (n - 4) * 4

    def e2e_units(self):
        n = self.N
        return float(n * n * 4 + (n - 4) * (n - 4) * 4)

    def e2e_step(self):
        n = self.N
        self.ctx.blur3x3_host(self.h_in[: n - 2, : n - 2], self.h_out)

    def config(self):
        n = self.N
        return {"workload": f"fused 2-stage 3-tap blur, {n}x{n} fp32 image per GPU -> {n - 4}x{n - 4}",
                "rows_per_gpu": n, "cols": n,
                "sharding": f"row bands, 2-row halo by {self.mode}" if self.world > 1 else "none",
                "cache": "inputs larger than L2 (268 MB read + 268 MB written per step)"}

    def cpu_sample(self, oracle, ref):
        rows = 1024
        x = np.random.default_rng(0).random((rows + 2, self.N - 2), dtype=np.float32)
        fn = ref.blur_xy if ref is not None else oracle.blur_xy
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0 or reps < 2:
            fn(x)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        units = (rows + 2) * self.N * 4 + rows * (self.N - 4) * 4
        return units / dt / 1e9, f"{rows + 2} x {self.N} band ({reps} passes)"


class SoftmaxWorkload(Workload):
    name = "softmax"
    metric = "row softmax, algorithmic HBM bytes per second"
    unit = "GB/s"
    dtype = "f32"
    kernel = "softmax_cta_kernel"
    ROWS, COLS = 65536, 4096

    def __init__(self, ctx, rank, world, torch, dist=None):
        super().__init__(ctx, rank, world, torch)
        g = torch.Generator(device="cuda").manual_seed(99 + rank)
        self.x = torch.randn((self.ROWS, self.COLS), generator=g, device="cuda") * 3
        self.out = torch.empty_like(self.x)

    def units_per_step(self):
        return float(2 * self.ROWS * self.COLS * 4)

    def step(self, stream):
        self.ctx.softmax_rows(self.x, self.out, stream=stream)

    def e2e_setup(self):
        torch = self.torch
        self.h_in = (torch.randn((self.ROWS, self.COLS)) * 3).pin_memory()
        self.h_out = torch.empty((self.ROWS, self.COLS)).pin_memory()
        b = self.ROWS * self.COLS * 4
        return b, b

    def e2e_units(self):
        return self.units_per_step()

    def e2e_step(self):
        self.ctx.softmax_rows_host(self.h_in, self.h_out)

    def config(self):
        return {"workload": f"row softmax fp32 {self.ROWS}x{self.COLS} per GPU", "sharding": "rows",
                "cache": "inputs larger than L2 (1 GiB read + 1 GiB written per step)"}

    def cpu_sample(self, oracle, ref):
        rows = 2048
        x = (np.random.default_rng(0).standard_normal((rows, self.COLS)) * 3).astype(np.float32)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0 or reps < 2:
            oracle.softmax_rows(x)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return 2 * rows * self.COLS * 4 / dt / 1e9, f"{rows} x {self.COLS} rows ({reps} passes)"


class GemmBf16Workload(Workload):
    name = "gemm_bf16"
    metric = "bf16 GEMM (fp32 accumulate), dense FLOP per second"
    unit = "TFLOP/s"
    dtype = "bf16"
    bound = "tensor"
    kernel = "gemm_bf16_2cta_kernel"
    N = 8192
    SHAPE = None        # (M, N, K) from --shape: a kernel-only side measurement, not the headline
    VS_CUBLAS = False   # --vs-cublas: time torch.matmul (cuBLAS) on the same operands beside it

    def __init__(self, ctx, rank, world, torch, dist=None):
        super().__init__(ctx, rank, world, torch)
        m, n, k = self.SHAPE if self.SHAPE else (self.N, self.N, self.N)
        self.mnk = (m, n, k)
        g = torch.Generator(device="cuda").manual_seed(7 + rank)
        self.a = (torch.randn((m, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

    def units_per_step(self):
        m, n, k = self.mnk
        return 2.0 * m * n * k

    def step(self, stream):
        self.ctx.gemm_bf16(self.a, self.b, self.c, stream=stream)

    def library_baseline(self, steps, warmup):
        """cuBLAS through torch.matmul on the same operands, timed like the kernel above."""
        torch = self.torch
        bt = self.b.T
        for _ in range(warmup):
            torch.matmul(self.a, bt, out=self.c)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            torch.matmul(self.a, bt, out=self.c)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"library": "cuBLAS via torch.matmul", "ms_per_step": ms,
                "value": self.units_per_step() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}

    def e2e_setup(self):
        torch = self.torch
        n = self.N
        self.h_a = (torch.randn((n, n)) * 0.02).to(torch.bfloat16).pin_memory()
        self.h_b = (torch.randn((n, n)) * 0.02).to(torch.bfloat16).pin_memory()
        self.h_c = torch.empty((n, n), dtype=torch.bfloat16).pin_memory()
        return 2 * n * n * 2, n * n * 2

    def e2e_units(self):
        return self.units_per_step()

    def e2e_step(self):
        self.ctx.gemm_bf16_host(self.h_a, self.h_b, self.h_c)

    def config(self):
        n = self.N
        if self.SHAPE:
            m, n2, k = self.SHAPE
            return {"workload": f"bf16 GEMM M={m} N={n2} K={k} per GPU (A row-major, B column-major, fp32 accumulate)",
                    "sharding": "M panels, B replicated", "cache": "operands as they are (may fit L2)"}
        return {"workload": f"bf16 GEMM M=N=K={n} per GPU (A row-major, B column-major, fp32 accumulate)",
                "sharding": "M panels, B replicated", "cache": "flush not needed: 384 MB of operands > L2"}

    def cpu_sample(self, oracle, ref):
        from oracle import pyoracle
        rows = 8
        rng = np.random.default_rng(0)
        a = pyoracle.to_bf16_bits((rng.standard_normal((rows, self.N)) * 0.02).astype(np.float32))
        b = pyoracle.to_bf16_bits((rng.standard_normal((self.N, self.N)) * 0.02).astype(np.float32))
        t0 = time.perf_counter()
        oracle.gemm_bf16(a, b)
        dt = time.perf_counter() - t0
        return 2.0 * rows * self.N * self.N / dt / 1e12, f"{rows} rows of C (M-panel of {rows} x {self.N} x {self.N})"


class AttentionWorkload(Workload):
    name = "attention"
    metric = "GEMM->softmax->GEMM chain, dense FLOP per second"
    unit = "TFLOP/s"
    dtype = "bf16"
    bound = "tensor"
    kernel = "attention_bf16_kernel"
    NQ, NKV, D = 32768, 4096, 128

    def __init__(self, ctx, rank, world, torch, dist=None):
        super().__init__(ctx, rank, world, torch)
        g = torch.Generator(device="cuda").manual_seed(17 + rank)
        self.q = torch.randn((self.NQ, self.D), generator=g, device="cuda").to(torch.bfloat16)
        self.k = torch.randn((self.NKV, self.D), generator=g, device="cuda").to(torch.bfloat16)
        self.v = torch.randn((self.NKV, self.D), generator=g, device="cuda").to(torch.bfloat16)
        self.o = torch.empty((self.NQ, self.D), dtype=torch.bfloat16, device="cuda")
        self.scale = 1.0 / math.sqrt(self.D)

    def units_per_step(self):
        return 4.0 * self.NQ * self.NKV * self.D

    def step(self, stream):
        self.ctx.attention_bf16(self.q, self.k, self.v, self.o, self.scale, stream=stream)

    def e2e_setup(self):
        torch = self.torch
        self.h_q = torch.randn((self.NQ, self.D)).to(torch.bfloat16).pin_memory()
        self.h_k = torch.randn((self.NKV, self.D)).to(torch.bfloat16).pin_memory()
        self.h_v = torch.randn((self.NKV, self.D)).to(torch.bfloat16).pin_memory()
        self.h_o = torch.empty((self.NQ, self.D), dtype=torch.bfloat16).pin_memory()
        return (self.NQ + 2 * self.NKV) * self.D * 2, self.NQ * self.D * 2

    def e2e_units(self):
        return self.units_per_step()

    def e2e_step(self):
        self.ctx.attention_bf16_host(self.h_q, self.h_k, self.h_v, self.h_o, self.scale)

    def config(self):
        return {"workload": f"softmax(Q K^T / sqrt(128)) V, Q {self.NQ}x128, K,V {self.NKV}x128 bf16 per GPU",
                "sharding": "Q rows, K and V replicated",
                "cache": "L2-resident operands by design (K, V = 2 MiB are re-read by every CTA)"}

    def cpu_sample(self, oracle, ref):
        from oracle import pyoracle
        rows = 64
        rng = np.random.default_rng(0)
        q = pyoracle.to_bf16_bits(rng.standard_normal((rows, self.D)).astype(np.float32))
        k = pyoracle.to_bf16_bits(rng.standard_normal((self.NKV, self.D)).astype(np.float32))
        v = pyoracle.to_bf16_bits(rng.standard_normal((self.NKV, self.D)).astype(np.float32))
        t0 = time.perf_counter()
        oracle.attention_bf16(q, k, v, self.scale)
        dt = time.perf_counter() - t0
        return 4.0 * rows * self.NKV * self.D / dt / 1e12, f"{rows} rows of Q against all {self.NKV} keys"


class GemmF32ShapeWorkload(Workload):
    """fp32 matmul at a shape given with --shape: a kernel-only side measurement (the headline fp32
    configuration is 512^3, GemmF32Workload).  Large shapes run on the tensor cores through
    three-way bf16 splits; --vs-cublas adds torch.matmul with tf32 switched off."""
    name = "gemm_f32_shape"
    metric = "fp32 matmul, FLOP per second"
    unit = "TFLOP/s"
    dtype = "f32"
    bound = "tensor"
    kernel = "gemm_bf16_tc_kernel"
    SHAPE = (4096, 4096, 4096)
    VS_CUBLAS = False

    def __init__(self, ctx, rank, world, torch, dist=None):
        super().__init__(ctx, rank, world, torch)
        m, n, k = self.SHAPE
        g = torch.Generator(device="cuda").manual_seed(11 + rank)
        self.a = torch.rand((m, k), generator=g, device="cuda") * 2 - 1
        self.b = torch.rand((k, n), generator=g, device="cuda") * 2 - 1
        self.c = torch.zeros((m, n), device="cuda")

    def units_per_step(self):
        m, n, k = self.SHAPE
        return 2.0 * m * n * k

    def step(self, stream):
        self.ctx.gemm_f32(self.a, self.b, self.c, stream=stream)

    def library_baseline(self, steps, warmup):
        torch = self.torch
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            for _ in range(warmup):
                torch.matmul(self.a, self.b, out=self.c)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                torch.matmul(self.a, self.b, out=self.c)
            e1.record()
            torch.cuda.synchronize()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = old
        ms = e0.elapsed_time(e1) / steps
        return {"library": "cuBLAS fp32 (tf32 off) via torch.matmul", "ms_per_step": ms,
                "value": self.units_per_step() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}

    def e2e_setup(self):
        return 0, 0

    def config(self):
        m, n, k = self.SHAPE
        return {"workload": f"fp32 matmul M={m} N={n} K={k} per GPU, uniform[-1,1) (replicas only)",
                "sharding": "replicas only", "cache": "operands as they are (may fit L2)"}

    def cpu_sample(self, oracle, ref):
        return 0.0, "none"


class GemmF32Workload(Workload):
    name = "gemm_f32"
    metric = "fp32 matmul 512^3, FLOP per second"
    unit = "TFLOP/s"
    dtype = "f32"
    bound = "tensor"
    kernel = "gemm_f32_warpk_kernel"
    N = 512

    def __init__(self, ctx, rank, world, torch, dist=None):
        super().__init__(ctx, rank, world, torch)
        a = mt19937_uniform(self.N * self.N, -1.0, 1.0).reshape(self.N, self.N)
        self.a = torch.from_numpy(a).cuda()
        self.c = torch.zeros((self.N, self.N), device="cuda")
        self.flush = torch.empty(64 * 1024 * 1024, device="cuda")  # 256 MB > L2

    def units_per_step(self):
        return 2.0 * self.N ** 3

    def pre_step(self):
        self.flush.zero_()      # evict the 3 MB of operands from L2; outside the per-step events

    def step(self, stream):
        self.ctx.gemm_f32(self.a, self.a, self.c, stream=stream)

    def e2e_setup(self):
        torch = self.torch
        self.h_a = self.a.cpu().pin_memory()
        self.h_c = torch.zeros((self.N, self.N)).pin_memory()
        return 2 * self.N * self.N * 4, self.N * self.N * 4

    def e2e_units(self):
        return self.units_per_step()

    def e2e_step(self):
        self.ctx.gemm_f32_host(self.h_a, self.h_a, self.h_c)

    def config(self):
        return {"workload": "fp32 matmul M=N=K=512, A=B=uniform[-1,1) mt19937(0) (replicas only)",
                "sharding": "replicas only", "cache": "L2 flushed between steps (256 MB memset)"}

    def cpu_sample(self, oracle, ref):
        a = self.a.cpu().numpy()
        fn = (lambda: ref.matmul_tiled(a, a, 64, 64, 64)) if ref is not None else (
            lambda: oracle.matmul_tiled(a, a, 64, 64, 64))
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 5.0 or reps < 2:
            fn()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return 2.0 * self.N ** 3 / dt / 1e12, f"whole 512^3 problem, tiles 64/64/64 ({reps} passes)"


WORKLOADS = {w.name: w for w in (BlurWorkload, SoftmaxWorkload, GemmBf16Workload, AttentionWorkload,
                                 GemmF32Workload, GemmF32ShapeWorkload)}


def scale_of(unit):
    return 1e9 if unit == "GB/s" else 1e12


# ----------------------------------------------------------------------------------------------
def run_reference_arm(args, rank, world):
    """Times the reference's CPU path on this box's host cores (rank 0 only)."""
    if rank != 0:
        return
    from oracle import pyoracle
    oracle = pyoracle.Oracle()
    ref = pyoracle.Reference() if pyoracle.Reference.available() else None
    cls = WORKLOADS[args.workload]
    cores = oracle.max_threads()
    oracle.set_threads(cores)
    n = cls.N if hasattr(cls, "N") else None
    times = []
    units = 0.0
    sample = ""
    kind = "port"
    total = args.warmup + args.steps
    if args.workload == "blur":
        rows = 512
        x = np.random.default_rng(0).random((rows + 2, n), dtype=np.float32)
        units = (rows + 2) * n * 4 + rows * (n - 2) * 4
        sample = f"{rows + 2} x {n} row band of the {n} x {n} image per step"
        # The compiled reference (cpu_blur_x / cpu_blur_y, single-threaded as written) when it was
        # built, else the restatement fanned out over all host cores.
        if ref is not None:
            kind, cores, fn = "reference", 1, (lambda: ref.blur_xy(x))
        else:
            fn = lambda: oracle.blur_xy(x)
    elif args.workload == "softmax":
        rows = 1024
        x = (np.random.default_rng(0).standard_normal((rows, cls.COLS)) * 3).astype(np.float32)
        units = 2 * rows * cls.COLS * 4
        sample = f"{rows} x {cls.COLS} rows per step"
        fn = lambda: oracle.softmax_rows(x)
    elif args.workload == "gemm_f32":
        a = pyoracle.mt19937_uniform(n * n, -1.0, 1.0).reshape(n, n)
        units = 2.0 * n ** 3
        sample = "whole 512^3 problem per step (tiles 64/64/64)"
        if ref is not None:
            kind, cores, fn = "reference", 1, (lambda: ref.matmul_tiled(a, a, 64, 64, 64))
        else:
            fn = lambda: oracle.matmul_tiled(a, a, 64, 64, 64)
    elif args.workload == "gemm_bf16":
        rows = 2 * cores
        rng = np.random.default_rng(0)
        a = pyoracle.to_bf16_bits((rng.standard_normal((rows, n)) * 0.02).astype(np.float32))
        b = pyoracle.to_bf16_bits((rng.standard_normal((n, n)) * 0.02).astype(np.float32))
        units = 2.0 * rows * n * n
        sample = f"{rows}-row M panel of the {n}^3 problem per step"
        fn = lambda: oracle.gemm_bf16(a, b)
    else:
        rows = 16 * cores
        rng = np.random.default_rng(0)
        q = pyoracle.to_bf16_bits(rng.standard_normal((rows, 128)).astype(np.float32))
        k = pyoracle.to_bf16_bits(rng.standard_normal((cls.NKV, 128)).astype(np.float32))
        v = pyoracle.to_bf16_bits(rng.standard_normal((cls.NKV, 128)).astype(np.float32))
        units = 4.0 * rows * cls.NKV * 128
        sample = f"{rows} rows of Q against {cls.NKV} keys per step"
        fn = lambda: oracle.attention_bf16(q, k, v, 1.0 / math.sqrt(128.0))
    for i in range(total):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            times.append(dt)
    per = sum(times) / len(times)
    value = units / per / scale_of(cls.unit)
    # the configuration this arm stands beside: the library arm's, word for word
    shell = cls.__new__(cls)
    shell.world = world
    shell.mode = "peer loads over NVLink (symmetric memory)"
    cfg = cls.config(shell)
    line = {"impl": "reference", "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": cls.dtype, "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": cls.unit, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="blur", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="gern_b200", choices=["gern_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--small", action="store_true",
                    help="reduced sizes (still larger than L2) for profiler captures; not a bench number")
    ap.add_argument("--variant", type=int, default=None,
                    help="blur only, one GPU: kernel variant of gb200_blur3x3_f32_variant (52 = TMA-staged, short strips)")
    ap.add_argument("--shape", default="", help="gemm_bf16 / gemm_f32: M,N,K of a side measurement (kernel only)")
    ap.add_argument("--vs-cublas", action="store_true",
                    help="with --shape: add cuBLAS (torch.matmul) timed the same way under 'library'")
    ap.add_argument("--also", default="softmax,attention,gemm_bf16",
                    help="comma list of further workloads summarised under 'also' (N=1 only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the gern_b200 kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from gern_b200 import api
    ctx = api.Context(local_rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if args.variant is not None:
        BlurWorkload.VARIANT = args.variant
        if 2 <= args.variant < 40 or args.variant >= 50:
            BlurWorkload.kernel = "blur3x3_tma_kernel"
    if args.shape:
        GemmBf16Workload.SHAPE = tuple(int(v) for v in args.shape.split(","))
        GemmF32ShapeWorkload.SHAPE = GemmBf16Workload.SHAPE
        args.no_e2e = args.no_cpu_baseline = True
        if args.workload == "gemm_f32":
            args.workload = "gemm_f32_shape"
    GemmBf16Workload.VS_CUBLAS = args.vs_cublas
    GemmF32ShapeWorkload.VS_CUBLAS = args.vs_cublas
    if args.small:
        SoftmaxWorkload.ROWS = 16384
        GemmBf16Workload.N = 4096
        AttentionWorkload.NQ = 8192

    def run_workload(name, steps, warmup, want_e2e, want_cpu):
        wl = WORKLOADS[name](ctx, rank, world, torch, dist)
        stream = torch.cuda.current_stream()
        for _ in range(warmup):
            wl.step(stream)
        barrier()
        launches0 = ctx.launch_count()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        pre = getattr(wl, "pre_step", None)
        evs = []
        barrier()
        start.record()
        if pre is None:
            # One kernel launch per step and nothing else on the stream: the K launches run back to
            # back between one pair of events, so the average launch duration is region / K (an
            # event pair around every launch would cost each kernel its overlap with the launch
            # set-up of the next: 76 instead of 68 us for the 70-us attention kernel).
            for i in range(steps):
                wl.step(stream)
        else:
            # a workload that flushes L2 between steps is timed by per-step events only
            for i in range(steps):
                pre()
                evs.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
                evs[i][0].record()
                wl.step(stream)
                evs[i][1].record()
        stop.record()
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        ctx.sync()  # also surfaces a kernel that gave up a bounded wait
        launches = ctx.launch_count() - launches0
        if pre is None:
            total_ms = start.elapsed_time(stop)
            per_launch_ms = total_ms / steps
        else:
            per_launch_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
            total_ms = per_launch_ms * steps
        t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        units = torch.tensor([wl.units_per_step()], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(units, op=dist.ReduceOp.SUM)
        all_units = float(units.item())
        sc = scale_of(wl.unit)
        value = all_units * steps / (total_ms * 1e-3) / sc
        peaks = load_peaks()
        if wl.bound == "hbm":
            peak, punit = peaks["hbm_gbs"], "GB/s"
        else:
            peak, punit = peaks["bf16_tflops"], "TFLOP/s"
        achieved = wl.units_per_step() / (per_launch_ms * 1e-3) / sc
        res = {"metric": wl.metric, "value": value, "unit": wl.unit, "ms_per_step": total_ms / steps,
               "dtype": wl.dtype, "config": wl.config(),
               "roofline": {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": punit,
                            "frac": achieved / peak, "traffic": load_traffic(wl.kernel),
                            "peak_source": peaks["source"], "kernel": wl.kernel,
                            "kernel_ms": per_launch_ms},
               "gpu_launches": launches, "clocks": clocks}
        if getattr(wl, "VS_CUBLAS", False) and world == 1:
            res["library"] = wl.library_baseline(steps, warmup)
        if want_e2e:
            h2d, d2h = wl.e2e_setup()
            e_steps = max(2, min(steps, 5))
            wl.e2e_step()
            barrier()
            t0 = time.perf_counter()
            for _ in range(e_steps):
                wl.e2e_step()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            tt = torch.tensor([dt], dtype=torch.float64, device="cuda")
            if dist is not None:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e_val = wl.e2e_units() * world * e_steps / float(tt.item()) / sc
            res["e2e"] = {"value": e_val, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                          "steps": e_steps, "ms_per_step": float(tt.item()) / e_steps * 1e3}
        if want_cpu and rank == 0 and world == 1:
            from oracle import pyoracle
            oracle = pyoracle.Oracle()
            cores = oracle.max_threads()
            oracle.set_threads(cores)
            v, sample = wl.cpu_sample(oracle, None)
            res["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": cores, "kind": "port", "sample": sample}
        del wl
        torch.cuda.empty_cache()
        return res

    main_res = run_workload(args.workload, args.steps, args.warmup, not args.no_e2e, not args.no_cpu_baseline)
    also = {}
    if world == 1 and args.also:
        for name in [s for s in args.also.split(",") if s in WORKLOADS and s != args.workload]:
            try:
                r = run_workload(name, min(args.steps, 20), 5, False, False)
                also[name] = {"value": r["value"], "unit": r["unit"], "ms_per_step": r["ms_per_step"],
                              "frac_of_peak": r["roofline"]["frac"], "bound": r["roofline"]["bound"]}
            except Exception as e:  # a failing side workload must not hide the headline line
                also[name] = {"error": str(e)[:200]}
    if rank == 0:
        line = {"metric": main_res["metric"], "value": main_res["value"], "unit": main_res["unit"],
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": main_res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": main_res["dtype"], "data": "synthetic",
                "config": dict(main_res["config"], **({"small": True} if args.small else {})),
                "roofline": main_res["roofline"],
                "gpu_launches": main_res["gpu_launches"], "clocks": main_res["clocks"]}
        if "e2e" in main_res:
            line["e2e"] = main_res["e2e"]
        if "cpu_baseline" in main_res:
            line["cpu_baseline"] = main_res["cpu_baseline"]
        if "library" in main_res:
            line["library"] = main_res["library"]
        if also:
            line["also"] = also
        print(json.dumps(line), flush=True)
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
