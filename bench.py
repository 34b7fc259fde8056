#!/usr/bin/env python
"""Benchmark of the gern_b200 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of a fused kernel over one batch of seeded synthetic input.  The headline
workload is the fused two-stage blur on an 8192 x 8192 fp32 image per GPU (at N > 1: row bands of a
taller image, weak scaling, the 2-row halo read from the neighbour inside the timed region).  The
other workloads -- softmax (65536 x 4096 fp32), gemm_bf16 (8192^3), attention (32768 x 4096 x 128),
gemm_f32 (512^3) -- are measured in the same run and reported under `also`:

  * N = 1: each entry is a full record (roofline with traffic, e2e through the host-buffer entry
    point, CPU baseline, clocks, parity against the oracle);
  * N > 1: each sharded workload is measured weak (the whole configuration per GPU) and strong (the
    one configuration cut N ways: softmax rows, GEMM M panels with B replicated, attention Q rows,
    blur row bands of the one 8192 x 8192 image), with the speed-up of the strong form over the
    same problem on rank 0 alone, and every rank compares rows of its own output with the oracle.

Rank 0 prints one JSON line; a parity mismatch makes every rank exit non-zero after the line.
`--impl reference` times the reference's CPU path instead (the compiled reference code under
oracle/_ref when present, else the CPU restatement under oracle/).
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


def bind_to_gpu_numa(index: int) -> str:
    """Pins this process to the CPUs NVML names as local to GPU `index`, so that the pinned host
    buffers of the end-to-end leg are first touched, and therefore placed, on the GPU's own NUMA
    node.  Returns a description for the bench line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        ncpu = os.cpu_count() or 64
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cpus = {w * 64 + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if not cpus:
            return "not bound (NVML names no usable CPU)"
        os.sched_setaffinity(0, cpus)
        return f"bound to the GPU's {len(cpus)} local CPUs ({min(cpus)}-{max(cpus)})"
    except Exception as e:  # noqa: BLE001
        return f"not bound ({type(e).__name__})"


def bits_of(t, torch):
    """bf16 tensor -> numpy uint16 bit patterns."""
    return np.ascontiguousarray(t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16))


def spread_rows(total: int, count: int):
    """`count` row indices spread over [0, total) at offsets that move through any power-of-two tile."""
    count = min(count, total)
    return sorted({(i * total) // count + (i * 37) % max(1, total // count) for i in range(count)})


# ----------------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------------
class Workload:
    """One benchmarked fused kernel: device-resident run, host-buffer run, CPU sample, parity check.
    mode: "single" (one GPU, the whole configuration), "weak" (the whole configuration per GPU) or
    "strong" (the one configuration cut `world` ways by rows)."""
    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "hbm"
    kernel = ""
    sharded = True

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        self.ctx, self.rank, self.world, self.torch, self.dist, self.mode = ctx, rank, world, torch, dist, mode
        self.parts = world if mode == "strong" else 1

    def units_per_step(self) -> float:          # bytes or flops this rank processes per step
        raise NotImplementedError

    def step(self, stream):
        raise NotImplementedError

    def parity(self, oracle):
        """Compares rows of this rank's output with the oracle: (rows checked, ok, detail)."""
        raise NotImplementedError

    def e2e_setup(self):
        raise NotImplementedError

    def e2e_step(self):
        raise NotImplementedError

    def config(self) -> dict:
        raise NotImplementedError


class BlurWorkload(Workload):
    """8192 x 8192 stored image; as in the reference's app (apps/blur/blur.cpp:28-44) the output is
    8188 x 8188: the last two rows and columns of the stored image are padding."""
    name = "blur"
    metric = "fused two-stage blur, algorithmic HBM bytes per second"
    unit = "GB/s"
    dtype = "f32"
    kernel = "blur3x3_reg_kernel"
    N = 8192
    VARIANT = None      # --variant: a kernel variant of the library's test hook (N = 1 only)

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        super().__init__(ctx, rank, world, torch, dist, mode)
        from gern_b200 import sharding
        self.sharding = sharding
        n = self.N
        # weak: the job's image has world * 8192 stored rows (8192 per GPU); strong: the one
        # 8192-row image.  Either way the last two stored rows and columns are padding, so the
        # valid image has stored_rows - 2 rows and 8190 columns.
        stored = n if mode != "weak" else world * n
        self.band = sharding.blur_band(stored - 2, world, rank)
        rows = self.band.band_rows
        self.oc = n - 4                                   # output columns
        self.out = torch.empty((self.band.out_rows, self.oc), device="cuda")
        self.halo = None
        self.transport = "none"
        # A band under 48 MiB is a 10-us kernel whose launches the host cannot issue evenly from
        # eight Python processes: its timed steps are captured into one CUDA graph.  (Such a band
        # reads its halo rows itself; larger bands have them prefetched on a second stream, which
        # a graph of this stream would not hold, and are long enough not to need one.)
        small = rows * n * 4 < (48 << 20)
        self.graph_ok = world > 1 and (small or os.environ.get("GERN_B200_BENCH_GRAPH") == "1")
        if self.graph_ok and not small:
            from gern_b200 import api
            import ctypes
            api.lib.gb200_ctx_set_halo_prefetch_min_bytes(ctx.handle, ctypes.c_longlong(1 << 60))
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        if world > 1:
            # Preferred: the band lives in symmetric memory and the library is handed the address
            # of the next rank's first two rows; every step it has a copy engine fetch them over
            # NVLink into a local slot that the kernel's last block row waits for (no collective,
            # no extra launch, and the kernel itself reads local memory only).  Fallback: NCCL
            # send/recv into a local halo buffer each step.
            cap = -(-(stored - 2) // world) + 2
            try:
                import torch.distributed._symmetric_memory as symm
                buf = symm.empty((cap, n), dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
                hdl = symm.rendezvous(buf, dist.group.WORLD)
                self.x = buf[:rows]
                self.x.copy_(torch.rand((rows, n), generator=g, device="cuda"))
                if self.band.recvs_halo:
                    peer = hdl.get_buffer(rank + 1, (cap, n), torch.float32)
                    self.halo = peer[0:2]
                self.transport = "copy engine over NVLink from the neighbour's band (symmetric memory) into a local slot, inside the step"
                self._symm = (buf, hdl)
                # every band is complete before any rank's kernel may read a neighbour's rows
                torch.cuda.synchronize()
                dist.barrier()
            except Exception as e:  # noqa: BLE001
                self.transport = f"NCCL send/recv ({type(e).__name__})"
                self.x = torch.rand((rows, n), generator=g, device="cuda")
                self.halo = torch.empty((2, n), device="cuda") if self.band.recvs_halo else None
                self.side = torch.cuda.Stream()
        else:
            self.x = torch.rand((n, n), generator=g, device="cuda")[:rows]

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
        if self.transport.startswith("NCCL"):
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                for w in self.sharding.exchange_blur_halo(self.dist, band, self.x[0:2], self.halo):
                    w.wait()
            torch.cuda.current_stream().wait_stream(self.side)
        # One launch: the last block row of the band reads the two halo rows through `halo`.
        halo = self.halo[:, : n - 2] if band.recvs_halo else None
        self.ctx.blur3x3_band(self.x[:, : n - 2], halo, self.out, stream=stream)

    def parity(self, oracle):
        """Bit equality on the first, a middle and the last 6 output rows of this rank's band.  The
        last 6 consumed the neighbour's two rows: those are fetched for the check by an NCCL
        send/recv (sharding.exchange_blur_halo), a path that shares nothing with the kernel's own
        peer loads."""
        torch = self.torch
        n, band = self.N, self.band
        if self.world > 1:
            nb = torch.empty((2, n), device="cuda")
            for w in self.sharding.exchange_blur_halo(self.dist, band, self.x[0:2].contiguous(), nb):
                w.wait()
            torch.cuda.synchronize()
            avail = torch.cat([self.x, nb]) if band.recvs_halo else self.x
        else:
            avail = self.x
        got = self.out.cpu().numpy() if band.out_rows <= 64 else None
        checked, ok, detail = 0, True, ""
        starts = sorted({0, max(0, band.out_rows // 2 - 3), max(0, band.out_rows - 6)})
        for r0 in starts:
            cnt = min(6, band.out_rows - r0)
            if cnt <= 0:
                continue
            xs = np.ascontiguousarray(avail[r0:r0 + cnt + 2, : n - 2].cpu().numpy())
            want = oracle.blur_xy(xs)
            have = got[r0:r0 + cnt] if got is not None else self.out[r0:r0 + cnt].cpu().numpy()
            checked += cnt
            if not np.array_equal(have, want):
                ok = False
                detail = f"rank {self.rank}: blur rows {r0}..{r0 + cnt} differ from the oracle"
        return checked, ok, detail

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
        if self.mode == "strong":
            what = f"fused 2-stage 3-tap blur, one {n}x{n} fp32 image -> {n - 4}x{n - 4}, cut into {self.world} row bands"
        else:
            what = f"fused 2-stage 3-tap blur, {n}x{n} fp32 image per GPU -> {n - 4}x{n - 4}"
        transport = self.transport
        if self.world > 1 and self.graph_ok and transport.startswith("copy engine"):
            transport = "peer loads over NVLink from the neighbour's band (symmetric memory), inside the kernel"
        cfg = {"timed_as": getattr(self, "timed_as", "K launches back to back")} if self.world > 1 else {}
        return {**cfg, "workload": what, "rows_per_gpu": self.band.band_rows if self.mode == "strong" else n, "cols": n,
                "sharding": f"row bands, 2-row halo by {transport}" if self.world > 1 else "none",
                "cache": "inputs larger than L2 (268 MB read + 268 MB written per step)" if self.mode != "strong"
                else "bands of the one image (at 8 GPUs a band's 34 MB of input fits L2; it is rewritten by no one, so steps after the first may hit)"}

    def cpu_sample(self, oracle, ref):
        rows = 1024
        x = np.random.default_rng(0).random((rows + 2, self.N - 2), dtype=np.float32)
        fn = ref.blur_xy if ref is not None else oracle.blur_xy
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 5.0 or reps < 2:
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

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        super().__init__(ctx, rank, world, torch, dist, mode)
        from gern_b200 import sharding
        b, e = sharding.row_block(self.ROWS, self.parts, rank if mode == "strong" else 0)
        self.rows = e - b
        g = torch.Generator(device="cuda").manual_seed(99 + rank)
        self.x = torch.randn((self.rows, self.COLS), generator=g, device="cuda") * 3
        self.out = torch.empty_like(self.x)

    def units_per_step(self):
        return float(2 * self.rows * self.COLS * 4)

    def step(self, stream):
        self.ctx.softmax_rows(self.x, self.out, stream=stream)

    def parity(self, oracle):
        torch = self.torch
        idx = spread_rows(self.rows, 64)
        sel = torch.tensor(idx, device="cuda")
        xs = np.ascontiguousarray(self.x[sel].cpu().numpy())
        got = self.out[sel].cpu().numpy().astype(np.float64)
        rel_of = lambda want: float((np.abs(got - want) / np.maximum(np.abs(want), 1e-30)).max())
        # 1e-5 against the exact softmax; against the fp32 oracle, 1e-5 plus the drift of its
        # sequential fp32 row sum (the reference's sum_row) from the exact value on the same rows
        exact, want = oracle.softmax_rows_f64(xs), oracle.softmax_rows(xs)
        drift = float((np.abs(want - exact) / np.maximum(exact, 1e-30)).max())
        ok = rel_of(exact) <= 1e-5 and rel_of(want) <= 1e-5 + drift
        return len(idx), ok, "" if ok else f"rank {self.rank}: softmax rel err {rel_of(want):.3g} vs oracle, {rel_of(exact):.3g} vs fp64"

    def e2e_setup(self):
        torch = self.torch
        self.h_in = (torch.randn((self.ROWS, self.COLS)) * 3).pin_memory()
        self.h_out = torch.empty((self.ROWS, self.COLS)).pin_memory()
        b = self.ROWS * self.COLS * 4
        return b, b

    def e2e_units(self):
        return float(2 * self.ROWS * self.COLS * 4)

    def e2e_step(self):
        self.ctx.softmax_rows_host(self.h_in, self.h_out)

    def config(self):
        what = (f"row softmax fp32, one {self.ROWS}x{self.COLS} matrix cut into {self.world} row blocks"
                if self.mode == "strong" else f"row softmax fp32 {self.ROWS}x{self.COLS} per GPU")
        mb = 2 * self.rows * self.COLS * 4 / 2 ** 20
        return {"workload": what, "sharding": "rows", "rows_per_gpu": self.rows,
                "cache": f"inputs larger than L2 ({mb:.0f} MiB read + written per step)"}

    def cpu_sample(self, oracle, ref):
        rows = 2048
        x = (np.random.default_rng(0).standard_normal((rows, self.COLS)) * 3).astype(np.float32)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 5.0 or reps < 2:
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

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        super().__init__(ctx, rank, world, torch, dist, mode)
        from gern_b200 import sharding
        m, n, k = self.SHAPE if self.SHAPE else (self.N, self.N, self.N)
        if mode == "strong":
            b, e = sharding.row_block(m, world, rank)
            m = e - b
        self.mnk = (m, n, k)
        ga = torch.Generator(device="cuda").manual_seed(7 + rank)
        # B is the replicated operand: the same bits on every rank
        gb = torch.Generator(device="cuda").manual_seed(7000)
        self.a = (torch.randn((m, k), generator=ga, device="cuda") * 0.02).to(torch.bfloat16)
        self.b = (torch.randn((n, k), generator=gb, device="cuda") * 0.02).to(torch.bfloat16)
        self.c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

    def units_per_step(self):
        m, n, k = self.mnk
        return 2.0 * m * n * k

    def step(self, stream):
        self.ctx.gemm_bf16(self.a, self.b, self.c, stream=stream)

    def parity(self, oracle):
        torch = self.torch
        m = self.mnk[0]
        idx = spread_rows(m, 64)
        sel = torch.tensor(idx, device="cuda")
        want = oracle.gemm_bf16(bits_of(self.a[sel], torch), bits_of(self.b, torch))
        got = self.c[sel].float().cpu().numpy()
        err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
        ok = err <= 1e-2
        return len(idx), ok, "" if ok else f"rank {self.rank}: gemm_bf16 rel Frobenius {err:.3g} > 1e-2"

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
        return 2.0 * self.N ** 3

    def e2e_step(self):
        self.ctx.gemm_bf16_host(self.h_a, self.h_b, self.h_c)

    def config(self):
        m, n, k = self.mnk
        if self.SHAPE:
            return {"workload": f"bf16 GEMM M={m} N={n} K={k} per GPU (A row-major, B column-major, fp32 accumulate)",
                    "sharding": "M panels, B replicated", "cache": "operands as they are (may fit L2)"}
        if self.mode == "strong":
            return {"workload": f"bf16 GEMM, one M=N=K={n} problem cut into {self.world} M panels of {m} rows (A row-major, B column-major, fp32 accumulate)",
                    "sharding": "M panels, B replicated", "rows_per_gpu": m,
                    "cache": "B (128 MiB) alone exceeds L2"}
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


class GemmEpilogueWorkload(GemmBf16Workload):
    """The bf16 GEMM with consumers fused into its epilogue (gb200_gemm_bf16_epilogue): E = exp(A B - sub)
    stored as bf16 plus the row sums of E, the shape of a softmax numerator.  A side measurement
    beside the plain GEMM (same operands, same FLOP count; the consumers add 67 M exponentials)."""
    name = "gemm_epilogue"
    metric = "bf16 GEMM with exp and row-sum consumers in the epilogue, dense FLOP per second"
    kernel = "gemm_bf16_2cta_kernel<epilogue>"
    sharded = False
    VARIANT = None      # --variant 1: single-CTA tiles, 2: CTA pairs (default: the library picks)

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        super().__init__(ctx, rank, world, torch, dist, mode)
        m = self.mnk[0]
        self.sub = torch.full((m,), 0.25, device="cuda")
        self.row_sum = torch.empty((m,), device="cuda")

    def step(self, stream):
        self.ctx.gemm_bf16_epilogue(self.a, self.b, self.c, alpha=1.0, row_sub=self.sub, apply_exp=True,
                                    row_sum=self.row_sum, stream=stream, variant=self.VARIANT)

    def launches_note(self):
        return "two launches per step: the row-sum vector is initialised by a small kernel"

    def parity(self, oracle):
        torch = self.torch
        idx = spread_rows(self.mnk[0], 64)
        sel = torch.tensor(idx, device="cuda")
        t, _, rs = oracle.gemm_bf16_epilogue(bits_of(self.a[sel], torch), bits_of(self.b, torch), alpha=1.0,
                                             row_sub=np.full(len(idx), 0.25, np.float32), apply_exp=True)
        got = self.c[sel].float().cpu().numpy()
        err = float(np.linalg.norm(got - t) / max(np.linalg.norm(t), 1e-30))
        rel = float(np.abs(self.row_sum[sel].cpu().numpy() - rs).max() / np.abs(rs).max())
        ok = err <= 1e-2 and rel <= 1e-3
        return len(idx), ok, "" if ok else f"gemm_epilogue: C rel Frobenius {err:.3g}, row sums {rel:.3g}"

    def e2e_setup(self):
        return 0, 0

    def config(self):
        m, n, k = self.mnk
        return {"workload": f"bf16 GEMM M={m} N={n} K={k} with E = exp(A B - sub) stored as bf16 and row sums of E (fused consumers)",
                "sharding": "replicas only", "cache": "flush not needed: 384 MB of operands > L2"}

    def cpu_sample(self, oracle, ref):
        return 0.0, "none"


class AttentionWorkload(Workload):
    name = "attention"
    metric = "GEMM->softmax->GEMM chain, dense FLOP per second"
    unit = "TFLOP/s"
    dtype = "bf16"
    bound = "tensor"
    kernel = "attention_bf16_kernel"
    NQ, NKV, D = 32768, 4096, 128

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        super().__init__(ctx, rank, world, torch, dist, mode)
        from gern_b200 import sharding
        b, e = sharding.row_block(self.NQ, self.parts, rank if mode == "strong" else 0)
        self.nq = e - b
        gq = torch.Generator(device="cuda").manual_seed(17 + rank)
        gkv = torch.Generator(device="cuda").manual_seed(1700)        # K, V replicated: same bits everywhere
        self.q = torch.randn((self.nq, self.D), generator=gq, device="cuda").to(torch.bfloat16)
        self.k = torch.randn((self.NKV, self.D), generator=gkv, device="cuda").to(torch.bfloat16)
        self.v = torch.randn((self.NKV, self.D), generator=gkv, device="cuda").to(torch.bfloat16)
        self.o = torch.empty((self.nq, self.D), dtype=torch.bfloat16, device="cuda")
        self.scale = 1.0 / math.sqrt(self.D)

    def units_per_step(self):
        return 4.0 * self.nq * self.NKV * self.D

    def step(self, stream):
        self.ctx.attention_bf16(self.q, self.k, self.v, self.o, self.scale, stream=stream)

    def parity(self, oracle):
        torch = self.torch
        idx = spread_rows(self.nq, 64)
        sel = torch.tensor(idx, device="cuda")
        want = oracle.attention_bf16(bits_of(self.q[sel], torch), bits_of(self.k, torch), bits_of(self.v, torch), self.scale)
        got = self.o[sel].float().cpu().numpy()
        err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
        ok = err <= 1e-2
        return len(idx), ok, "" if ok else f"rank {self.rank}: attention rel Frobenius {err:.3g} > 1e-2"

    def e2e_setup(self):
        torch = self.torch
        self.h_q = torch.randn((self.NQ, self.D)).to(torch.bfloat16).pin_memory()
        self.h_k = torch.randn((self.NKV, self.D)).to(torch.bfloat16).pin_memory()
        self.h_v = torch.randn((self.NKV, self.D)).to(torch.bfloat16).pin_memory()
        self.h_o = torch.empty((self.NQ, self.D), dtype=torch.bfloat16).pin_memory()
        return (self.NQ + 2 * self.NKV) * self.D * 2, self.NQ * self.D * 2

    def e2e_units(self):
        return 4.0 * self.NQ * self.NKV * self.D

    def e2e_step(self):
        self.ctx.attention_bf16_host(self.h_q, self.h_k, self.h_v, self.h_o, self.scale)

    def config(self):
        what = (f"softmax(Q K^T / sqrt(128)) V, one Q {self.NQ}x128 cut into {self.world} row blocks of {self.nq}, K,V {self.NKV}x128 bf16"
                if self.mode == "strong" else
                f"softmax(Q K^T / sqrt(128)) V, Q {self.NQ}x128, K,V {self.NKV}x128 bf16 per GPU")
        return {"workload": what, "sharding": "Q rows, K and V replicated", "rows_per_gpu": self.nq,
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
    sharded = False
    SHAPE = (4096, 4096, 4096)
    VS_CUBLAS = False

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        super().__init__(ctx, rank, world, torch, dist, mode)
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

    def parity(self, oracle):
        torch = self.torch
        idx = spread_rows(self.SHAPE[0], 16)
        sel = torch.tensor(idx, device="cuda")
        want = (self.a[sel].double() @ self.b.double()).cpu().numpy()
        got = self.c[sel].cpu().numpy()
        err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
        ok = err < 1e-5
        return len(idx), ok, "" if ok else f"gemm_f32 rel Frobenius {err:.3g} vs fp64"

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
    kernel = "gemm_f32_fused_kernel"
    sharded = False
    N = 512

    def __init__(self, ctx, rank, world, torch, dist=None, mode="single"):
        super().__init__(ctx, rank, world, torch, dist, mode)
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

    def parity(self, oracle):
        """The whole product against Gern's tiled CPU loop nest (tiles 64/64/64): the apps' bar
        |delta| < 1e-3 (gernels/mm/float-error.h) and relative Frobenius error < 1e-5."""
        a = self.a.cpu().numpy()
        want = oracle.matmul_tiled(a, a, 64, 64, 64)
        got = self.c.cpu().numpy()
        err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        ok = err < 1e-5 and float(np.abs(got - want).max()) < 1e-3
        return self.N, ok, "" if ok else f"gemm_f32 512^3 rel Frobenius {err:.3g}"

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
        while time.perf_counter() - t0 < 3.0 or reps < 2:
            fn()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return 2.0 * self.N ** 3 / dt / 1e12, f"whole 512^3 problem, tiles 64/64/64 ({reps} passes)"


WORKLOADS = {w.name: w for w in (BlurWorkload, SoftmaxWorkload, GemmBf16Workload, AttentionWorkload,
                                 GemmF32Workload, GemmF32ShapeWorkload, GemmEpilogueWorkload)}


HOST_ENTRY = {"blur": "gb200_blur3x3_f32_host", "softmax": "gb200_softmax_rows_f32_host",
              "gemm_bf16": "gb200_gemm_bf16_host", "attention": "gb200_attention_bf16_host",
              "gemm_f32": "gb200_gemm_f32_host", "gemm_f32_shape": "gb200_gemm_f32_host"}


def scale_of(unit):
    return 1e9 if unit == "GB/s" else 1e12


# ----------------------------------------------------------------------------------------------
# reference arm: the reference's CPU path on the host cores
# ----------------------------------------------------------------------------------------------
def reference_sample(name, oracle, ref, cores):
    """(fn, units per call, sample text, kind, cores) for one workload's bounded CPU sample."""
    from oracle import pyoracle
    cls = WORKLOADS[name]
    n = getattr(cls, "N", None)
    kind = "port"
    if name == "blur":
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
    elif name == "softmax":
        rows = 1024
        x = (np.random.default_rng(0).standard_normal((rows, cls.COLS)) * 3).astype(np.float32)
        units = 2 * rows * cls.COLS * 4
        sample = f"{rows} x {cls.COLS} rows per step"
        fn = lambda: oracle.softmax_rows(x)
    elif name == "gemm_f32":
        a = pyoracle.mt19937_uniform(n * n, -1.0, 1.0).reshape(n, n)
        units = 2.0 * n ** 3
        sample = "whole 512^3 problem per step (tiles 64/64/64)"
        if ref is not None:
            kind, cores, fn = "reference", 1, (lambda: ref.matmul_tiled(a, a, 64, 64, 64))
        else:
            fn = lambda: oracle.matmul_tiled(a, a, 64, 64, 64)
    elif name == "gemm_bf16":
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
    return fn, units, sample, kind, cores


def time_reference(name, oracle, ref, all_cores, warmup, steps):
    fn, units, sample, kind, cores = reference_sample(name, oracle, ref, all_cores)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    per = sum(times) / len(times)
    cls = WORKLOADS[name]
    value = units / per / scale_of(cls.unit)
    return {"value": value, "unit": cls.unit, "ms_per_step": per * 1e3,
            "cpu_baseline": {"value": value, "unit": cls.unit, "cores": cores, "kind": kind, "sample": sample}}


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
    main = time_reference(args.workload, oracle, ref, cores, args.warmup, args.steps)
    # the configuration this arm stands beside: the library arm's, word for word
    shell = cls.__new__(cls)
    shell.world = world
    shell.mode = "single" if world == 1 else "weak"
    shell.transport = "copy engine over NVLink from the neighbour's band (symmetric memory) into a local slot, inside the step"
    shell.band = type("B", (), {"band_rows": getattr(cls, "N", 0)})()
    shell.rows = getattr(cls, "ROWS", 0)
    shell.nq = getattr(cls, "NQ", 0)
    shell.mnk = (getattr(cls, "N", 0),) * 3
    cfg = cls.config(shell)
    line = {"impl": "reference", "metric": cls.metric, "value": main["value"], "unit": cls.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": cls.dtype, "data": "synthetic", "config": cfg,
            "cpu_baseline": main["cpu_baseline"],
            "e2e": {"value": main["value"], "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    also = {}
    for name in [s for s in args.also.split(",") if s in WORKLOADS and s != args.workload]:
        r = time_reference(name, oracle, ref, cores, min(args.warmup, 2), min(args.steps, 5))
        r["metric"] = WORKLOADS[name].metric
        r["e2e"] = {"value": r["value"], "unit": r["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
        also[name] = r
    if also:
        line["also"] = also
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="blur", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="gern_b200", choices=["gern_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison after the timed loops")
    ap.add_argument("--small", action="store_true",
                    help="reduced sizes (still larger than L2) for profiler captures; not a bench number")
    ap.add_argument("--variant", type=int, default=None,
                    help="blur, one GPU: kernel variant of gb200_blur3x3_f32_variant (52 = TMA-staged, short strips); "
                         "gemm_epilogue: 1 = single-CTA tiles, 2 = CTA pairs")
    ap.add_argument("--shape", default="", help="gemm_bf16 / gemm_f32: M,N,K of a side measurement (kernel only)")
    ap.add_argument("--vs-cublas", action="store_true",
                    help="with --shape: add cuBLAS (torch.matmul) timed the same way under 'library'")
    ap.add_argument("--also", default="softmax,attention,gemm_bf16,gemm_f32",
                    help="comma list of further workloads reported under 'also'")
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
    # Before any host buffer is pinned: run on the CPUs next to this rank's GPU.
    numa = bind_to_gpu_numa(local_rank) if world > 1 else "single rank: not bound"
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from gern_b200 import api
    ctx = api.Context(local_rank)
    oracle = None
    if not args.no_parity or not args.no_cpu_baseline:
        from oracle import pyoracle           # the checker and the CPU baseline; never the product
        oracle = pyoracle.Oracle()
        oracle.set_threads(max(1, oracle.max_threads() // max(1, world)))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def allreduce(value, op):
        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=getattr(dist.ReduceOp, op))
        return float(t.item())

    if args.variant is not None and args.workload == "gemm_epilogue":
        GemmEpilogueWorkload.VARIANT = args.variant
        if args.variant == 1:
            GemmEpilogueWorkload.kernel = "gemm_bf16_tc_kernel<epilogue>"
    elif args.variant is not None:
        BlurWorkload.VARIANT = args.variant
        if 2 <= args.variant < 40 or args.variant >= 50:
            BlurWorkload.kernel = "blur3x3_tma_kernel"
    if args.workload == "gemm_epilogue":
        args.no_e2e = args.no_cpu_baseline = True
    if args.shape:
        GemmBf16Workload.SHAPE = tuple(int(v) for v in args.shape.split(","))
        GemmF32ShapeWorkload.SHAPE = GemmBf16Workload.SHAPE
        args.no_e2e = args.no_cpu_baseline = True
        args.also = ""
        if args.workload == "gemm_f32":
            args.workload = "gemm_f32_shape"
    GemmBf16Workload.VS_CUBLAS = args.vs_cublas
    GemmF32ShapeWorkload.VS_CUBLAS = args.vs_cublas
    if args.small:
        SoftmaxWorkload.ROWS = 16384
        GemmBf16Workload.N = 4096
        AttentionWorkload.NQ = 8192
        args.also = ""

    failures = []

    def timed_loop(wl, steps, warmup, group=True):
        """W warm-up steps, then K steps between one pair of events.  group=False: this rank alone
        (no barrier with the others).  Returns (total ms as max over ranks, this rank's ms per launch)."""
        stream = torch.cuda.current_stream()
        sync = barrier if group else torch.cuda.synchronize
        for _ in range(warmup):
            wl.step(stream)
        sync()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        pre = getattr(wl, "pre_step", None)
        evs = []
        graph = None
        if pre is None and getattr(wl, "graph_ok", False):
            # the K timed launches as one graph (see BlurWorkload): every call under capture is one
            # the warm-up has already made, so nothing but kernel launches is recorded
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    for i in range(steps):
                        wl.step(torch.cuda.current_stream())
                wl.timed_as = "one CUDA graph of the K launches"
            except Exception as e:  # noqa: BLE001  (fall back to launching one by one)
                graph = None
                torch.cuda.synchronize()
                wl.timed_as = f"K launches back to back (graph capture failed: {type(e).__name__})"
        sync()
        l0 = ctx.launch_count()
        start.record()
        if graph is not None:
            graph.replay()
        elif pre is None:
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
        launches = steps if graph is not None else ctx.launch_count() - l0
        sync()
        if pre is None:
            mine = start.elapsed_time(stop) / steps
        else:
            mine = statistics.mean(a.elapsed_time(b) for a, b in evs)
        total = mine * steps
        if group:
            total = allreduce(total, "MAX")
        return total, mine, launches

    def run_workload(name, mode, steps, warmup, want_e2e, want_cpu):
        wl = WORKLOADS[name](ctx, rank, world, torch, dist, mode)
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        total_ms, per_launch_ms, launches = timed_loop(wl, steps, warmup)
        clocks = sampler.stop() if rank == 0 else None
        ctx.sync()  # also surfaces a kernel that gave up a bounded wait
        all_units = allreduce(wl.units_per_step(), "SUM")
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
                            "frac": achieved / peak,
                            "traffic": load_traffic(wl.kernel) if mode == "single" else None,
                            "peak_source": peaks["source"], "kernel": wl.kernel,
                            "kernel_ms": per_launch_ms},
               "gpu_launches": launches, "clocks": clocks}
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, round(per_launch_ms, 6))
            res["ms_per_step_by_rank"] = gathered
        if not args.no_parity:
            rows, ok, detail = wl.parity(oracle)
            all_rows = int(allreduce(rows, "SUM"))
            all_ok = allreduce(1.0 if ok else 0.0, "MIN") > 0.5
            res["parity"] = {"checked_rows": all_rows, "ok": all_ok, "against": "CPU oracle, every rank its own rows"}
            if not ok:
                failures.append(detail)
                sys.stderr.write(detail + "\n")
            if not all_ok and ok:
                failures.append(f"{name}: another rank's rows differ from the oracle")
        if getattr(wl, "VS_CUBLAS", False) and world == 1:
            res["library"] = wl.library_baseline(steps, warmup)
        if want_e2e:
            h2d, d2h = wl.e2e_setup()
            e_steps = max(2, min(steps, 5))
            alone = None
            if world > 1:
                # rank 0 alone first: the figure the all-ranks aggregate is compared with
                if rank == 0:
                    wl.e2e_step()
                    t0 = time.perf_counter()
                    for _ in range(e_steps):
                        wl.e2e_step()
                    torch.cuda.synchronize()
                    alone = wl.e2e_units() * e_steps / (time.perf_counter() - t0) / sc
                barrier()
            wl.e2e_step()
            barrier()
            t0 = time.perf_counter()
            for _ in range(e_steps):
                wl.e2e_step()
            torch.cuda.synchronize()
            dt = allreduce(time.perf_counter() - t0, "MAX")
            e_val = wl.e2e_units() * world * e_steps / dt / sc
            res["e2e"] = {"value": e_val, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                          "steps": e_steps, "ms_per_step": dt / e_steps * 1e3,
                          "api": HOST_ENTRY[name] + ", pinned host buffers"}
            if world > 1:
                alone = allreduce(alone or 0.0, "MAX")
                res["e2e"].update({"one_rank_alone": alone, "efficiency_vs_one_rank": e_val / (world * alone) if alone else None,
                                   "host_binding": numa,
                                   "note": "every rank moves its own whole image through its own PCIe link; the shared limit is host DRAM / the PCIe roots"})
        if want_cpu and rank == 0 and world == 1:
            oracle.set_threads(oracle.max_threads())
            v, sample = wl.cpu_sample(oracle, None)
            res["cpu_baseline"] = {"value": v, "unit": wl.unit, "cores": oracle.max_threads(), "kind": "port", "sample": sample}
        del wl
        torch.cuda.empty_cache()
        return res

    def strong_with_reference(name, steps, warmup):
        """The one configuration cut `world` ways, beside the same problem on rank 0 alone."""
        # Every rank runs the whole problem by itself first (rank 0's time is the one reported): the
        # ranks then enter the strong-scaled run in the same thermal and power state.  With rank 0
        # alone doing the 40 ms of full-size GEMMs, its panel ran a third slower than the others'.
        solo = WORKLOADS[name](ctx, 0, 1, torch, None, "single")
        _, t1, _ = timed_loop(solo, steps, warmup, group=False)
        del solo
        torch.cuda.empty_cache()
        barrier()
        t1 = allreduce(t1 if rank == 0 else 0.0, "MAX")
        r = run_workload(name, "strong", steps, warmup, False, False)
        r["one_gpu_ms_per_step"] = t1
        r["speedup_vs_one_gpu"] = t1 / r["ms_per_step"]
        r["scaling"] = "strong"
        return r

    def brief(r):
        out = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "dtype", "config", "roofline", "gpu_launches",
                                 "clocks", "parity", "e2e", "cpu_baseline", "library", "ms_per_step_by_rank",
                                 "one_gpu_ms_per_step", "speedup_vs_one_gpu", "scaling") if k in r}
        return out

    # The side workloads follow one another with host work (allocation, the oracle) in between, and
    # a sub-100-us kernel measured 5 % slower on its first launches after such a pause than once the
    # GPU had been busy for a few milliseconds: they warm up longer than the headline's W.
    SIDE_WARMUP = 50
    main_mode = "single" if world == 1 else "weak"
    main_res = run_workload(args.workload, main_mode, args.steps, args.warmup, not args.no_e2e, not args.no_cpu_baseline)
    also = {}
    side_steps = min(args.steps, 20)
    for name in [s for s in args.also.split(",") if s in WORKLOADS and s != args.workload]:
        try:
            if world == 1:
                also[name] = brief(run_workload(name, "single", side_steps, SIDE_WARMUP, not args.no_e2e, not args.no_cpu_baseline))
            elif WORKLOADS[name].sharded:
                weak = brief(run_workload(name, "weak", side_steps, SIDE_WARMUP, False, False))
                weak["scaling"] = "weak"
                also[name] = {"weak": weak, "strong": brief(strong_with_reference(name, side_steps, SIDE_WARMUP))}
        except Exception as e:  # a failing side workload must not hide the headline line
            also[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
            failures.append(f"{name}: {e}")
    if world > 1 and WORKLOADS[args.workload].sharded and args.also:
        try:
            also[args.workload + "_strong"] = brief(strong_with_reference(args.workload, side_steps, SIDE_WARMUP))
        except Exception as e:  # noqa: BLE001
            also[args.workload + "_strong"] = {"error": f"{type(e).__name__}: {e}"[:300]}
            failures.append(f"{args.workload}_strong: {e}")
    if rank == 0:
        line = {"metric": main_res["metric"], "value": main_res["value"], "unit": main_res["unit"],
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": main_res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": main_res["dtype"], "data": "synthetic",
                "config": dict(main_res["config"], **({"small": True} if args.small else {})),
                "roofline": main_res["roofline"],
                "gpu_launches": main_res["gpu_launches"], "clocks": main_res["clocks"]}
        for key in ("e2e", "cpu_baseline", "library", "parity", "ms_per_step_by_rank"):
            if key in main_res:
                line[key] = main_res[key]
        if also:
            line["also"] = also
        print(json.dumps(line), flush=True)
    n_fail = allreduce(float(len(failures)), "MAX")
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    if n_fail > 0:
        raise SystemExit("parity or side-workload failure: " + "; ".join(failures or ["on another rank"]))


if __name__ == "__main__":
    main()
