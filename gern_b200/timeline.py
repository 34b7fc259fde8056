"""Device-side timelines of two kernels, from debug builds of their sources.

    python -m gern_b200.timeline build                      # here or on the GPU machine (needs nvcc)
    python -m gern_b200.timeline attention [--cta 1] [--splits -1]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m gern_b200.timeline blur-band

`build` compiles ctx.cu, attention.cu, attention_pair.cu with -DGB200_ATTN_TRACE and blur.cu with
-DGB200_BLUR_TRACE into build/timeline/ (git-ignored); the shipped library carries no trace code.

`attention`: clock64 stamps of one CTA of the GEMM -> softmax -> GEMM kernel at the benchmark shape
(per K/V block and Q tile: S seen, maximum done, P done, arrived; the MMA warp's view; per segment:
Q reloaded, first Q K^T issued, block loop left, O complete, epilogue done) and the SM clock the
CTA saw (clock64 against %globaltimer).

`blur-band`: two ranks, one 8192-row band each in symmetric memory; %globaltimer stamps of the block
row that reads the neighbour's two rows (entry, previous kernel complete, loads back, stores
issued), of an ordinary block row, and of the last block to finish, with the halo rows read from
the peer and, for comparison, from a local copy.
"""
from __future__ import annotations

import argparse
import ctypes
import math
import os
import subprocess
import sys

from . import build as _build

OUT_DIR = os.path.join(_build.ROOT, "build", "timeline")
ATTN_LIB = os.path.join(OUT_DIR, "libattention_trace.so")
BLUR_LIB = os.path.join(OUT_DIR, "libblur_trace.so")
i64, vp = ctypes.c_int64, ctypes.c_void_p


def build_traced(cta: int = 1) -> None:
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = _build._nvcc()

    def obj(name, *flags):
        out = os.path.join(OUT_DIR, name + ".o")
        subprocess.run([nvcc] + _build.NVCC_FLAGS + list(flags) + ["-c", os.path.join(_build.CSRC, name + ".cu"), "-o", out],
                       check=True)
        return out

    ctx = obj("ctx")
    pair = obj("attention_pair")
    attn = obj("attention", "-DGB200_ATTN_TRACE", f"-DGB200_ATTN_TRACE_CTA={cta}")
    blur = obj("blur", "-DGB200_BLUR_TRACE")
    subprocess.run([nvcc, "-shared", "-o", ATTN_LIB, ctx, attn, pair, "-cudart", "static", "-lcuda"], check=True)
    subprocess.run([nvcc, "-shared", "-o", BLUR_LIB, ctx, blur, "-cudart", "static", "-lcuda"], check=True)


def _load(path: str, device: int):
    if not os.path.exists(path):
        raise SystemExit(f"{path} is missing: run `python -m gern_b200.timeline build` first")
    lib = ctypes.CDLL(path)
    h = ctypes.c_void_p()
    if lib.gb200_ctx_create(device, ctypes.byref(h)) != 0:
        raise SystemExit("gb200_ctx_create failed")
    return lib, h


def attention(splits: int) -> None:
    import numpy as np
    import torch
    lib, h = _load(ATTN_LIB, 0)
    lib.gb200_attention_bf16_splitkv.argtypes = [vp, vp, i64, vp, i64, vp, i64, vp, i64, i64, i64, i64, ctypes.c_float, vp,
                                                 ctypes.c_int]
    nq, nkv = 32768, 4096
    g = torch.Generator(device="cuda").manual_seed(17)
    q, k, v = (torch.randn((r, 128), generator=g, device="cuda").to(torch.bfloat16) for r in (nq, nkv, nkv))
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    for _ in range(60):
        rc = lib.gb200_attention_bf16_splitkv(h, q.data_ptr(), 128, k.data_ptr(), 128, v.data_ptr(), 128, o.data_ptr(), 128,
                                              nq, nkv, 128, 1 / math.sqrt(128), None, splits)
        assert rc == 0
    torch.cuda.synchronize()
    buf = (ctypes.c_longlong * (28 * 64))()
    assert lib.gb200_attn_trace_read(buf) == 0
    t = np.array(buf[:]).reshape(28, 64)
    t0 = t[0, 0]
    per_block = ["t0 S seen", "t0 max done", "t0 P done", "t0 arrived", "t1 S seen", "t1 max done", "t1 P done", "t1 arrived",
                 "mma t0 P seen", "mma t0 issued", "mma t1 P seen", "mma t1 issued"]
    per_segment = ["tma Q asked for", "tma K0 issued", "mma segment entered", "mma Q there", "mma K0 there",
                   "mma first QK issued", "t0 block loop left", "t0 O complete", "t0 epilogue done", "t1 block loop left",
                   "t1 O complete", "t1 epilogue done"]
    print(f"clock64 cycles from tile 0's first S; splits = {splits}")
    for s, name in enumerate(per_block):
        print(f"{name:20s}", " ".join(f"{int(x - t0):7d}" for x in t[s, :32] if x > 0))
    for s, name in enumerate(per_segment):
        print(f"{name:20s}", " ".join(f"{int(x - t0):7d}" for x in t[12 + s, :3] if x > 0))
    cycles, ns = int(t[26, 0] - t[24, 0]), int(t[27, 0] - t[25, 0])
    print(f"CTA entered at {int(t[24, 0] - t0)}, previous kernel complete at {int(t[24, 1] - t0)}, left at {int(t[26, 0] - t0)}: "
          f"{cycles} cycles in {ns} ns = {cycles / ns * 1e3:.0f} MHz")


def blur_band() -> None:
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm
    from . import sharding
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if world != 2:
        raise SystemExit("run with two ranks")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    lib, h = _load(BLUR_LIB, rank)
    lib.gb200_blur3x3_f32_band.argtypes = [vp, vp, i64, i64, i64, vp, i64, vp, i64, vp]
    n = 8192
    band = sharding.blur_band(world * n - 2, world, rank)
    rows = band.band_rows
    cap = -(-(world * n - 2) // world) + 2
    buf = symm.empty((cap, n), dtype=torch.float32, device=torch.device("cuda", rank))
    hdl = symm.rendezvous(buf, dist.group.WORLD)
    x = buf[:rows]
    x.copy_(torch.rand((rows, n), device="cuda"))
    out = torch.empty((band.out_rows, n - 4), device="cuda")
    torch.cuda.synchronize()
    dist.barrier()
    remote = hdl.get_buffer(rank + 1, (cap, n), torch.float32)[0:2] if band.recvs_halo else None
    local = remote.clone() if remote is not None else None
    torch.cuda.synchronize()
    dist.barrier()

    def run(halo, label, chain=10, reps=5):
        # every rank calls run() the same number of times: it holds barriers
        def launch():
            return lib.gb200_blur3x3_f32_band(h, x.data_ptr(), n, rows, n - 2, halo.data_ptr() if halo is not None else None,
                                              n, out.data_ptr(), n - 4, None)
        for _ in range(20):
            assert launch() == 0
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(reps):
            stamps = (ctypes.c_ulonglong * 16)()
            lib.gb200_blur_trace_read(stamps)          # resets
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(chain):
                launch()
            e1.record()
            torch.cuda.synchronize()
            lib.gb200_blur_trace_read(stamps)
            t = list(stamps)
            first = [int(t[i]) - int(t[1]) for i in range(4)]
            other = [int(t[4 + i]) - int(t[1]) for i in range(4)]
            print(f"rank {rank} {label:13s} {e0.elapsed_time(e1) / chain * 1e3:6.1f} us/launch | first block row "
                  f"(entered, released, loads back, stores issued) {first} ns | second block row {other} ns | "
                  f"last block done {int(t[8]) - int(t[1])} ns", flush=True)

    run(remote, "halo: remote" if remote is not None else "no halo")
    run(local, "halo: local" if local is not None else "no halo")
    run(remote, "halo: remote" if remote is not None else "no halo")
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["build", "attention", "blur-band"])
    ap.add_argument("--cta", type=int, default=1, help="build: the CTA whose timeline the attention kernel records")
    ap.add_argument("--splits", type=int, default=-1, help="attention: schedule (1 whole pairs, -1 equal runs)")
    args = ap.parse_args()
    if args.what == "build":
        build_traced(args.cta)
    elif args.what == "attention":
        attention(args.splits)
    else:
        blur_band()


if __name__ == "__main__":
    main()
