#!/usr/bin/env python
"""Hardware probes (benchmarks/hw_probe.cu): tcgen05.mma shape rates, synchronisation-primitive latencies,
mbarrier wake-up latency and special-function issue rates on one SM of the current GPU.

    python benchmarks/hw_probe.py [umma] [prim] [wake] [xu]        (default: all)

The shared library is built next to this file with nvcc on first use (sm_100a only)."""
import ctypes as C
import os
import subprocess
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "_build", "libhw_probe.so")


def build() -> str:
    src = os.path.join(HERE, "hw_probe.cu")
    if not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(SO), exist_ok=True)
        subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                               "-shared", src, "-o", SO])
    return SO


def main():
    which = set(sys.argv[1:]) or {"umma", "prim", "wake", "xu"}
    lib = C.CDLL(build())
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    if "umma" in which:
        lib.umma_bench_run.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        out = (C.c_ulonglong * 3)()
        names = {0: "128x128x16 K/K", 1: "128x64x16 MN/MN", 2: "128x64x16 K/MN", 3: "128x256x16 K/K", 5: "128x64x16 K/K",
                 4: "attention-backward mix (32 MMAs)"}
        for mode in (0, 1, 2, 3, 5, 4):
            for reps in (4, 64):
                for _ in range(2):
                    rc = lib.umma_bench_run(mode, reps, 1, out, st.data_ptr())
                print(f"umma {names[mode]:34s} {out[2]:5d} MMAs: issue {out[0] / out[2]:6.1f} cycles/MMA, until commit "
                      f"{out[1] / out[2]:6.1f} cycles/MMA (rc {rc}, status {st.item()})")
    if "prim" in which:
        lib.prim_bench_run.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        g = torch.zeros(1 << 20, device="cuda")
        out = (C.c_longlong * 12)()
        names = ["clock pair", "try_wait (complete phase)", "vote", "arrive + syncwarp", "tcgen05.ld x32 + wait", "16 st.shared.v4",
                 "fence.proxy.async", "tcgen05 fence", "bulk wait_group.read", "global load (L2 hit)"]
        for spin in (0, 3):
            for _ in range(2):
                rc = lib.prim_bench_run(spin, 100, out, g.data_ptr(), st.data_ptr())
            print(f"prim ({spin} spinning warps, rc {rc}): " + "; ".join(f"{n} {out[i] / 100:.0f}" for i, n in enumerate(names)))
    if "wake" in which:
        lib.wake_bench_run.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p]
        out = (C.c_longlong * 2)()
        for mode, name in ((0, "try_wait loop"), (1, "test_wait loop"), (2, "try_wait, 32 ns hint")):
            for delay in (200, 20000):
                for _ in range(2):
                    rc = lib.wake_bench_run(mode, 200, delay, out)
                print(f"wake {name:22s} arrive after {delay:6d} cycles: mean {out[0] / 200:.0f}, worst {out[1]} cycles (rc {rc})")
    if "xu" in which:
        out = (C.c_longlong * 8)()
        for _ in range(2):
            rc = lib.xu_bench_run(1000, out)
        names = ["ex2.approx.ftz.f32", "ex2.approx.ftz.bf16x2", "cvt.rn.bf16x2.f32", "fma.rn.f32", "ex2.approx.f16x2", "max.f32",
                 "fma.rn.bf16x2"]
        for i, n in enumerate(names):   # 8 warps on the SM = 2 per sub-partition, 16 instructions per repetition and warp
            print(f"xu {n:24s}: {out[i] / (1000 * 16 * 2):6.2f} cycles per warp instruction per sub-partition (rc {rc})")


if __name__ == "__main__":
    main()
