#!/usr/bin/env python
"""Micro-benchmarks of the hand-written kernels: CUDA-event timing after warm-up with an L2 flush
between iterations, achieved TFLOP/s or GB/s, and the fraction of the measured peaks
(MEASURED_PEAKS.json next to the repo root when present, else 1.59 PFLOP/s / 6.65 TB/s).

    python benchmarks/kernel_bench.py gemm --m 65536 --n 4096 --k 1024 [--a-mn --b-mn]
    python benchmarks/kernel_bench.py attn_fwd --batch 32 --seq 1024 --heads 16 --kv 16 --hd 64
    python benchmarks/kernel_bench.py attn_bwd ...
    python benchmarks/kernel_bench.py rmsnorm|swiglu|adamw --rows 65536 --cols 1024

The same commands are what the ncu captures under profiles/ were taken with (small shapes there).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from prime_b200.ops import attention as A  # noqa: E402
from prime_b200.ops import kernels as K  # noqa: E402


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], d["hbm_gbs"], "of measured"
    return 1590.0, 6650.0, "of fallback"


def timeit(fn, iters, flush):
    for _ in range(3):
        fn()
    evs = []
    for _ in range(iters):
        flush.zero_()      # > L2 sized write between timed iterations
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    ms = sorted(a.elapsed_time(b) for a, b in evs)
    return ms[len(ms) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv", type=int, default=16)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=1024)
    ap.add_argument("--mb", type=int, default=1024, help="dl_allreduce: fp32 payload in MB")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--torch", action="store_true", help="also time the torch / library op for comparison")
    a = ap.parse_args()
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tf, gbs, tag = peaks()
    out = {"kernel": a.kernel}
    if a.kernel == "gemm":
        x = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device=dev, dtype=torch.bfloat16)
        w = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device=dev, dtype=torch.bfloat16)
        y = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        ms = timeit(lambda: K.gemm(x, w, out=y, a_mn=a.a_mn, b_mn=a.b_mn, bn=a.bn), a.iters, flush)
        fl = 2.0 * a.m * a.n * a.k
        out.update(shape=[a.m, a.n, a.k], ms=ms, tflops=fl / ms / 1e9, frac=fl / ms / 1e9 / tf, frac_of=tag)
        if a.torch:
            xe = x.t() if a.a_mn else x
            we = w if a.b_mn else w.t()
            ms_t = timeit(lambda: torch.matmul(xe, we, out=y), a.iters, flush)
            out.update(torch_ms=ms_t, torch_tflops=fl / ms_t / 1e9)
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        M = a.batch * a.seq
        qkv = (torch.randn(M, (a.heads + 2 * a.kv) * a.hd, device=dev) * 0.5).bfloat16()
        ss = A.seq_start_from_batch(a.batch, a.seq, dev)
        o, lse = A.attention_fwd(qkv, ss, a.heads, a.kv, a.hd)
        fl = 4.0 * a.batch * a.heads * a.seq * a.seq * a.hd / 2
        if a.kernel == "attn_fwd":
            ms = timeit(lambda: A.attention_fwd(qkv, ss, a.heads, a.kv, a.hd, out=o), a.iters, flush)
        else:
            do = torch.randn_like(o)
            dq = torch.empty_like(qkv)
            ms = timeit(lambda: A.attention_bwd(qkv, o, do, lse, ss, a.heads, a.kv, a.hd, dqkv=dq, seq_len=a.seq), a.iters, flush)
            fl *= 2.5
        out.update(shape=[a.batch, a.seq, a.heads, a.kv, a.hd], ms=ms, tflops=fl / ms / 1e9, frac=fl / ms / 1e9 / tf, frac_of=tag)
    elif a.kernel == "dl_allreduce":
        # the quantised pseudo-gradient all-reduce (stages A, B, C) as a one-rank group: every byte stays on this GPU, so
        # the time is the kernels' own HBM / shared-memory cost without any link in the way
        import torch.distributed as dist
        from prime_b200.config import Compression
        from prime_b200.parallel.diloco_comm import NvlinkWorkerGroup
        from prime_b200.parallel.symm import SymmComm
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        n = a.mb * (1 << 20) // 4
        grp = NvlinkWorkerGroup(SymmComm(), n)
        x = torch.randn(n, device=dev) * 1e-3
        ms = timeit(lambda: grp.all_reduce_tensor(x, Compression.UINT8), a.iters, flush)
        K.check_status()
        # HBM bytes per element: read 4, write 1 (A); read 1, write 1 (B, one rank); read 1, write 4 (C) = 12
        out.update(shape=[n], ms=ms, gbs=12.0 * n / ms / 1e6, frac=12.0 * n / ms / 1e6 / gbs, frac_of=tag)
        dist.destroy_process_group()
    elif a.kernel in ("rmsnorm", "rmsnorm_bwd", "swiglu", "swiglu_bwd", "adamw"):
        R, Cn = a.rows, a.cols
        if a.kernel == "rmsnorm":
            x = torch.randn(R, Cn, device=dev, dtype=torch.bfloat16)
            w = torch.ones(Cn, device=dev, dtype=torch.bfloat16)
            y = torch.empty_like(x)
            r = torch.empty(R, device=dev)
            ms = timeit(lambda: K.rmsnorm_fwd(x, w, 1e-5, out=y, rstd=r), a.iters, flush)
            nbytes = 2 * R * Cn * 2
        elif a.kernel == "rmsnorm_bwd":
            x = torch.randn(R, Cn, device=dev, dtype=torch.bfloat16)
            w = torch.ones(Cn, device=dev, dtype=torch.bfloat16)
            _, r = K.rmsnorm_fwd(x, w, 1e-5)
            dy, dres, dx = torch.randn_like(x), torch.randn_like(x), torch.empty_like(x)
            dw = torch.zeros(Cn, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: K.rmsnorm_bwd(x, w, r, dy, dw, dres=dres, dx=dx), a.iters, flush)
            nbytes = 4 * R * Cn * 2
        elif a.kernel == "swiglu":
            h = torch.randn(R, 2 * Cn, device=dev, dtype=torch.bfloat16)
            o = torch.empty(R, Cn, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: K.swiglu_fwd(h, out=o), a.iters, flush)
            nbytes = 3 * R * Cn * 2
        elif a.kernel == "swiglu_bwd":
            h = torch.randn(R, 2 * Cn, device=dev, dtype=torch.bfloat16)
            d = torch.randn(R, Cn, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: K.swiglu_bwd(h, d, dh13=h), a.iters, flush)
            nbytes = 5 * R * Cn * 2
        else:
            n = R * Cn
            p, m, v = torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
            g = torch.randn(n, device=dev).bfloat16()
            pl = torch.empty(n, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: K.adamw_(p, g, m, v, pl, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1), a.iters, flush)
            nbytes = n * (4 * 3 * 2 + 2 + 2)
        out.update(shape=[R, Cn], ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / gbs, frac_of=tag)
    else:
        raise SystemExit(f"unknown kernel {a.kernel}")
    K.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
