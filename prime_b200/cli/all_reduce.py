"""Pseudo-gradient all-reduce benchmark (reference: scripts/all_reduce.py:29-69).

CPU / cross-node transports (launch one process per rank, e.g. with torchrun and gloo):
    torchrun --nproc-per-node 2 -m prime_b200.cli.all_reduce --transport tcp --compression uint8 --size-mb 100
GPU transport inside one NVSwitch domain (one process per GPU, NCCL only for rendezvous):
    torchrun --nproc-per-node 8 -m prime_b200.cli.all_reduce --transport nvlink --sweep

Prints seconds / iteration, algorithmic MB/s (``size * 4 / 1e6 / t`` like the reference), bus GB/s
(``2 (W-1)/W`` of the fp32 payload) and the relative error against an exact fp32 all-reduce.
GPU numbers are device-timed with CUDA events and reported as the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from ..config import Compression


def _bench_host(args, rank, world):
    from ..collectives import TcpRing, all_reduce
    store = dist.distributed_c10d._get_default_store()
    group = TcpRing(dist.PrefixStore("bench_ring", store), rank, world, host=os.environ.get("MASTER_ADDR", "127.0.0.1")) \
        if args.transport == "tcp" else dist.group.WORLD
    n = int(args.size_mb * 1e6 / 4)
    torch.manual_seed(rank)
    x = torch.randn(n) * 1e-3
    exact = x.clone()
    dist.all_reduce(exact)
    comp = Compression(args.compression)
    y = x.clone()
    all_reduce(comp, y, dist.ReduceOp.SUM, group)
    err = ((y - exact).norm() / exact.norm()).item()
    ts = []
    for _ in range(args.iters):
        y = x.clone()
        dist.barrier()
        t0 = time.perf_counter()
        all_reduce(comp, y, dist.ReduceOp.SUM, group)
        ts.append(time.perf_counter() - t0)
    t = sorted(ts)[len(ts) // 2]
    return {"transport": args.transport, "compression": args.compression, "world": world, "numel": n, "s_per_iter": t,
            "MB_per_s": n * 4 / 1e6 / t, "bus_GB_per_s": 2 * (world - 1) / world * n * 4 / t / 1e9, "rel_err": err}


def _bench_nvlink(args, rank, world, sizes_mb):
    from ..parallel.diloco_comm import NvlinkWorkerGroup
    from ..parallel.symm import SymmComm
    grp = NvlinkWorkerGroup(SymmComm(), int(max(sizes_mb) * 1e6 / 4))
    rows = []
    for mb in sizes_mb:
        n = int(mb * 1e6 / 4)
        torch.manual_seed(rank)
        x = torch.randn(n, device="cuda") * 1e-3
        exact = x.clone()
        dist.all_reduce(exact)
        res = {}
        for name, fn in (("nvlink_uint8", lambda t: grp.all_reduce_tensor(t, Compression.UINT8)),
                         ("nccl_fp32", lambda t: dist.all_reduce(t))):
            y = x.clone()
            fn(y)
            err = ((y - exact).norm() / exact.norm()).item()
            for _ in range(3):
                fn(y)
            evs = []
            for _ in range(args.iters):
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn(y)
                e1.record()
                evs.append((e0, e1))
            torch.cuda.synchronize()
            ms = sorted(a.elapsed_time(b) for a, b in evs)[len(evs) // 2]
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
            res[name] = {"ms": ms, "bus_GB_per_s": 2 * (world - 1) / world * n * 4 / (ms / 1e3) / 1e9, "rel_err": err}
        rows.append({"size_mb": mb, "world": world, **res})
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--transport", choices=["tcp", "gloo", "nvlink"], default="tcp")
    ap.add_argument("--compression", choices=["no", "uint8"], default="uint8")
    ap.add_argument("--size-mb", type=float, default=100.0)
    ap.add_argument("--sweep", action="store_true", help="1 MB .. 4 GB (nvlink transport)")
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.transport == "nvlink":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))))
        sizes = [1, 4, 16, 64, 256, 1024, 4096] if args.sweep else [args.size_mb]
        rows = _bench_nvlink(args, rank, world, sizes)
        if rank == 0:
            for r in rows:
                print(json.dumps(r))
    else:
        dist.init_process_group("gloo")
        out = _bench_host(args, rank, world)
        if rank == 0:
            print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
