"""Run under torchrun: the all-gather-fused GEMM against a plain matmul on the full weight, plus a
device-timed comparison with NCCL all_gather followed by the same GEMM kernel."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from prime_b200.ops import kernels as K  # noqa: E402
from prime_b200.parallel.ag_gemm import AllGatherLinear  # noqa: E402
from prime_b200.parallel.symm import SymmComm  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = SymmComm()
    ok = True
    for (M, N, Kd) in [(1024, 512, 256), (8192, 4096, 1024), (4096, 1024, 4096)]:
        torch.manual_seed(3)
        w_full = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
        torch.manual_seed(10 + rank)
        x = torch.randn(M, Kd, device="cuda").bfloat16()
        lin = AllGatherLinear(comm, N, Kd)
        for it in range(2):      # second call: counters keep growing, stale rows must be refreshed
            lin.weight.zero_()
            scale = 1.0 + it
            lin.local_rows().copy_(w_full[rank * lin.rows_per_rank: (rank + 1) * lin.rows_per_rank] * scale)
            torch.cuda.synchronize()
            y = lin.forward(x)
            ref = x.float() @ (w_full.float() * scale).t()
            torch.cuda.synchronize()
            K.check_status()
            err = ((y.float() - ref).norm() / ref.norm()).item()
            full_ok = torch.equal(lin.weight, (w_full * scale).bfloat16())
            if err > 1e-2 or not full_ok:
                print(f"[rank {rank}] M{M} N{N} K{Kd} call {it}: rel err {err:.4f}, gathered weight exact: {full_ok}")
                ok = False
    # timing: fused vs NCCL all_gather + GEMM (device events, max over ranks)
    M, N, Kd = 32768, 4096, 1024
    lin = AllGatherLinear(comm, N, Kd)
    lin.local_rows().normal_(0, 0.02)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    shard = lin.local_rows().clone()
    gathered = torch.empty(N, Kd, device="cuda", dtype=torch.bfloat16)

    def fused():
        lin.forward(x, out=out)

    def unfused():
        dist.all_gather_into_tensor(gathered, shard)
        K.gemm(x, gathered, out=out)

    res = {}
    for name, fn in (("fused", fused), ("nccl_then_gemm", unfused), ("gemm_only", lambda: K.gemm(x, gathered, out=out))):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(10):
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[5]], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = t.item()
    K.check_status()
    if rank == 0:
        print(f"ag-gemm M{M} N{N} K{Kd} world {world}: fused {res['fused'] * 1e3:.0f} us, nccl all_gather + gemm "
              f"{res['nccl_then_gemm'] * 1e3:.0f} us, gemm alone {res['gemm_only'] * 1e3:.0f} us")
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if flag.item() else 0)


if __name__ == "__main__":
    main()
