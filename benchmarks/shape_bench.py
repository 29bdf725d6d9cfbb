#!/usr/bin/env python
"""Training-step timing of the fused engine on the model shapes of the named configurations, on the GPUs of one
box: tokens/s, ms per optimizer step and model-FLOP utilisation against the measured cuBLAS peak.

    python benchmarks/shape_bench.py --model 1B --seq 2048 --micro-bs 4 --steps 4
    python benchmarks/shape_bench.py --model 10B --layers 4 --seq 8192 --micro-bs 1 --steps 3   # 10B shapes, 4 of 42 blocks
    torchrun --nproc-per-node 8 benchmarks/shape_bench.py --model 10B --seq 8192 --micro-bs 1   # the full model (ZeRO-3)

`--layers` truncates the depth so that the 10B shapes (dim 4096, 32 heads / 8 KV heads of 128, ffn 14336, vocab 128256,
8192-token sequences) can be exercised on a single GPU, whose 180 GB cannot hold the full model's optimizer state.
Synthetic uniform-random tokens, random-init weights, bf16 compute, AdamW with gradient clipping.
"""
import argparse
import json
import os
import sys
from dataclasses import replace

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from prime_b200.engine.fused_llama import FusedLlama  # noqa: E402
from prime_b200.models.llama import bench_configs  # noqa: E402
from prime_b200.ops.kernels import check_status  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1B", choices=sorted(bench_configs))
    ap.add_argument("--layers", type=int, default=0, help="use only this many transformer blocks (0 = all)")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--micro-bs", type=int, default=1)
    ap.add_argument("--grad-accum", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from prime_b200.parallel.symm import SymmComm
        comm = SymmComm()
    args = bench_configs[a.model]
    if a.layers:
        args = replace(args, n_layers=a.layers)
    seq = a.seq or args.max_seq_len
    args = replace(args, max_seq_len=max(seq, 1))
    eng = FusedLlama(args, device=torch.device("cuda", local), comm=comm)
    eng.init_weights(seed=0, std=0.02)
    B = a.micro_bs * a.grad_accum
    g = torch.Generator().manual_seed(1234 + rank)
    tok = torch.randint(0, args.vocab_size, (B, seq + 1), generator=g).cuda()
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    losses = []
    for _ in range(a.warmup):
        losses.append(eng.train_step(x, y, 3e-4, micro_bs=a.micro_bs)[0])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss, gnorm = eng.train_step(x, y, 3e-4, micro_bs=a.micro_bs, sync_loss=False)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    check_status()
    n_params = sum(p.numel for p in eng.layout.params)
    n_embed = args.vocab_size * args.dim
    tokens = world * B * seq
    # 6 N (matmul parameters, the input embedding is a gather) + causal attention 12 L H hd T / 2 per token
    flops_per_token = 6 * (n_params - n_embed) + 6 * args.n_layers * args.n_heads * args.head_dim * seq
    peak = 1640.8e12
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk))["bf16_tflops"] * 1e12
    if rank == 0:
        print(json.dumps({"model": a.model, "layers": args.n_layers, "params": n_params, "seq": seq, "micro_bs": a.micro_bs,
                          "grad_accum": a.grad_accum, "n_gpus": world, "ms_per_step": ms.item(),
                          "tokens_per_s": tokens / (ms.item() / 1e3),
                          "model_tflops_per_gpu": flops_per_token * tokens / world / (ms.item() / 1e3) / 1e12,
                          "mfu_of_measured_cublas_peak": flops_per_token * tokens / world / (ms.item() / 1e3) / peak,
                          "first_loss": float(losses[0]) if losses else None, "last_loss": float(loss),
                          "max_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
