#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s) of Llama-150M (12 x 1024, 16 heads, SwiGLU 4096,
vocab 32000, seq 1024), bf16 compute with fp32 master weights / AdamW, ZeRO-3-sharded over the GPUs of
one node, 64 sequences per GPU per optimizer step (global batch 512 at 8 GPUs, weak scaling), synthetic
uniform-random tokens, N(0, 0.02) weights.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...        # same step through the reference's own model code

Prints ONE JSON line on rank 0. `value` is device-timed (CUDA events around exactly K steps, max over
ranks) with inputs already resident; `e2e` times the same K steps through the public
`FusedLlama.train_step` API including the per-step host->device copy of the batch from pinned memory
and the device->host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEQ = 1024
PER_GPU_SEQS = 64
VOCAB = 32000
BASELINE_TOKENS_PER_S = None   # the reference publishes no 150M number (its only throughput is 10B on 8xH100)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def max_over_ranks(ms: float, world: int) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def make_batches(n: int, rank: int, pinned: bool):
    g = torch.Generator().manual_seed(1234 + rank)
    out = []
    for _ in range(n):
        tok = torch.randint(0, VOCAB, (PER_GPU_SEQS, SEQ + 1), generator=g)
        x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        if pinned:
            x, y = x.pin_memory(), y.pin_memory()
        out.append((x, y))
    return out


def run_ours(args, world, rank, local):
    from prime_b200.engine.fused_llama import FusedLlama
    from prime_b200.models.llama import bench_configs
    from prime_b200 import native
    comm = None
    if world > 1:
        from prime_b200.parallel.symm import SymmComm
        comm = SymmComm()
    margs = bench_configs["150M"]
    eng = FusedLlama(margs, device=torch.device("cuda", local), comm=comm, ce_chunk_tokens=args.ce_chunk)
    eng.init_weights(seed=0, std=0.02)
    host = make_batches(args.steps + args.warmup, rank, pinned=True)
    dev = [(x.cuda(non_blocking=True), y.cuda(non_blocking=True)) for x, y in host]
    lr = 4e-4

    def step_dev(i):
        x, y = dev[i]
        return eng.train_step(x, y, lr, micro_bs=args.micro_bs, sync_loss=False)

    for i in range(args.warmup):
        step_dev(i)
    barrier_sync(world)
    from prime_b200.ops.kernels import check_status
    check_status()
    sampler = ClockSampler(local)
    sampler.start()
    native.launch_counter_reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss, _ = step_dev(args.warmup + i)
    e1.record()
    barrier_sync(world)
    launches = native.launch_counter()
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    clocks = sampler.stop()
    final_loss = float(loss.item())
    check_status()

    # end to end through the public step API: H2D of the batch from pinned memory + D2H of the loss each step
    barrier_sync(world)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(args.steps):
        x, y = host[args.warmup + i]
        loss_f, _ = eng.train_step(x, y, lr, micro_bs=args.micro_bs, sync_loss=True)
    f1.record()
    barrier_sync(world)
    ms_e2e = max_over_ranks(f0.elapsed_time(f1), world)
    tokens = args.steps * world * PER_GPU_SEQS * SEQ
    h2d = 2 * PER_GPU_SEQS * SEQ * 8
    return {
        "value": tokens / (ms / 1e3), "ms_per_step": ms / args.steps, "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 12},
        "final_loss": final_loss, "e2e_final_loss": loss_f,
    }


def run_reference(args, world, rank, local):
    """The reference's own model / loss code (copied verbatim under baseline/_ref) driven with the FSDP2
    recipe of its train.py:144-168 (fully_shard per block + root, bf16 params, torch.compile, AdamW, clip)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "zeroband")):
        return {"unavailable": "baseline/_ref/zeroband is missing (pip install of the reference needs hatchling, absent offline)"}
    sys.path.insert(0, ref_dir)
    try:
        from zeroband.models.llama.model import ModelArgs, Transformer
        from zeroband.loss import compute_cross_entropy_loss
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"reference import failed: {type(e).__name__}: {e}"[:200]}
    import torch.distributed as dist
    torch.set_float32_matmul_precision("high")
    margs = ModelArgs(dim=1024, n_layers=12, n_heads=16, multiple_of=4096, vocab_size=VOCAB, max_seq_len=SEQ, attn_fn="flex")
    torch.manual_seed(42)
    with torch.device("cuda"):
        model = Transformer(margs)
    for p in model.parameters():
        torch.nn.init.normal_(p, 0.0, 0.02) if p.dim() > 1 else None
    if world > 1:
        from torch.distributed.device_mesh import init_device_mesh
        mesh = init_device_mesh("cuda", (world,))
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=None)
        for lid, blk in model.layers.items():
            fully_shard(blk, mp_policy=mp, mesh=mesh, reshard_after_forward=int(lid) < margs.n_layers - 1)
        fully_shard(model, mp_policy=mp, mesh=mesh, reshard_after_forward=True)
        autocast = None
    else:
        autocast = torch.autocast("cuda", dtype=torch.bfloat16)   # 1 GPU: no FSDP wrapper to carry the bf16 policy
    opt = torch.optim.AdamW(model.parameters(), lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95))
    model = torch.compile(model)
    micro = args.ref_micro_bs
    n_micro = PER_GPU_SEQS // micro
    host = make_batches(args.steps + args.warmup, rank, pinned=True)

    def step(x, y):
        tot = 0.0
        for mb in range(n_micro):
            xs, ys = x[mb * micro:(mb + 1) * micro], y[mb * micro:(mb + 1) * micro]
            if world > 1:
                model.set_requires_gradient_sync(mb == n_micro - 1)
            if autocast is not None:
                with autocast:
                    logits = model(tokens=xs, block_mask=None).contiguous()
            else:
                logits = model(tokens=xs, block_mask=None).contiguous()
            ce, _ = compute_cross_entropy_loss(logits, ys, z_weight=None, num_chunks=None, fused_linear_weight=None)
            loss = ce / n_micro
            loss.backward()
            tot = tot + loss.detach()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        return tot

    dev = [(x.cuda(), y.cuda()) for x, y in host]
    for i in range(args.warmup):
        step(*dev[i])
    barrier_sync(world)
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(*dev[args.warmup + i])
    e1.record()
    barrier_sync(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    clocks = sampler.stop()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(args.steps):
        x, y = host[args.warmup + i]
        lf = float(step(x.cuda(non_blocking=True), y.cuda(non_blocking=True)).item())
    f1.record()
    barrier_sync(world)
    ms_e2e = max_over_ranks(f0.elapsed_time(f1), world)
    tokens = args.steps * world * PER_GPU_SEQS * SEQ
    return {"value": tokens / (ms / 1e3), "ms_per_step": ms / args.steps, "clocks": clocks, "gpu_launches": None,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * PER_GPU_SEQS * SEQ * 8,
                    "d2h_bytes_per_step": 4},
            "final_loss": float(loss.item()), "e2e_final_loss": lf}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--micro-bs", type=int, default=32)
    ap.add_argument("--ref-micro-bs", type=int, default=64)  # the reference's own 150M config uses 64 (configs/150M/H100.toml)
    ap.add_argument("--ce-chunk", type=int, default=32768)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        else:
            print(json.dumps({"metric": "tokens/sec", "value": None, "error": "no CUDA device"}))
        return
    if args.gpus != world_env:
        if world_env == 1 and args.gpus > 1:   # convenience: re-launch under torchrun
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr",
                   "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__)] + sys.argv[1:]
            raise SystemExit(subprocess.call(cmd))
    world, rank, local = dist_setup()
    try:
        res = run_ours(args, world, rank, local) if args.impl == "ours" else run_reference(args, world, rank, local)
    except Exception as e:  # noqa: BLE001
        if args.impl == "reference":
            res = {"unavailable": f"reference run failed: {type(e).__name__}: {str(e)[:160]}"}
        else:
            raise
    if rank == 0:
        if "unavailable" in res:
            print(json.dumps({"impl": "reference", "unavailable": res["unavailable"]}))
        else:
            line = {
                "metric": "tokens/sec", "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": (res["value"] / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None, "dtype": "bf16",
                "data": "synthetic uniform-random token ids (seeded), random-init N(0,0.02) weights",
                "config": {"model": "Llama-150M (12L, dim 1024, 16 heads, ffn 4096, vocab 32000)", "global_batch": world * PER_GPU_SEQS,
                           "seq_len": SEQ, "parallelism": f"zero3-dp{world}",
                           "micro_bs": args.micro_bs if args.impl == "ours" else args.ref_micro_bs,
                           "l2": "per-step working set (tens of GB of activations) far exceeds the 126 MB L2; no explicit flush"},
                "clocks": res["clocks"], "e2e": res["e2e"], "gpu_launches": res["gpu_launches"], "impl": args.impl,
                "final_loss": res["final_loss"],
            }
            print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
