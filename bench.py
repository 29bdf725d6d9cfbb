#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s) of Llama-150M (12 x 1024, 16 heads, SwiGLU 4096,
vocab 32000, seq 1024), bf16 compute with fp32 master weights / AdamW, ZeRO-3-sharded over the GPUs of
one node, 64 sequences per GPU per optimizer step in one micro-batch (global batch 512 at 8 GPUs, weak scaling), synthetic
uniform-random tokens, N(0, 0.02) weights.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 8 --warmup 3
    python bench.py --impl reference ...        # same step through the reference's own model code

    python bench.py --config {150M,1B-diloco,10B,allreduce} ...   # the other named configurations (benchmarks/bench_configs.py)

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


def dist_setup(cpu_too: bool = False):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    host_only = cpu_too == "host"          # CPU ranks only (the reference's all-reduce arm): more ranks than GPUs are fine
    if not host_only:
        torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # the other configurations also talk over gloo (the reference's outer step runs on CPU tensors)
        if host_only:
            dist.init_process_group("gloo")
        else:
            dist.init_process_group("cpu:gloo,cuda:nccl" if cpu_too else "nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def run_other(args, world, rank, local):
    """1B-diloco / 10B / allreduce: benchmarks/bench_configs.py, with the clock sampler around the whole run."""
    sys.path.insert(0, os.path.join(ROOT, "benchmarks"))
    import bench_configs as BC
    table = {("1B-diloco", "ours"): BC.run_1b_diloco_ours, ("1B-diloco", "reference"): BC.run_1b_diloco_reference,
             ("10B", "ours"): BC.run_10b_ours, ("10B", "reference"): BC.run_10b_reference,
             ("allreduce", "ours"): BC.run_allreduce_ours, ("allreduce", "reference"): BC.run_allreduce_reference}
    if args.config == "allreduce" and world < 2:
        return {"unavailable": "the all-reduce sweep needs at least 2 ranks"} if args.impl == "reference" else \
            {"metric": "outer-step all-reduce ms", "value": None, "error": "needs at least 2 ranks", "config": {}}
    if args.config == "allreduce" and args.impl == "reference":
        return table[(args.config, args.impl)](args, world, rank, local)       # CPU ranks: no GPU clocks to sample
    sampler = ClockSampler(local)
    sampler.start()
    res = table[(args.config, args.impl)](args, world, rank, local)
    res["clocks"] = sampler.stop()
    return res


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
    eng = FusedLlama(margs, device=torch.device("cuda", local), comm=comm, ce_chunk_tokens=args.ce_chunk, reshard=args.reshard)
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
    out = {
        "value": tokens / (ms / 1e3), "ms_per_step": ms / args.steps, "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 16},
        "final_loss": final_loss, "e2e_final_loss": loss_f,
    }
    if world > 1:
        del eng
        torch.cuda.empty_cache()
        out["numerics"] = zero_equivalence(comm, world, rank, local)
    return out


def zero_equivalence(comm, world, rank, local):
    """Outside the timed region: the W-rank sharded engine on a split batch against a single-rank engine on the whole
    batch (same weights, same data), two optimizer steps of a small Llama. Reports the worst relative error of the fp32
    master shards, of the gradient norm and of the loss, and whether the bf16 replicas of all ranks are bit-identical."""
    import torch.distributed as dist
    from prime_b200.engine.fused_llama import FusedLlama
    from prime_b200.models.llama import ModelArgs, Transformer
    margs = ModelArgs(dim=512, n_layers=4, n_heads=8, n_kv_heads=4, ffn_hidden=1536, vocab_size=4096, max_seq_len=256,
                      init_mode="normal", init_std=0.05)
    torch.manual_seed(0)
    model = Transformer(margs)
    g = torch.Generator().manual_seed(1)
    per, T = 4, 256
    B = per * world
    tok = torch.randint(0, margs.vocab_size, (2, B, T + 1), generator=g)
    dev = torch.device("cuda", local)
    sharded = FusedLlama(margs, device=dev, comm=comm, ce_chunk_tokens=1024)
    sharded.load_from_module(model)
    single = FusedLlama(margs, device=dev, ce_chunk_tokens=1024)
    single.load_from_module(model)
    loss_err = norm_err = 0.0
    for step in range(2):
        x, y = tok[step, :, :-1].contiguous(), tok[step, :, 1:].contiguous()
        l1, n1 = single.train_step(x, y, lr=1e-3, micro_bs=per)
        lw, nw = sharded.train_step(x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per], lr=1e-3, micro_bs=per)
        lt = torch.tensor([lw], device="cuda")
        dist.all_reduce(lt)
        loss_err = max(loss_err, abs(lt.item() / world - l1) / abs(l1))
        norm_err = max(norm_err, abs(nw - n1) / n1)
    worst = 0.0
    ref = dict(single.named_master_shards())
    for name, shard in sharded.named_master_shards():
        seg = sharded.layout.segments[rank][sharded.layout.by_name[name]]
        r = ref[name][seg.row_start: seg.row_end]
        if shard.numel():
            worst = max(worst, ((shard - r).norm() / (r.norm() + 1e-12)).item())
    mine = sharded.params.view(torch.int16).to(torch.int64).sum()
    allsum = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allsum, mine)
    t = torch.tensor([worst, norm_err, loss_err], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"zero_equiv_max_rel_err": t[0].item(), "grad_norm_rel_err": t[1].item(), "loss_rel_err": t[2].item(),
            "replicas_bit_identical": all(int(a) == int(allsum[0]) for a in allsum),
            "how": f"{world}-rank sharded vs 1-rank engine, 2 optimizer steps, small Llama (dim 512, 4 layers), fp32 master shards compared"}


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
    ap.add_argument("--config", default="150M", choices=["150M", "1B-diloco", "10B", "allreduce"])
    ap.add_argument("--micro-bs", type=int, default=None)
    ap.add_argument("--ref-micro-bs", type=int, default=None)
    ap.add_argument("--ce-chunk", type=int, default=32768)
    ap.add_argument("--per-gpu-seqs", type=int, default=0, help="sequences per GPU and optimizer step (1B-diloco: 8, 10B: 2)")
    ap.add_argument("--layers", type=int, default=0, help="10B: use only this many blocks (for boxes with fewer than 8 GPUs)")
    ap.add_argument("--sizes-mb", default="", help="allreduce: comma-separated tensor sizes in MiB")
    ap.add_argument("--reshard", action="store_true", help="150M / 10B: no resident bf16 replica, blocks re-gathered when they run")
    ap.add_argument("--ckpt-dir", default="", help="10B: where the staged checkpoint is persisted (removed afterwards)")
    ap.add_argument("--skip-ckpt", action="store_true", help="10B: leave the checkpoint part out (steps and outer step only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.config == "150M":
        args.micro_bs = args.micro_bs or 64           # both arms: the micro-batch of the reference's own 150M config
        args.ref_micro_bs = args.ref_micro_bs or 64   # (configs/150M/H100.toml)
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available() and not (args.config == "allreduce" and args.impl == "reference"):
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
    host_arm = args.config == "allreduce" and args.impl == "reference"
    world, rank, local = dist_setup(cpu_too="host" if host_arm else args.config != "150M")
    try:
        if args.config == "150M":
            res = run_ours(args, world, rank, local) if args.impl == "ours" else run_reference(args, world, rank, local)
        else:
            res = run_other(args, world, rank, local)
    except Exception as e:  # noqa: BLE001
        if args.impl == "reference":
            res = {"unavailable": f"reference run failed: {type(e).__name__}: {str(e)[:160]}"}
        else:
            raise
    if rank == 0:
        if "unavailable" in res:
            print(json.dumps({"impl": "reference", "unavailable": res["unavailable"]}))
        elif args.config != "150M":
            line = {"metric": res.pop("metric", "tokens/sec"), "value": res.pop("value", None), "unit": res.pop("unit", ""),
                    "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res.pop("ms_per_step", None),
                    "higher_is_better": res.pop("higher_is_better", True), "scaling": res.pop("scaling", "weak"), "vs_baseline": None,
                    "dtype": "bf16" if args.config != "allreduce" else "fp32 payload, uint8 on the wire",
                    "data": "synthetic uniform-random token ids (seeded), random-init N(0,0.02) weights" if args.config != "allreduce"
                    else "synthetic N(0, 1e-3) fp32 values (seeded)", "impl": args.impl, "bench_config": args.config}
            line.update(res)
            print(json.dumps(line))
        else:
            line = {
                "metric": "tokens/sec", "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": (res["value"] / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None, "dtype": "bf16",
                "data": "synthetic uniform-random token ids (seeded), random-init N(0,0.02) weights",
                "config": {"model": "Llama-150M (12L, dim 1024, 16 heads, ffn 4096, vocab 32000)", "global_batch": world * PER_GPU_SEQS,
                           "seq_len": SEQ, "parallelism": f"zero3-dp{world}" + ("-reshard" if args.reshard and world > 1 else ""),
                           "micro_bs": args.micro_bs if args.impl == "ours" else args.ref_micro_bs,
                           "l2": "per-step working set (tens of GB of activations) far exceeds the 126 MB L2; no explicit flush"},
                "clocks": res["clocks"], "e2e": res["e2e"], "gpu_launches": res["gpu_launches"], "impl": args.impl,
                "final_loss": res["final_loss"],
            }
            if "numerics" in res:
                line["numerics"] = res["numerics"]
            print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
