"""The configurations of bench.py other than the 150M headline: the DiLoCo 1B run (two workers inside one box), the
10B shape with activation checkpointing, an asynchronous checkpoint and the outer sync, and the pseudo-gradient
all-reduce sweep. Each has an arm for this package and an arm that drives the reference's own code (copied verbatim
under baseline/_ref). Every function returns the dict that bench.py prints as its one JSON line.

The reference pins packages that are not installed here (`toposolve`, `distributed_shampoo`); its modules are imported
with empty stand-ins for those two names registered first. Its C++ ring cannot be built on this image (the gloo headers
its `ProcessGroupGloo.hpp` include wants are absent), so the int8 ring arm runs the reference's own Python twin of that
ring (`zeroband.collectives.ring_allreduce_py`, the oracle of its tests) with the reference's C++ quantiser.
"""
from __future__ import annotations

import os
import sys
import time
import types
from dataclasses import replace

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HBM_GBS, LINK_GBS = 6534.8, 770.0       # measured copy bandwidth; measured peer copy per direction


def _peaks():
    import json
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", HBM_GBS), d.get("bf16_tflops", 1640.8)
    return HBM_GBS, 1640.8


def _max_over_ranks(v: float, group=None) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return v
    t = torch.tensor([v], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def _sync(group=None):
    torch.cuda.synchronize()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier(group=group)
    torch.cuda.synchronize()


def _reference_importable():
    """sys.path + stand-ins for the two third-party names the reference imports at module top and that are not installed."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "zeroband")):
        return "baseline/_ref/zeroband is missing"
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    if "toposolve" not in sys.modules:
        m = types.ModuleType("toposolve")

        class TSPSolver:
            def solve_tsp(self, d):
                return 0, list(range(len(d))) + [0]
        m.TSPSolver = TSPSolver
        sys.modules["toposolve"] = m
    for name in ("distributed_shampoo", "distributed_shampoo.utils", "distributed_shampoo.utils.shampoo_fsdp_utils"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            for attr in ("DistributedShampoo", "EighEigenvalueCorrectionConfig", "FullyShardShampooConfig", "ShampooPT2CompileConfig",
                         "compile_fsdp_parameter_metadata"):
                setattr(m, attr, type(attr, (), {}))
            sys.modules[name] = m
    return None


# =====================================================================================================
# all-reduce sweep (BASELINE configuration 5)
# =====================================================================================================
def _allreduce_bound_ms(n: int, world: int) -> float:
    """Roofline of the uint8 all-reduce of n fp32 values: the slower of its HBM traffic (read x, write codes, read the
    W peer slices, write and re-read the reduced codes, write the fp32 result: ~11 bytes per element) at the measured copy
    bandwidth and of the int8 payload 2 (W-1)/W n crossing NVLink at the measured peer-copy bandwidth."""
    hbm, _ = _peaks()
    t_hbm = 11.0 * n / (hbm * 1e9)
    t_link = 2.0 * (world - 1) / world * n / (LINK_GBS * 1e9)
    return 1e3 * max(t_hbm, t_link)


def run_allreduce_ours(args, world, rank, local):
    from prime_b200 import native
    from prime_b200.config import Compression
    from prime_b200.parallel.diloco_comm import NvlinkWorkerGroup
    from prime_b200.parallel.symm import SymmComm
    sizes_mb = [1, 4, 16, 64, 256, 1024, 4096] if not args.sizes_mb else [float(s) for s in args.sizes_mb.split(",")]
    iters = max(args.steps, 3)
    grp = NvlinkWorkerGroup(SymmComm(), int(max(sizes_mb) * 2 ** 20 / 4))
    rows = []
    native.launch_counter_reset()
    for mb in sizes_mb:
        n = int(mb * 2 ** 20 / 4)
        g = torch.Generator(device="cuda").manual_seed(1000 + rank)
        x = torch.randn(n, device="cuda", generator=g) * 1e-3
        exact = x.clone()
        dist.all_reduce(exact)
        row = {"size_mb": mb, "world": world}
        arms = {"nvlink_uint8": lambda t: grp.all_reduce_tensor(t, Compression.UINT8),
                "nccl_fp32": lambda t: dist.all_reduce(t)}
        for name, fn in arms.items():
            y = x.clone()
            fn(y)
            err = ((y - exact).norm() / exact.norm()).item()
            for _ in range(max(args.warmup, 3)):
                y.copy_(x)
                fn(y)
            evs = []
            for _ in range(iters):
                y.copy_(x)                      # also evicts part of L2; inputs above 126 MB exceed it anyway
                _sync()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn(y)
                e1.record()
                evs.append((e0, e1))
            torch.cuda.synchronize()
            ms = _max_over_ranks(sorted(a.elapsed_time(b) for a, b in evs)[len(evs) // 2])
            row[name] = {"ms": ms, "bus_GB_per_s": 2 * (world - 1) / world * n * 4 / (ms / 1e3) / 1e9, "rel_err": err}
        bound = _allreduce_bound_ms(n, world)
        row["nvlink_uint8"]["roofline_ms"] = bound
        row["nvlink_uint8"]["of_roofline"] = bound / row["nvlink_uint8"]["ms"]
        rows.append(row)
    # elastic resize: the last rank leaves (it is simply not part of the next reduction), then rejoins contributing a
    # zero pseudo-gradient once. Membership changes between launches, on the host, never inside a kernel.
    resize = None
    if world >= 2 and hasattr(grp, "set_participants"):
        n = int(16 * 2 ** 20 / 4)
        g = torch.Generator(device="cuda").manual_seed(2000 + rank)
        x = torch.randn(n, device="cuda", generator=g) * 1e-3
        resize = {}
        for label, members, fake_rank in (("all", list(range(world)), None), ("one_left", list(range(world - 1)), None),
                                          ("rejoined_zero", list(range(world)), world - 1)):
            grp.set_participants(members)
            contrib = x.clone()
            if rank not in members or rank == fake_rank:
                contrib.zero_()
            exact = contrib.clone()
            dist.all_reduce(exact)
            y = x.clone()
            grp.all_reduce_tensor(y, Compression.UINT8, fake=(rank == fake_rank))      # returns at once on a rank that is not a member
            err = ((y - exact).norm() / exact.norm()).item() if rank in members else 0.0
            _sync()
            resize[label] = {"participants": len(members), "rel_err": _max_over_ranks(err)}
        grp.set_participants(list(range(world)))
    launches = native.launch_counter()
    from prime_b200.ops.kernels import check_status
    check_status()
    big = next((r for r in rows if r["size_mb"] == 1024), rows[-1])
    return {"metric": "outer-step all-reduce ms (uint8 over NVLink, 1 GiB fp32 pseudo-gradient)", "value": big["nvlink_uint8"]["ms"],
            "unit": "ms", "higher_is_better": False, "scaling": "strong", "ms_per_step": big["nvlink_uint8"]["ms"],
            "gpu_launches": launches, "rows": rows, "elastic_resize": resize,
            "config": {"model": "fp32 pseudo-gradient, N(0, 1e-3) values", "sizes_mb": sizes_mb, "parallelism": f"allreduce-w{world}",
                       "l2": "the input is rewritten before every timed call; tensors of 256 MB and more exceed the 126 MB L2"}}


def run_allreduce_reference(args, world, rank, local):
    """CPU ranks over gloo, as the reference runs its outer all-reduce: its Python ring with its C++ quantiser (uint8)
    and its gloo fp32 all-reduce (compression "no"); scripts/all_reduce.py:29-58 is the harness this mirrors."""
    why = _reference_importable()
    if why:
        return {"unavailable": why}
    try:
        from zeroband.collectives import gloo_all_reduce, ring_allreduce_py
        from zeroband.C.compression import uniform_8bit_quantize
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"reference collectives import failed: {type(e).__name__}: {str(e)[:150]}"}
    c_ring = None
    try:
        from zeroband.C.collectives import ring_allreduce as c_ring  # noqa: F401
    except Exception as e:  # noqa: BLE001
        c_ring_err = f"{type(e).__name__}: gloo headers absent" if "gloo" in str(e) or "extension" in str(e) else str(e)[:120]
    gloo = dist.group.WORLD if dist.get_backend() == "gloo" else dist.new_group(backend="gloo")
    sizes_mb = [1, 4, 16, 64, 256] if not args.sizes_mb else [float(s) for s in args.sizes_mb.split(",")]
    rows = []
    for mb in sizes_mb:
        n = int(mb * 2 ** 20 / 4)
        n -= n % (2 * world * 2)        # the Python ring asserts divisibility by its chunk count
        g = torch.Generator().manual_seed(1000 + rank)
        x = torch.randn(n, generator=g) * 1e-3
        exact = x.clone()
        dist.all_reduce(exact, group=gloo)
        row = {"size_mb": mb, "world": world}
        arms = {"gloo_fp32": lambda t: gloo_all_reduce(t, dist.ReduceOp.SUM, gloo)}
        if c_ring is not None:
            arms["ref_cpp_uint8_ring"] = lambda t: c_ring(t, dist.ReduceOp.SUM, gloo)
        arms["ref_py_uint8_ring"] = lambda t: ring_allreduce_py(t, dist.ReduceOp.SUM, gloo, quantization_func=uniform_8bit_quantize)
        for name, fn in arms.items():
            y = x.clone()
            fn(y)
            err = ((y - exact).norm() / exact.norm()).item()
            ts = []
            for _ in range(2 if mb >= 64 else 3):
                y = x.clone()
                dist.barrier(group=gloo)
                t0 = time.perf_counter()
                fn(y)
                ts.append(time.perf_counter() - t0)
            t = torch.tensor([sorted(ts)[len(ts) // 2] * 1e3], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=gloo)
            ms = float(t.item())
            row[name] = {"ms": ms, "bus_GB_per_s": 2 * (world - 1) / world * n * 4 / (ms / 1e3) / 1e9, "rel_err": err}
        rows.append(row)
    big = rows[-1]
    out = {"metric": f"outer-step all-reduce ms (reference int8 ring over gloo, {big['size_mb']} MB fp32 pseudo-gradient)",
           "value": big["ref_py_uint8_ring"]["ms"], "unit": "ms", "higher_is_better": False, "scaling": "strong",
           "ms_per_step": big["ref_py_uint8_ring"]["ms"], "gpu_launches": None, "rows": rows,
           "config": {"model": "fp32 pseudo-gradient, N(0, 1e-3) values", "sizes_mb": sizes_mb, "parallelism": f"allreduce-w{world}",
                      "timing": "host wall clock, max over ranks (the reference's outer all-reduce runs on the CPU)"}}
    if c_ring is None:
        out["config"]["cpp_ring"] = f"not built ({c_ring_err}); its Python twin ring_allreduce_py ran instead"
    return out


# =====================================================================================================
# 1B DiLoCo: two workers inside the box (BASELINE configuration 3)
# =====================================================================================================
class _StaticMesh:
    """What Diloco needs from an ElasticDeviceMesh when membership is static (the reference's tests use the same kind
    of stub, tests/test_dist/test_diloco.py:25-29)."""

    def __init__(self, global_pg, cpu_local_mesh=None):
        self.global_pg = global_pg
        self.cpu_local_mesh = cpu_local_mesh

    def maybe_reinit_global_pg(self, *a, **k):
        return False

    def get_global_pg(self, maybe_reinit: bool = False):
        return self.global_pg

    def monitored_barrier(self, flag):
        b = self.global_pg.barrier()
        if hasattr(b, "wait"):
            b.wait()


def _split_workers(world: int, rank: int, workers: int):
    per = world // workers
    me = rank // per
    local_pg = worker_pg = None
    for w in range(workers):
        g = dist.new_group([w * per + r for r in range(per)])
        if w == me:
            local_pg = g
    for r in range(per):
        g = dist.new_group([w * per + r for w in range(workers)])
        if r == rank % per:
            worker_pg = g
    return per, me, local_pg, worker_pg


def run_1b_diloco_ours(args, world, rank, local):
    from prime_b200 import native
    from prime_b200.config import Compression, DilocoConfig
    from prime_b200.diloco import Diloco
    from prime_b200.engine.fused_llama import FusedLlama
    from prime_b200.models.llama import bench_configs
    from prime_b200.ops.kernels import check_status
    from prime_b200.parallel.diloco_comm import NvlinkWorkerGroup
    from prime_b200.parallel.symm import SymmComm
    workers = 2 if world >= 2 else 1
    per, me, local_pg, worker_pg = _split_workers(world, rank, workers) if world > 1 else (1, 0, None, None)
    dev = torch.device("cuda", local)
    comm = SymmComm(local_pg, dev) if per > 1 else None
    margs = bench_configs["1B"]
    seq, per_gpu, micro = margs.max_seq_len, args.per_gpu_seqs or 8, args.micro_bs or 4
    eng = FusedLlama(margs, device=dev, comm=comm)
    eng.init_weights(seed=0, std=0.02)
    n_shard = eng.master.numel()
    wgroup = NvlinkWorkerGroup(SymmComm(worker_pg, dev), n_shard) if workers > 1 else None
    g = torch.Generator().manual_seed(1234 + rank)
    tok = torch.randint(0, margs.vocab_size, (per_gpu, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    xd, yd = x.cuda(), y.cuda()
    inner = args.steps
    for _ in range(max(args.warmup, 3)):
        eng.train_step(xd, yd, 3e-4, micro_bs=micro, sync_loss=False)
    _sync()
    check_status()
    native.launch_counter_reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(inner):
        loss, _ = eng.train_step(xd, yd, 3e-4, micro_bs=micro, sync_loss=False)
    e1.record()
    _sync()
    launches = native.launch_counter()
    ms_inner = _max_over_ranks(e0.elapsed_time(e1))
    # end to end: host batches + loss read each step (a shorter stretch: the outer steps below need time too)
    k_e2e = min(inner, 10)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(k_e2e):
        eng.train_step(x, y, 3e-4, micro_bs=micro, sync_loss=True)
    f1.record()
    _sync()
    ms_e2e = _max_over_ranks(f0.elapsed_time(f1))
    outer = {}
    if wgroup is not None:
        # outer state resident on the device (the default: the copy back to the pinned host mirrors runs behind the next
        # inner step) and staged both ways inside the outer step (what a host-offloaded outer optimizer costs)
        for comp, resident in (("uint8", True), ("no", True), ("uint8", False), ("no", False)):
            dl = Diloco(DilocoConfig(inner_steps=inner, compression=Compression(comp), outer_state_resident=resident), eng,
                        _StaticMesh(wgroup))
            for _ in range(2):                      # inner progress, so the pseudo-gradient is not zero
                eng.train_step(xd, yd, 3e-4, micro_bs=micro, sync_loss=False)
            ts, after_all = [], []
            for rep in range(4):                    # first call allocates buffers and reads the host copies; the last is the number
                _sync()
                t0 = time.perf_counter()
                dl.step(eng, flag=f"{comp}{int(resident)}{rep}")
                torch.cuda.current_stream().synchronize()       # not the side stream that refreshes the host mirrors
                ts.append((time.perf_counter() - t0) * 1e3)
                # the step that follows, with its loss read: in resident mode that read shares the copy engine with the
                # refresh of the host mirrors and returns when the refresh is over
                tw = time.perf_counter()
                e0.record()
                eng.train_step(xd, yd, 3e-4, micro_bs=micro, sync_loss=True)
                e1.record()
                torch.cuda.current_stream().synchronize()
                step_after_wall = (time.perf_counter() - tw) * 1e3
                _sync()
                step_after = e0.elapsed_time(e1)
                after_all.append([round(step_after, 1), round(step_after_wall, 1)])
                dl.wait_host_state()
            phases = {k: (_max_over_ranks(v) if isinstance(v, float) else v) for k, v in getattr(wgroup, "last_timing_ms", {}).items()}
            key = comp if resident else comp + "_staged"
            outer[key] = {"outer_step_ms": _max_over_ranks(ts[-1]), "first_call_ms": _max_over_ranks(ts[0]), "device_phases_ms": phases,
                          "inner_step_after_ms": _max_over_ranks(step_after), "inner_step_after_wall_ms": _max_over_ranks(step_after_wall),
                          "inner_step_after_all_reps_device_wall_ms": after_all, "shard_numel": n_shard,
                          "host_refresh_on_demand_ms": _max_over_ranks(getattr(wgroup, "last_host_refresh_ms", 0.0)) if resident else None,
                          "includes": ("pseudo-gradient, exchange, Nesterov, inner refresh, replica refresh; the pinned host copies "
                                       "are written on demand (checkpoint save, live recovery), not per outer step") if resident else
                                      "H2D of outer params + momentum, exchange, Nesterov, D2H, replica refresh"}
            del dl
    check_status()
    tokens = inner * world * per_gpu * seq
    return {"metric": "tokens/sec", "value": tokens / (ms_inner / 1e3), "unit": "tokens/s", "ms_per_step": ms_inner / inner,
            "higher_is_better": True, "scaling": "weak", "gpu_launches": launches, "outer_step": outer, "final_loss": float(loss.item()),
            "e2e": {"value": k_e2e * world * per_gpu * seq / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * per_gpu * seq * 8,
                    "d2h_bytes_per_step": 16},
            "config": {"model": "Llama-1B (18L, dim 2048, 16 heads, ffn 8192, vocab 32000)", "global_batch": world * per_gpu, "seq_len": seq,
                       "parallelism": f"diloco {workers} workers x zero3-dp{per}", "micro_bs": micro, "inner_steps": inner,
                       "l2": "per-step working set far exceeds the 126 MB L2; no explicit flush"}}


def _ref_model(dim, n_layers, n_heads, n_kv_heads, multiple_of, ffn_dim_multiplier, vocab, seq):
    from zeroband.models.llama.model import ModelArgs, Transformer
    kw = dict(dim=dim, n_layers=n_layers, n_heads=n_heads, multiple_of=multiple_of, vocab_size=vocab, max_seq_len=seq, attn_fn="flex")
    if n_kv_heads:
        kw["n_kv_heads"] = n_kv_heads
    if ffn_dim_multiplier:
        kw["ffn_dim_multiplier"] = ffn_dim_multiplier
    margs = ModelArgs(**kw)
    with torch.device("cuda"):
        model = Transformer(margs)
    for p in model.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, 0.0, 0.02)
    return model, margs


def _ref_fsdp(model, n_layers, mesh):
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=None)
    for lid, blk in model.layers.items():
        fully_shard(blk, mp_policy=mp, mesh=mesh, reshard_after_forward=int(lid) < n_layers - 1)
    fully_shard(model, mp_policy=mp, mesh=mesh, reshard_after_forward=True)


def _ref_step_fn(model, opt, micro, per_gpu, sharded):
    from zeroband.loss import compute_cross_entropy_loss
    n_micro = per_gpu // micro

    def step(x, y):
        tot = 0.0
        for mb in range(n_micro):
            xs, ys = x[mb * micro:(mb + 1) * micro], y[mb * micro:(mb + 1) * micro]
            if sharded:
                model.set_requires_gradient_sync(mb == n_micro - 1)
            logits = model(tokens=xs, block_mask=None).contiguous()
            ce, _ = compute_cross_entropy_loss(logits, ys, z_weight=None, num_chunks=None, fused_linear_weight=None)
            loss = ce / n_micro
            loss.backward()
            tot = tot + loss.detach()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad()
        return tot
    return step


def run_1b_diloco_reference(args, world, rank, local):
    """The reference's Transformer under its FSDP2 recipe (train.py:144-168) inside each of two workers, its own `Diloco`
    (diloco.py:24-215) for the outer step over a gloo group between the workers."""
    why = _reference_importable()
    if why:
        return {"unavailable": why}
    if world < 2:
        return {"unavailable": "the DiLoCo configuration needs at least 2 GPUs (2 workers)"}
    try:
        from torch.distributed.device_mesh import DeviceMesh
        from zeroband.config import Compression, DilocoConfig
        from zeroband.diloco import Diloco
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"reference import failed: {type(e).__name__}: {str(e)[:160]}"}
    torch.set_float32_matmul_precision("high")
    workers = 2
    per, me, local_pg, _ = _split_workers(world, rank, workers)
    mine = [me * per + r for r in range(per)]
    # the outer exchange of the reference runs on CPU tensors over gloo, one group per shard index
    gloo_worker_pg = None
    for r in range(per):
        g = dist.new_group([w * per + r for w in range(workers)], backend="gloo")
        if r == rank % per:
            gloo_worker_pg = g
    cpu_mesh = None
    for w in range(workers):
        g = dist.new_group([w * per + r for r in range(per)], backend="gloo")
        if w == me:
            cpu_mesh = DeviceMesh.from_group(g, "cpu", torch.tensor(mine))
    cuda_mesh = DeviceMesh.from_group(local_pg, "cuda", torch.tensor(mine))
    torch.manual_seed(42)
    seq, per_gpu, micro = 2048, args.per_gpu_seqs or 8, args.ref_micro_bs or 4
    model, margs = _ref_model(2048, 18, 16, None, 8192, None, 32000, seq)
    _ref_fsdp(model, margs.n_layers, cuda_mesh)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1, betas=(0.9, 0.95))
    os.environ.setdefault("GLOBAL_UNIQUE_ID", str(me))
    os.environ.setdefault("GLOBAL_RANK", str(me))
    os.environ.setdefault("GLOBAL_WORLD_SIZE", str(workers))
    dl_no = Diloco(DilocoConfig(inner_steps=args.steps, compression=Compression.NO), model, _StaticMesh(gloo_worker_pg, cpu_mesh))
    cmodel = torch.compile(model)
    step = _ref_step_fn(cmodel, opt, micro, per_gpu, sharded=True)
    g = torch.Generator().manual_seed(1234 + rank)
    tok = torch.randint(0, 32000, (per_gpu, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    xd, yd = x.cuda(), y.cuda()
    for _ in range(max(args.warmup, 3)):
        step(xd, yd)
    _sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step(xd, yd)
    e1.record()
    _sync()
    ms_inner = _max_over_ranks(e0.elapsed_time(e1))
    k_e2e = min(args.steps, 10)
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(k_e2e):
        lf = float(step(x.cuda(non_blocking=True), y.cuda(non_blocking=True)).item())
    f1.record()
    _sync()
    ms_e2e = _max_over_ranks(f0.elapsed_time(f1))
    outer = {}
    ts = []
    for rep in range(2):
        _sync()
        t0 = time.perf_counter()
        dl_no.step(model, flag=f"no{rep}")
        torch.cuda.synchronize()
        ts.append((time.perf_counter() - t0) * 1e3)
        step(xd, yd)
    outer["no"] = {"outer_step_ms": _max_over_ranks(ts[-1]), "first_call_ms": _max_over_ranks(ts[0])}
    try:
        Diloco(DilocoConfig(inner_steps=args.steps, compression=Compression.UINT8), model, _StaticMesh(gloo_worker_pg, cpu_mesh))
        outer["uint8"] = {"note": "built"}
    except Exception as e:  # noqa: BLE001
        outer["uint8"] = {"unavailable": f"the reference's C++ ring does not build here ({type(e).__name__}: gloo headers absent)"}
    tokens = args.steps * world * per_gpu * seq
    return {"metric": "tokens/sec", "value": tokens / (ms_inner / 1e3), "unit": "tokens/s", "ms_per_step": ms_inner / args.steps,
            "higher_is_better": True, "scaling": "weak", "gpu_launches": None, "outer_step": outer, "final_loss": float(loss.item()),
            "e2e": {"value": k_e2e * world * per_gpu * seq / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * per_gpu * seq * 8,
                    "d2h_bytes_per_step": 4},
            "e2e_final_loss": lf,
            "config": {"model": "Llama-1B (18L, dim 2048, 16 heads, ffn 8192, vocab 32000)", "global_batch": world * per_gpu, "seq_len": seq,
                       "parallelism": f"diloco {workers} workers x fsdp2-dp{per}", "micro_bs": micro, "inner_steps": args.steps}}


# =====================================================================================================
# 10B shape (BASELINE configuration 4)
# =====================================================================================================
def _shm_free_gb() -> float:
    try:
        st = os.statvfs("/dev/shm")
        return st.f_bavail * st.f_frsize / 2 ** 30
    except OSError:
        return 0.0


def run_10b_ours(args, world, rank, local):
    """INTELLECT-1 shape on the GPUs of one box: activation checkpointing on, micro-batch 1, one staged checkpoint inside
    the run (time the loop is blocked, and time until the background copy is on disk) and one outer synchronisation with
    the outer state in pinned host memory."""
    from prime_b200 import native
    from prime_b200.backend import FusedBackend
    from prime_b200.checkpoint import CkptManager, TrainingProgress
    from prime_b200.config import AdamConfig, CkptConfig, Compression, DilocoConfig
    from prime_b200.diloco import Diloco
    from prime_b200.engine.fused_llama import FusedLlama
    from prime_b200.lr_scheduler import get_scheduler
    from prime_b200.models.llama import bench_configs
    from prime_b200.ops.kernels import check_status
    from prime_b200.parallel.symm import SymmComm
    dev = torch.device("cuda", local)
    margs = bench_configs["10B"]
    if args.layers:
        margs = replace(margs, n_layers=args.layers)
    comm = SymmComm() if world > 1 else None
    seq, per_gpu, micro = margs.max_seq_len, args.per_gpu_seqs or 2, 1
    eng = FusedLlama(margs, device=dev, comm=comm, ac_ckpt=True, reshard=getattr(args, "reshard", False))
    eng.init_weights(seed=0, std=0.02)
    g = torch.Generator().manual_seed(1234 + rank)
    tok = torch.randint(0, margs.vocab_size, (per_gpu, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    xd, yd = x.cuda(), y.cuda()
    for _ in range(max(args.warmup, 3)):
        eng.train_step(xd, yd, 7.5e-5, micro_bs=micro, sync_loss=False)
    _sync()
    check_status()
    native.launch_counter_reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss, _ = eng.train_step(xd, yd, 7.5e-5, micro_bs=micro, sync_loss=False)
    e1.record()
    _sync()
    launches = native.launch_counter()
    ms = _max_over_ranks(e0.elapsed_time(e1))
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        eng.train_step(x, y, 7.5e-5, micro_bs=micro, sync_loss=True)
    f1.record()
    _sync()
    ms_e2e = _max_over_ranks(f0.elapsed_time(f1))
    mem_gb = torch.cuda.max_memory_allocated() / 2 ** 30
    # ---- outer synchronisation (one worker: no exchange partner, the host-side pseudo-gradient + Nesterov + refresh) ----
    outer = {}
    mesh_pg = types.SimpleNamespace(size=lambda: 1, rank=lambda: 0, barrier=lambda: types.SimpleNamespace(wait=lambda: None),
                                    all_reduce_tensor=lambda t, c, average=False: None)
    dl = Diloco(DilocoConfig(inner_steps=100, compression=Compression.NO), eng, _StaticMesh(mesh_pg))
    ts = []
    for rep in range(2):          # the first call allocates the device copies and the pinned momentum mirror
        eng.train_step(xd, yd, 7.5e-5, micro_bs=micro, sync_loss=False)
        _sync()
        t0 = time.perf_counter()
        dl.step(eng, flag=f"o{rep}")
        torch.cuda.synchronize()
        ts.append((time.perf_counter() - t0) * 1e3)
    outer["outer_step_ms"] = _max_over_ranks(ts[-1])
    outer["first_call_ms"] = _max_over_ranks(ts[0])
    t0 = time.perf_counter()
    dl.wait_host_state()
    outer["host_refresh_on_demand_ms"] = _max_over_ranks((time.perf_counter() - t0) * 1e3)
    outer["includes"] = ("one worker, host-side exchange path: pseudo-gradient on the device, device-to-host copy, (no partner: "
                         "identity all-reduce), copy back, Nesterov on the device copies of the outer state, inner refresh")
    outer["shard_numel"] = eng.master.numel()
    # ---- one asynchronous checkpoint through the staging directory ----
    ckpt = {}
    need_gb = eng.master.numel() * 4 * 4 * world / 2 ** 30 * 1.15       # master + two moments + outer momentum, all ranks
    free_gb = _shm_free_gb()
    ckpt_dir = args.ckpt_dir or "/tmp/prime_b200_bench_ckpt"
    import shutil
    os.makedirs(ckpt_dir, exist_ok=True)
    disk_gb = shutil.disk_usage(ckpt_dir).free / 2 ** 30
    if getattr(args, "skip_ckpt", False):
        ckpt["skipped"] = "--skip-ckpt"
    elif free_gb < need_gb:
        ckpt["skipped"] = f"/dev/shm has {free_gb:.0f} GB free, the staged checkpoint needs about {need_gb:.0f} GB"
    elif disk_gb < need_gb:
        ckpt["skipped"] = f"{ckpt_dir} has {disk_gb:.0f} GB free, the persisted checkpoint needs about {need_gb:.0f} GB"
    else:
        opt_cfg = AdamConfig()
        backend = FusedBackend(eng, opt_cfg, lambda o: get_scheduler("cosine", o, 10, 100, 1000), mesh=None if world == 1 else _local_mesh(world))
        prog = TrainingProgress(0, 0, 100)
        mgr = CkptManager(CkptConfig(path=ckpt_dir, interval=100), backend, backend.lr_scheduler, _NoData(), prog, None,
                          dl.param_list_cpu, dl.outer_optimizer, diloco=dl)
        _sync()
        t0 = time.perf_counter()
        mgr.save()
        ckpt["blocking_ms"] = _max_over_ranks((time.perf_counter() - t0) * 1e3)
        t1 = time.perf_counter()
        eng.train_step(xd, yd, 7.5e-5, micro_bs=micro, sync_loss=True)          # training goes on while the copy runs
        ckpt["step_during_copy_ms"] = _max_over_ranks((time.perf_counter() - t1) * 1e3)
        mgr.wait_for_blocking_job()
        ckpt["background_copy_s"] = _max_over_ranks(time.perf_counter() - t0)
        ckpt["bytes_gb"] = need_gb / 1.15
        mgr.close()
        if rank == 0:
            import shutil
            shutil.rmtree(ckpt_dir, ignore_errors=True)
    check_status()
    tokens = args.steps * world * per_gpu * seq
    n_params = sum(p.numel for p in eng.layout.params)
    fpt = 6 * (n_params - margs.vocab_size * margs.dim) + 6 * margs.n_layers * margs.n_heads * margs.head_dim * seq
    _, peak_tf = _peaks()
    return {"metric": "tokens/sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "gpu_launches": launches, "final_loss": float(loss.item()), "outer_step": outer, "checkpoint": ckpt,
            "max_mem_gb": mem_gb, "model_tflops_per_gpu": fpt * tokens / world / (ms / 1e3) / 1e12,
            "mfu_of_measured_cublas_peak": fpt * tokens / world / (ms / 1e3) / (peak_tf * 1e12),
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * per_gpu * seq * 8, "d2h_bytes_per_step": 16},
            "vs_published_8xH100": tokens / (ms / 1e3) / 46.0e3 if (world == 8 and not args.layers) else None,
            "config": {"model": f"INTELLECT-1 10B shape ({margs.n_layers}L, dim 4096, 32 heads / 8 KV, ffn 14336, vocab 128256)",
                       "global_batch": world * per_gpu, "seq_len": seq, "parallelism": f"zero3-dp{world}" + ("-reshard" if getattr(args, "reshard", False) and world > 1 else ""),
                       "micro_bs": micro, "activation_checkpointing": True, "l2": "per-step working set far exceeds the 126 MB L2; no explicit flush"}}


class _NoData:
    def state_dict(self):
        return {}

    def load_state_dict(self, sd):
        pass


def _local_mesh(world):
    from torch.distributed.device_mesh import init_device_mesh
    return init_device_mesh("cuda", (world,))


def run_10b_reference(args, world, rank, local):
    """The reference's Transformer at the 10B shape under its FSDP2 recipe with its activation checkpointing, micro-batch 1."""
    why = _reference_importable()
    if why:
        return {"unavailable": why}
    try:
        from torch.distributed.device_mesh import init_device_mesh
        from zeroband.utils.activation_ckpt import apply_ac_ckpt
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"reference import failed: {type(e).__name__}: {str(e)[:160]}"}
    if world < 8 and not args.layers:
        return {"unavailable": "the 10B shape with AdamW state needs the 8 GPUs of a box (12 bytes per parameter sharded)"}
    torch.set_float32_matmul_precision("high")
    torch.manual_seed(42)
    seq, per_gpu, micro = 8192, args.per_gpu_seqs or 2, 1
    n_layers = args.layers or 42
    model, margs = _ref_model(4096, n_layers, 32, 8, 1024, 1.3, 128256, seq)
    apply_ac_ckpt(model, 1)
    if world > 1:
        _ref_fsdp(model, margs.n_layers, init_device_mesh("cuda", (world,)))
    opt = torch.optim.AdamW(model.parameters(), lr=7.5e-5, weight_decay=0.1, betas=(0.9, 0.95))
    cmodel = torch.compile(model)
    step = _ref_step_fn(cmodel, opt, micro, per_gpu, sharded=world > 1)
    g = torch.Generator().manual_seed(1234 + rank)
    tok = torch.randint(0, 128256, (per_gpu, seq + 1), generator=g)
    x, y = tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory()
    xd, yd = x.cuda(), y.cuda()
    ctx = torch.autocast("cuda", dtype=torch.bfloat16) if world == 1 else None
    if ctx is not None:
        ctx.__enter__()
    for _ in range(max(args.warmup, 3)):
        step(xd, yd)
    _sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step(xd, yd)
    e1.record()
    _sync()
    ms = _max_over_ranks(e0.elapsed_time(e1))
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        lf = float(step(x.cuda(non_blocking=True), y.cuda(non_blocking=True)).item())
    f1.record()
    _sync()
    ms_e2e = _max_over_ranks(f0.elapsed_time(f1))
    tokens = args.steps * world * per_gpu * seq
    return {"metric": "tokens/sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "gpu_launches": None, "final_loss": float(loss.item()), "e2e_final_loss": lf,
            "max_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * per_gpu * seq * 8, "d2h_bytes_per_step": 4},
            "config": {"model": f"INTELLECT-1 10B shape ({n_layers}L, dim 4096, 32 heads / 8 KV, ffn 14336, vocab 128256)",
                       "global_batch": world * per_gpu, "seq_len": seq, "parallelism": f"fsdp2-dp{world}", "micro_bs": micro,
                       "activation_checkpointing": True}}
