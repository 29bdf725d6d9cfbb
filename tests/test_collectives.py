"""Ring all-reduce: C++ TCP ring vs Python ring vs exact all-reduce on CPU ranks (gloo)."""
import multiprocessing as mp
import os
import traceback

import pytest
import torch
import torch.distributed as dist

from prime_b200.collectives import AllReduceError, TcpRing, all_reduce, ring_allreduce_py
from prime_b200.config import Compression


def _worker(rank, world, port, fn, q, args):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        store = dist.distributed_c10d._get_default_store()
        q.put((rank, fn(rank, world, store, *args)))
    except Exception:
        q.put((rank, "ERR " + traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _spawn(world, fn, port, *args):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, world, port, fn, q, args)) for r in range(world)]
    for p in ps:
        p.start()
    out = dict(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(timeout=30)
    for r, v in out.items():
        assert not (isinstance(v, str) and v.startswith("ERR")), v
    return out


def _ring_case(rank, world, store, n, compression):
    torch.manual_seed(rank)
    x = torch.randn(n) * 10
    exact = x.clone()
    dist.all_reduce(exact)
    ring = TcpRing(dist.PrefixStore("ring0", store), rank, world, host="127.0.0.1", nconn=2)
    a = x.clone()
    all_reduce(compression, a, dist.ReduceOp.SUM, ring)
    b = x.clone()
    if compression == Compression.UINT8:
        ring_allreduce_py(b, dist.ReduceOp.SUM)
    else:
        dist.all_reduce(b)
    gathered = [torch.empty_like(a) for _ in range(world)]
    dist.all_gather(gathered, a)
    identical = all(torch.equal(g, gathered[0]) for g in gathered)
    ring.close()
    return ((a - exact).norm().item(), (b - exact).norm().item(), exact.norm().item(), identical)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("n", [1_000_000, 1_000_003, 5])
def test_uint8_ring_error_matches_python_ring(world, n, free_port):
    out = _spawn(world, _ring_case, free_port, n, Compression.UINT8)
    for ea, eb, norm, identical in out.values():
        assert identical, "all ranks must end with identical bits"
        assert abs(ea - eb) / (n ** 0.5) < 0.5          # the reference's acceptance inequality
        if n > 1000:
            assert ea / norm < 0.05


@pytest.mark.parametrize("world", [2, 3])
def test_fp32_ring_is_exact(world, free_port):
    out = _spawn(world, _ring_case, free_port, 300_001, Compression.NO)
    for ea, _, norm, identical in out.values():
        assert identical and ea / norm < 1e-6


def _fault_case(rank, world, store):
    ring = TcpRing(dist.PrefixStore("ringf", store), rank, world, host="127.0.0.1", nconn=1, timeout_s=3.0)
    x = torch.ones(4_000_000)
    if rank == 0:
        ring.inject_fault(100_000)
    try:
        ring.all_reduce(x, Compression.UINT8)
        ok = True
    except AllReduceError:
        ok = False
    ring.close()
    # a fresh ring works again
    ring2 = TcpRing(dist.PrefixStore("ringf2", store), rank, world, host="127.0.0.1", nconn=1, timeout_s=10.0)
    y = torch.full((1000,), float(rank + 1))
    ring2.all_reduce(y, Compression.NO)
    ring2.close()
    return ok, y[0].item()


def test_link_failure_surfaces_as_error_then_rebuild(free_port):
    out = _spawn(2, _fault_case, free_port)
    assert any(not ok for ok, _ in out.values())
    assert all(abs(v - 3.0) < 1e-6 for _, v in out.values())
