"""Pseudo-gradient all-reduce across DiLoCo workers: dispatch, transports and a Python oracle.

``all_reduce(compression, tensor, op, group)`` keeps the reference call shape
(src/zeroband/collectives.py:31-42). ``group`` is anything with ``size()`` / ``rank()``:
  * a :class:`TcpRing` — this package's C++ socket ring (csrc/host/tcp_ring.cpp), the cross-node
    transport for both fp32 and uint8 payloads;
  * a ``torch.distributed`` process group — fp32 goes through its own all-reduce, uint8 through
    ``ring_allreduce_py`` (isend/irecv), which is the readable oracle of the ring schedule
    (reference keeps its Python ring for the same purpose, collectives.py:53-192);
  * a group of size 1 (e.g. the FakeProcessGroup placeholder) — no-op.
"""
from __future__ import annotations

import ctypes as C
import socket
from enum import Enum

import torch
import torch.distributed as dist

from . import native
from .compression import host as host_quant
from .compression import uniform_8bit_quantize
from .config import Compression


class AllReduceError(RuntimeError):
    pass


class TcpRing:
    """A ring of W processes connected by this package's C++ TCP transport.

    Rendezvous goes through any key-value store with ``set``/``get`` (a ``TCPStore`` or
    ``PrefixStore``): each rank publishes ``ring_addr_{rank} = host:port`` and connects to its
    successor. ``close()`` (or garbage collection) tears the sockets down; after an I/O error the
    ring is poisoned and must be rebuilt, which is what the elastic mesh does on re-init."""

    def __init__(self, store, rank: int, world: int, host: str | None = None, nconn: int = 4, timeout_s: float = 30.0,
                 threads: int = 0):
        self._lib = _ring_lib()
        self._rank, self._world, self.threads = rank, world, threads
        self._h = self._lib.pbh_ring_create(rank, world, nconn, 0, timeout_s)
        if not self._h:
            raise AllReduceError("could not create ring endpoint")
        if world > 1:
            host = host or _my_ip()
            store.set(f"ring_addr_{rank}", f"{host}:{self._lib.pbh_ring_port(self._h)}")
            nxt = store.get(f"ring_addr_{(rank + 1) % world}").decode()
            nh, np_ = nxt.rsplit(":", 1)
            rc = self._lib.pbh_ring_connect(self._h, nh.encode(), int(np_))
            if rc != 0:
                self.close()
                raise AllReduceError(f"ring connect failed with code {rc}")

    def size(self) -> int:
        return self._world

    def rank(self) -> int:
        return self._rank

    def all_reduce(self, tensor: torch.Tensor, compression: Compression = Compression.NO, average: bool = False) -> None:
        assert tensor.dtype == torch.float32 and tensor.is_contiguous() and not tensor.is_cuda
        rc = self._lib.pbh_ring_allreduce(self._h, tensor.data_ptr(), tensor.numel(), int(compression == Compression.UINT8),
                                          int(average), self.threads)
        if rc != 0:
            raise AllReduceError(f"tcp ring all-reduce failed with code {rc}")

    def probe_seconds(self, nbytes: int = 8 << 20) -> float:
        return float(self._lib.pbh_ring_probe(self._h, nbytes))

    def inject_fault(self, after_bytes: int) -> None:
        """Test hook: this rank's outgoing link fails after ``after_bytes`` more bytes."""
        self._lib.pbh_ring_inject_fault(self._h, after_bytes)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.pbh_ring_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_ring_lib_cache = None


def _ring_lib():
    global _ring_lib_cache
    if _ring_lib_cache is None:
        lib = native.host()
        vp, i32, i64, f64 = C.c_void_p, C.c_int, C.c_longlong, C.c_double
        lib.pbh_ring_create.argtypes = [i32, i32, i32, i32, f64]
        lib.pbh_ring_create.restype = vp
        lib.pbh_ring_port.argtypes = [vp]
        lib.pbh_ring_port.restype = i32
        lib.pbh_ring_connect.argtypes = [vp, C.c_char_p, i32]
        lib.pbh_ring_connect.restype = i32
        lib.pbh_ring_destroy.argtypes = [vp]
        lib.pbh_ring_destroy.restype = None
        lib.pbh_ring_inject_fault.argtypes = [vp, i32]
        lib.pbh_ring_inject_fault.restype = None
        lib.pbh_ring_allreduce.argtypes = [vp, vp, i64, i32, i32, i32]
        lib.pbh_ring_allreduce.restype = i32
        lib.pbh_ring_probe.argtypes = [vp, i64]
        lib.pbh_ring_probe.restype = f64
        _ring_lib_cache = lib
    return _ring_lib_cache


def _my_ip() -> str:
    import os
    if os.environ.get("GLOBAL_ADDR", "") in ("localhost", "127.0.0.1"):
        return "127.0.0.1"
    try:
        s = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        s.connect(("10.255.255.255", 1))
        ip = s.getsockname()[0]
        s.close()
        return ip
    except Exception:
        return "127.0.0.1"


def gloo_all_reduce(tensor: torch.Tensor, op: dist.ReduceOp = dist.ReduceOp.SUM, group: dist.ProcessGroup | None = None):
    """fp32 all-reduce through a torch process group; AVG is SUM followed by a division."""
    if op not in (dist.ReduceOp.SUM, dist.ReduceOp.AVG):
        raise ValueError(f"Unsupported reduce operation {op}. Only SUM and AVG are supported.")
    group = group or dist.distributed_c10d._get_default_group()
    if op == dist.ReduceOp.AVG:
        tensor.div_(group.size())
    return dist.all_reduce(tensor, dist.ReduceOp.SUM, group=group)


def ring_allreduce_py(tensor: torch.Tensor, op: dist.ReduceOp = dist.ReduceOp.SUM, group: dist.ProcessGroup | None = None,
                      quantization_func=uniform_8bit_quantize) -> None:
    """uint8 ring all-reduce written with torch point-to-point ops: same schedule as the C++ ring
    (W chunks; W-1 quantised reduce-scatter hops with fp32 accumulation; the owner quantises its
    reduced chunk once and the all-gather forwards those bytes verbatim)."""
    if op not in (dist.ReduceOp.SUM, dist.ReduceOp.AVG):
        raise ValueError(f"Unsupported reduce operation {op}. Only SUM and AVG are supported.")
    group = group or dist.distributed_c10d._get_default_group()
    W, me = group.size(), group.rank()
    if W == 1:
        return
    flat = tensor.view(-1)
    n = flat.numel()
    per = -(-n // W)
    chunks = [flat[min(n, c * per): min(n, (c + 1) * per)] for c in range(W)]
    nxt, prv = dist.get_global_rank(group, (me + 1) % W), dist.get_global_rank(group, (me - 1) % W)

    def exchange(send_q, send_lut, recv_numel):
        rq = torch.empty(recv_numel, dtype=torch.uint8)
        rl = torch.empty(256, dtype=torch.float32)
        works = [dist.isend(send_lut, nxt, group=group), dist.irecv(rl, prv, group=group),
                 dist.isend(send_q, nxt, group=group), dist.irecv(rq, prv, group=group)]
        for w in works:
            w.wait()
        return rq, rl

    for step in range(W - 1):
        sc, rc = (me - step) % W, (me - step - 1) % W
        q, lut = quantization_func(chunks[sc])
        rq, rl = exchange(q.view(-1), lut, chunks[rc].numel())
        chunks[rc].add_(rl[rq.long()])
    own = (me + 1) % W
    if op == dist.ReduceOp.AVG:
        chunks[own].div_(W)
    q, lut = quantization_func(chunks[own])
    chunks[own].copy_(lut[q.view(-1).long()])
    held = {own: (q.view(-1), lut)}
    for step in range(W - 1):
        sc, rc = (own - step) % W, (own - step - 1) % W
        rq, rl = exchange(held[sc][0], held[sc][1], chunks[rc].numel())
        held[rc] = (rq, rl)
        chunks[rc].copy_(rl[rq.long()])


def all_reduce(compression: Compression, tensor: torch.Tensor, op: dist.ReduceOp = dist.ReduceOp.SUM, group=None) -> None:
    """In-place all-reduce of a flat fp32 CPU tensor across the worker group."""
    if group is not None and group.size() == 1:
        return
    if isinstance(group, TcpRing):
        group.all_reduce(tensor, compression, average=(op == dist.ReduceOp.AVG))
        return
    if hasattr(group, "all_reduce_tensor"):      # e.g. the NVLink worker group (parallel/diloco_comm.py)
        group.all_reduce_tensor(tensor, compression, average=(op == dist.ReduceOp.AVG))
        return
    if compression == Compression.UINT8:
        ring_allreduce_py(tensor, op, group)
    else:
        gloo_all_reduce(tensor, op, group)
