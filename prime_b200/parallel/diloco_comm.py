"""NVLink worker group: the DiLoCo outer step (and a generic uint8 all-reduce) executed on the GPUs
over symmetric memory, for workers that live in the same NVSwitch domain.

``NvlinkWorkerGroup`` plays the role of the cross-worker process group: ``size() / rank() /
barrier()``, ``all_reduce_tensor`` (used by :func:`prime_b200.collectives.all_reduce`) and
``fused_outer_step`` (picked up by :class:`prime_b200.diloco.Diloco`), all backed by the kernels in
csrc/diloco_comm.cu. The outer parameters and momentum stay in pinned host memory between outer
steps and are staged to HBM only for the duration of the fused step
(reference: src/zeroband/diloco.py:77-144, 203-215 does the whole outer step on the CPU over gloo).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import native
from ..config import Compression
from ..native import check, ptr, stream_ptr
from .symm import SymmComm

native.register_cuda_sigs({
    "pb_dl_chunk": [], "pb_dl_blocks_per_chunk": [],
    "pb_dl_stage_a": [native.vp, native.vp, native.i64, native.i32, native.i32, native.vp, native.vp, native.vp, native.vp, native.vp,
                      native.vp],
    "pb_dl_stage_b": [native.vp, native.vp, native.vp, native.vp, native.i32, native.i32, native.i64, native.vp, native.vp, native.vp,
                      native.vp, native.vp],
    "pb_dl_stage_c": [native.vp, native.vp, native.vp, native.vp, native.i32, native.i32, native.i64, native.vp, native.vp, native.vp,
                      native.f32, native.f32, native.vp, native.vp],
})


class _Work:
    def wait(self, *a, **k):
        torch.cuda.current_stream().synchronize()
        return True


class NvlinkWorkerGroup:
    def __init__(self, comm: SymmComm, max_numel: int):
        self.comm = comm
        self.device = comm.device
        lib = native.cuda()
        self.chunk = lib.pb_dl_chunk()
        self.bpc = lib.pb_dl_blocks_per_chunk()
        self.capacity = 0
        self._ensure(max_numel)

    def _ensure(self, n: int) -> None:
        """(Re)allocate the symmetric exchange buffers for up to ``n`` elements (collective)."""
        if n <= self.capacity:
            return
        W = self.comm.world
        chunks = -(-n // self.chunk)
        n_pad = chunks * self.chunk
        self.q = self.comm.alloc(n_pad, torch.uint8)
        self.lut = self.comm.alloc(chunks * 256, torch.float32)
        self.q2 = self.comm.alloc(n_pad, torch.uint8)
        self.lut2 = self.comm.alloc(chunks * 256, torch.float32)
        self._pq, self._plut = self.comm.peer_ptrs(self.q), self.comm.peer_ptrs(self.lut)
        self._pq2, self._plut2 = self.comm.peer_ptrs(self.q2), self.comm.peer_ptrs(self.lut2)
        dev = self.device
        self.partial = torch.empty(chunks * self.bpc, dtype=torch.float32, device=dev)
        self.bin_sum = torch.empty(chunks * self.bpc * 256, dtype=torch.int64, device=dev)
        self.bin_cnt = torch.empty(chunks * self.bpc * 256, dtype=torch.int32, device=dev)
        self.reduced = torch.empty((-(-chunks // W)) * self.chunk, dtype=torch.float32, device=dev)
        self.capacity = n_pad

    # ---- process-group-like surface ----
    def size(self) -> int:
        return self.comm.world

    def rank(self) -> int:
        return self.comm.rank

    def barrier(self):
        self.comm.barrier(slot=2)
        return _Work()

    # ---- kernels ----
    def _exchange(self, a: torch.Tensor, b: torch.Tensor | None, n: int, fake: bool, inv_world: bool):
        """Stages A and B (+ the barriers around them) for value (a - b) / W, or a / W, or a."""
        lib, W, r = native.cuda(), self.comm.world, self.comm.rank
        assert n <= self.capacity
        check(lib.pb_dl_stage_a(ptr(a), ptr(b), n, W if inv_world else 1, int(fake), ptr(self.q), ptr(self.lut), ptr(self.partial),
                                ptr(self.bin_sum), ptr(self.bin_cnt), stream_ptr()), "pb_dl_stage_a")
        self.comm.barrier(slot=3)
        check(lib.pb_dl_stage_b(self._pq, self._plut, self._pq2, self._plut2, W, r, n, ptr(self.reduced), ptr(self.partial),
                                ptr(self.bin_sum), ptr(self.bin_cnt), stream_ptr()), "pb_dl_stage_b")
        self.comm.barrier(slot=3)

    def all_reduce_tensor(self, tensor: torch.Tensor, compression: Compression = Compression.UINT8, average: bool = False) -> None:
        """In-place all-reduce of a flat fp32 tensor (host or device). ``uint8``: quantised exchange
        with fp32 accumulation by this package's kernels; ``no``: exact fp32 through the library
        all-reduce of the group (plain collective, nothing fused with it)."""
        x = tensor if tensor.is_cuda else tensor.to(self.device, non_blocking=True)
        if compression != Compression.UINT8:
            dist.all_reduce(x, group=self.comm.group)
            if average:
                x.div_(self.comm.world)
        else:
            n = x.numel()
            self._ensure_same(n)
            self._exchange(x, None, n, fake=False, inv_world=average)
            lib = native.cuda()
            check(lib.pb_dl_stage_c(self._pq, self._plut, self._pq2, self._plut2, self.comm.world, self.comm.rank, n, None, None, None,
                                    0.0, 0.0, ptr(x), stream_ptr()), "pb_dl_stage_c")
            self.comm.barrier(slot=3)
            # a peer wait that gave up must fail this reduction (the caller's retry path handles the exception)
            from ..ops.kernels import check_status
            check_status(self.device)
        if not tensor.is_cuda:
            tensor.copy_(x)
        return None

    def _ensure_same(self, n: int) -> None:
        if n > self.capacity:
            self._ensure(n)

    @torch.no_grad()
    def fused_outer_step(self, model, outer_host: torch.Tensor, mom_host: torch.Tensor, lr: float, momentum: float, fake: bool,
                         compression: Compression, first_step: bool = False) -> None:
        """One DiLoCo outer step for this rank's shard. ``model.master`` (fp32 device shard) is the
        inner state and receives the new outer parameters; ``outer_host`` / ``mom_host`` are the
        pinned host copies of outer parameters and momentum (updated in place)."""
        inner = model.master
        n = inner.numel()
        self._ensure_same(n)
        outer = getattr(self, "_outer_dev", None)
        if outer is None or outer.numel() != n:
            self._outer_dev = outer = torch.empty(n, dtype=torch.float32, device=self.device)
            self._mom_dev = torch.empty(n, dtype=torch.float32, device=self.device)
        mom = self._mom_dev
        outer.copy_(outer_host, non_blocking=True)
        mom.copy_(mom_host, non_blocking=True)
        lib, W, r = native.cuda(), self.comm.world, self.comm.rank
        if compression == Compression.UINT8:
            self._exchange(outer, inner, n, fake=fake, inv_world=True)
            check(lib.pb_dl_stage_c(self._pq, self._plut, self._pq2, self._plut2, W, r, n, ptr(outer), ptr(inner), ptr(mom), lr, momentum,
                                    None, stream_ptr()), "pb_dl_stage_c")
            self.comm.barrier(slot=3)
        else:
            g = torch.zeros_like(outer) if fake else (outer - inner)
            dist.all_reduce(g, group=self.comm.group)
            g.div_(W)
            mom.mul_(momentum).add_(g)
            outer.sub_(g.add_(mom, alpha=momentum), alpha=lr)
            inner.copy_(outer)
        outer_host.copy_(outer, non_blocking=True)
        mom_host.copy_(mom, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        from ..ops.kernels import check_status
        check_status(self.device)
