"""NVLink worker group: the DiLoCo outer step (and a generic uint8 all-reduce) executed on the GPUs
over symmetric memory, for workers that live in the same NVSwitch domain.

``NvlinkWorkerGroup`` plays the role of the cross-worker process group: ``size() / rank() /
barrier()``, ``all_reduce_tensor`` (used by :func:`prime_b200.collectives.all_reduce`) and
``fused_outer_step`` (picked up by :class:`prime_b200.diloco.Diloco`), all backed by the kernels in
csrc/diloco_comm.cu. The fp32 outer parameters and momentum either stay resident in HBM between outer
steps, with the pinned host copies written on demand (``resident=True``, the default of
``diloco.outer_state_resident``), or live in pinned host memory and are staged to HBM for the duration of
the fused step (reference: src/zeroband/diloco.py:77-144, 203-215 does the whole outer step on the CPU over gloo).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import native
from ..config import Compression
from ..native import check, ptr, stream_ptr
from ..ops.kernels import check_status, status_word
from .symm import SymmComm

native.register_cuda_sigs({
    "pb_dl_chunk": [],
    "pb_dl_allreduce": [native.vp] * 5 + [native.i32, native.i32, C.c_uint, native.i32, native.i32, native.i32, native.i64, native.vp, native.vp,
                                         native.f32, native.i32, native.vp, native.vp, native.vp, native.f32, native.f32, native.vp, native.vp,
                                         native.vp, native.i64, native.vp],
    "pb_get_peer_wait_budget_ns": [],
})

DL_FLAG_SLOT = 8        # three consecutive slots of the communicator's flag pads: stage A / B / C done


class _Work:
    def wait(self, *a, **k):
        torch.cuda.current_stream().synchronize()
        return True


class NvlinkWorkerGroup:
    """See module docstring. Membership of a call is a subset of the communicator's ranks (``set_participants``); it only
    changes between calls, after a host-side rendezvous of all ranks of the communicator. Every rank of the communicator
    calls ``all_reduce_tensor`` / ``fused_outer_step`` for every exchange, members or not (a non-member returns at once);
    that keeps the epoch numbers of the flag protocol in step."""

    def __init__(self, comm: SymmComm, max_numel: int):
        self.comm = comm
        self.device = comm.device
        lib = native.cuda()
        lib.pb_get_peer_wait_budget_ns.restype = C.c_longlong
        self.chunk = lib.pb_dl_chunk()
        self.capacity = 0
        self._mask = (1 << comm.world) - 1
        self._epoch = 0
        self._prev_epoch = 0
        self._counters = torch.zeros(4, dtype=torch.int32, device=self.device)
        import threading
        self._host_lock = threading.Lock()     # the host copies of the outer state: refreshed on demand, possibly from another thread
        self._ensure(max_numel)

    def _ensure(self, n: int) -> None:
        """(Re)allocate the symmetric exchange buffers for up to ``n`` elements (collective)."""
        if n <= self.capacity:
            return
        chunks = -(-n // self.chunk)
        n_pad = chunks * self.chunk
        self.q = self.comm.alloc(n_pad, torch.uint8)
        self.lut = self.comm.alloc(chunks * 256, torch.float32)
        self.q2 = self.comm.alloc(n_pad, torch.uint8)
        self.lut2 = self.comm.alloc(chunks * 256, torch.float32)
        self._pq, self._plut = self.comm.peer_ptrs(self.q), self.comm.peer_ptrs(self.lut)
        self._pq2, self._plut2 = self.comm.peer_ptrs(self.q2), self.comm.peer_ptrs(self.lut2)
        self.capacity = n_pad
        self._prev_epoch = 0          # fresh buffers after a collective allocation: nothing of an earlier call is being read

    # ---- membership ----
    def set_participants(self, ranks) -> None:
        """Active ranks of the following calls. Collective over the communicator (host rendezvous, so no kernel of an
        earlier call is still running anywhere when the membership changes)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(self.comm.group)
        mask = 0
        for r in ranks:
            assert 0 <= r < self.comm.world
            mask |= 1 << r
        assert mask, "at least one participant"
        self._mask = mask
        self._prev_epoch = 0

    def participants(self) -> list[int]:
        return [r for r in range(self.comm.world) if (self._mask >> r) & 1]

    # ---- process-group-like surface ----
    def size(self) -> int:
        return bin(self._mask).count("1")

    def rank(self) -> int:
        return self.comm.rank

    def barrier(self):
        self.comm.barrier(slot=2)
        return _Work()

    # ---- kernels ----
    def _run(self, n: int, a, b, scale: float, fake: bool, outer=None, inner=None, mom=None, lr: float = 0.0, mu: float = 0.0, g_out=None):
        """One exchange (stage A, B, C) for value (a - b) * scale, or a * scale."""
        lib, W, r = native.cuda(), self.comm.world, self.comm.rank
        self._epoch += 1
        epoch, prev = self._epoch, self._prev_epoch
        self._prev_epoch = epoch
        if not (self._mask >> r) & 1:
            return False
        assert n <= self.capacity
        check(lib.pb_dl_allreduce(self._pq, self._plut, self._pq2, self._plut2, self.comm._flag_ptrs, W, r, self._mask, epoch, prev,
                                  DL_FLAG_SLOT, n, ptr(a), ptr(b), scale, int(fake), ptr(outer), ptr(inner), ptr(mom), lr, mu, ptr(g_out),
                                  ptr(self._counters), ptr(status_word(self.device)), lib.pb_get_peer_wait_budget_ns(), stream_ptr()),
              "pb_dl_allreduce")
        return True

    def all_reduce_tensor(self, tensor: torch.Tensor, compression: Compression = Compression.UINT8, average: bool = False,
                          fake: bool = False) -> None:
        """In-place all-reduce of a flat fp32 tensor (host or device) over the active ranks. ``uint8``: quantised exchange
        with fp32 accumulation by this package's kernels (``fake``: this rank contributes zeros but receives the result);
        ``no``: exact fp32 through the library all-reduce of the group (plain collective, nothing fused with it)."""
        x = tensor if tensor.is_cuda else tensor.to(self.device, non_blocking=True)
        if compression != Compression.UINT8:
            assert self._mask == (1 << self.comm.world) - 1, "the library all-reduce runs over the whole communicator"
            if fake:
                x.zero_()
            dist.all_reduce(x, group=self.comm.group)
            if average:
                x.div_(self.comm.world)
        else:
            n = x.numel()
            self._ensure_same(n)
            ran = self._run(n, x, None, 1.0 / self.size() if average else 1.0, fake, g_out=x)
            if ran and not tensor.is_cuda:
                # host tensors (the DiLoCo bucket path): the copy back synchronises anyway, so a peer wait that gave up
                # fails this reduction here (the caller's retry path handles the exception). For device tensors the caller
                # checks the status word when it synchronises.
                tensor.copy_(x)
                check_status(self.device)
                return None
        if not tensor.is_cuda:
            tensor.copy_(x)
        return None

    def _ensure_same(self, n: int) -> None:
        if n > self.capacity:
            self._ensure(n)

    @torch.no_grad()
    def fused_outer_step(self, model, outer_host: torch.Tensor, mom_host: torch.Tensor, lr: float, momentum: float, fake: bool,
                         compression: Compression, first_step: bool = False, resident: bool = False,
                         host_changed: bool = True) -> None:
        """One DiLoCo outer step for this rank's shard. ``model.master`` (fp32 device shard) is the
        inner state and receives the new outer parameters; ``outer_host`` / ``mom_host`` are the
        pinned host copies of outer parameters and momentum.

        ``resident=False``: both are staged to the device, updated and copied back before this returns.
        ``resident=True``: the device copies are kept from one outer step to the next; they are re-read from the
        host only when ``host_changed`` says the host copies were written since (checkpoint load, live recovery), and
        they are copied back only on demand: call :meth:`wait_host_copies` before reading ``outer_host`` / ``mom_host``."""
        # the lock keeps a reader's on-demand refresh of the host copies (possibly on another thread) out of the step: it
        # either finishes before the device copies are rewritten or starts after the step, and then copies the new state
        with self._host_lock:
            self._refresh_args = None
            inner = model.master
            n = inner.numel()
            self._ensure_same(n)
            outer = getattr(self, "_outer_dev", None)
            fresh = outer is None or outer.numel() != n
            if fresh:
                self._outer_dev = outer = torch.empty(n, dtype=torch.float32, device=self.device)
                self._mom_dev = torch.empty(n, dtype=torch.float32, device=self.device)
            mom = self._mom_dev
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
            staged_in = fresh or host_changed or not resident
            if staged_in:
                outer.copy_(outer_host, non_blocking=True)
                mom.copy_(mom_host, non_blocking=True)
            ev[1].record()
            if resident:
                # from here on the device copies are the truth: if the exchange below fails before it changes them, the
                # caller's fallback can still bring the host copies up to date (wait_host_copies)
                self._refresh_args = (outer, mom, outer_host, mom_host, ev[1])
            if compression == Compression.UINT8:
                self._run(n, outer, inner, 1.0 / self.size(), fake, outer=outer, inner=inner, mom=mom, lr=lr, mu=momentum)
            else:
                W = self.comm.world
                g = torch.zeros_like(outer) if fake else (outer - inner)
                dist.all_reduce(g, group=self.comm.group)
                g.div_(W)
                mom.mul_(momentum).add_(g)
                outer.sub_(g.add_(mom, alpha=momentum), alpha=lr)
                inner.copy_(outer)
            ev[2].record()
            if resident:
                # no copy back here: wait_host_copies() makes it when somebody is about to read the host copies
                self._refresh_args = (outer, mom, outer_host, mom_host, ev[2])
                ev[2].synchronize()
            else:
                outer_host.copy_(outer, non_blocking=True)
                mom_host.copy_(mom, non_blocking=True)
                ev[3].record()
                torch.cuda.current_stream().synchronize()
            # device-timed phases of this outer step: staging in, exchange + Nesterov + inner refresh, staging out
            self.last_timing_ms = {"h2d": ev[0].elapsed_time(ev[1]) if staged_in else 0.0, "exchange_update": ev[1].elapsed_time(ev[2]),
                                   "d2h": 0.0 if resident else ev[2].elapsed_time(ev[3]), "resident": bool(resident)}
            # a peer wait that gave up raises here. The update kernel skips its work in that case, so the device copies
            # still hold the state from before this step, and _refresh_args lets the caller's fallback path bring the
            # host copies up to date from them.
            check_status(self.device)

    def wait_host_copies(self) -> None:
        """Resident mode: bring the pinned host copies of the outer state up to date with the device copies, if an outer
        step has run since they were last written. Called by whoever is about to read them (checkpoint save, live
        recovery, the hash log); an outer step itself never copies back, so neither it nor the inner steps that follow
        share a copy engine with gigabytes of transfer."""
        with self._host_lock:
            args = getattr(self, "_refresh_args", None)
            if args is None:
                return
            self._refresh_args = None
            outer, mom, outer_host, mom_host, after = args
            prev = torch.cuda.current_device()
            torch.cuda.set_device(self.device)          # the caller may be a checkpoint or recovery thread
            try:
                if getattr(self, "_d2h_stream", None) is None:
                    self._d2h_stream = torch.cuda.Stream(device=self.device)
                start, done = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self._d2h_stream.wait_event(after)
                with torch.cuda.stream(self._d2h_stream):
                    start.record()
                    outer_host.copy_(outer, non_blocking=True)
                    mom_host.copy_(mom, non_blocking=True)
                    done.record()
                done.synchronize()
                self.last_host_refresh_ms = start.elapsed_time(done)
            finally:
                torch.cuda.set_device(prev)

