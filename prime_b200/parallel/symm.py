"""Symmetric-memory communicator: peer-mapped buffers + flag pads for the in-kernel collectives.

One process per GPU. ``torch.distributed`` (NCCL backend) is only the plumbing: it provides the
rendezvous through which every rank maps every other rank's allocation
(``torch.distributed._symmetric_memory``, CUDA virtual-memory handles exchanged over the store).
All data movement afterwards is done by this package's own kernels with plain peer loads /
stores over NVLink (csrc/zero_comm.cu, csrc/diloco_comm.cu) and per-peer epoch flags; no NCCL
collective is on the training path and nothing here uses multicast TMA.

Reference counterpart: the NCCL process group FSDP2 uses inside a node
(src/zeroband/comms.py:65-76).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import native
from ..native import check, ptr, stream_ptr
from ..ops.kernels import status_word

MAX_RANKS = 16
FLAG_SLOTS = 64


class SymmComm:
    """Allocates symmetric buffers over a process group and exposes peer pointer tables."""

    def __init__(self, group: dist.ProcessGroup | None = None, device: torch.device | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        assert self.world <= MAX_RANKS
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self._handles = []
        # flag pads: int32 [FLAG_SLOTS, MAX_RANKS]; data pads: fp32 [FLAG_SLOTS, 2, MAX_RANKS, 8]
        self.flags = self._alloc_raw(FLAG_SLOTS * MAX_RANKS, torch.int32)
        self.data = self._alloc_raw(FLAG_SLOTS * 2 * MAX_RANKS * 8, torch.float32)
        self._flag_ptrs = self.peer_ptrs(self.flags)
        self._data_ptrs = self.peer_ptrs(self.data)
        self._epoch = [0] * FLAG_SLOTS
        dist.barrier(self.group)
        torch.cuda.synchronize()

    def host_barrier(self) -> None:
        """Host-level rendezvous of the group (not stream-ordered). Used before the first device barrier of a phase
        whose ranks may arrive seconds apart (start-up, checkpoint load): the device barriers give up after their
        wait budget, the host one does not."""
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def _alloc_raw(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        t.zero_()
        h = self._symm.rendezvous(t, self.group)
        self._handles.append((t, h))
        t._pb_symm_handle = h   # keep the mapping alive with the tensor
        return t

    def alloc(self, numel: int, dtype: torch.dtype, device=None) -> torch.Tensor:
        """Zero-filled symmetric buffer of ``numel`` elements (same size on every rank; collective)."""
        return self._alloc_raw(numel, dtype)

    def peer_ptrs(self, t: torch.Tensor):
        """ctypes ``void*[world]``: address of every rank's copy of symmetric tensor ``t``."""
        h = t._pb_symm_handle
        ptrs = list(h.buffer_ptrs)
        off = t.data_ptr() - ptrs[self.rank]
        return (C.c_void_p * self.world)(*[p + off for p in ptrs])

    def peer_tensor(self, t: torch.Tensor, rank: int) -> torch.Tensor:
        h = t._pb_symm_handle
        return h.get_buffer(rank, tuple(t.shape), t.dtype, 0)

    # ------------------------------------------------------------------ device-side primitives
    def barrier(self, slot: int = 0, stream=None) -> None:
        """Stream-ordered barrier across the group: everything enqueued before it on every rank's
        stream is visible to every rank's kernels enqueued after it. Bounded wait (error code on
        the device status word instead of a hang)."""
        self._epoch[slot] += 1
        check(native.cuda().pb_peer_barrier(self._flag_ptrs, self.world, self.rank, slot, self._epoch[slot],
                                            ptr(status_word(self.device)), stream_ptr(stream)), "pb_peer_barrier")

    def allreduce_scalars(self, src: torch.Tensor, dst: torch.Tensor, n: int, slot: int = 1) -> None:
        """dst[:n] = sum over ranks of src[:n] (n <= 8), same bits on every rank; doubles as a barrier."""
        self._epoch[slot] += 1
        check(native.cuda().pb_allreduce_scalars(self._flag_ptrs, self._data_ptrs, self.world, self.rank, slot, self._epoch[slot],
                                                 ptr(src), ptr(dst), n, ptr(status_word(self.device)), stream_ptr()),
              "pb_allreduce_scalars")
