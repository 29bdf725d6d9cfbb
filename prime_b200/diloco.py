"""DiLoCo: local AdamW inner steps, Nesterov-SGD outer steps on the averaged pseudo-gradient. The outer state has
pinned host copies as in the reference (src/zeroband/diloco.py:24-215); with the fused engine on CUDA the working
copies live in device memory and the host copies are written when something reads them.

Public surface kept from the reference: ``Diloco(config, model, elastic_device_mesh)``,
``step(model, fake, flag)``, ``sync_pseudo_gradient``, ``sync_inner_model``, ``get_offloaded_param``
and the attributes ``param_list_cpu``, ``outer_optimizer``, ``offloaded_data_flat_tensor``,
``offloaded_grad_flat_tensor``.

``model`` is either an ``nn.Module`` (eager path; its parameters are the local shards) or a
:class:`prime_b200.engine.fused_llama.FusedLlama` (its fp32 master shard is the local shard). In
both cases this rank only ever talks to the ranks that hold the *same shard* in the other workers.

Design differences from the reference:
  * the two host buffers are pinned, and for the fused engine they mirror the device shard layout,
    so the device<->host moves are one bulk copy each way instead of one pageable copy per
    parameter (the reference's G18 path, diloco.py:98-99, 143-144);
  * a worker group that offers ``fused_outer_step`` (NVLink peers inside one box,
    parallel/diloco_comm.py) runs pseudo-gradient, int8 all-reduce and the Nesterov update in one
    GPU kernel sequence; the host path below is used for TCP rings and torch process groups;
  * on that host path with the fused engine on CUDA (``diloco.outer_state_resident``, default on) the pseudo-gradient is
    formed on the device, only it crosses to the host for the exchange and back, and the Nesterov update runs on device
    copies of outer parameters and momentum; ``wait_host_state()`` refreshes ``param_list_cpu`` and the outer optimizer's
    momentum buffers on demand (checkpoint save, live recovery, hash log) and ``mark_host_state_written()`` tells this
    class that somebody rewrote them (checkpoint load, live recovery);
  * ``fake=True`` (a freshly joined worker) contributes a zero pseudo-gradient but still receives
    the average, as the reference's README describes.
"""
from __future__ import annotations

import re
import threading
import time

import torch
import torch.distributed as dist
from torch import nn

from .collectives import all_reduce
from .config import Compression, DilocoConfig
from .utils.logger import get_logger


def _find_first_number(s: str) -> int | None:
    m = re.search(r"\d+", s)
    return int(m.group()) if m else None


def _is_engine(model) -> bool:
    """True for backends whose local shards live in one flat fp32 buffer (``.master``)."""
    return hasattr(model, "master") and hasattr(model, "named_master_shards")


def _named_local_shards(model):
    """(name, fp32 local shard tensor) in parameter order."""
    if hasattr(model, "named_master_shards"):
        return list(model.named_master_shards())
    out = []
    for name, p in model.named_parameters():
        if p.requires_grad:
            t = p.data
            out.append((name, t.to_local() if hasattr(t, "to_local") else t))
    return out


class Diloco:
    def __init__(self, config: DilocoConfig, model, elastic_device_mesh):
        self.config = config
        self.elastic_device_mesh = elastic_device_mesh
        self._logger = get_logger()
        if config.compression == Compression.UINT8:
            from . import native
            native.host()   # build / load the native quantiser + ring now rather than at the first outer step
        self._host_changed = True      # the device copies of the outer state are older than the host's
        self._dev = None               # (outer, momentum, pseudo-gradient) fp32 device copies of this rank's shard, see _device_state
        self._host_stale = False       # the device copies are newer than the host's (refreshed on demand by wait_host_state)
        self._state_lock = threading.Lock()
        self._init_offloaded_optimizer(model)

    # ------------------------------------------------------------------ host copies of the outer state
    def wait_host_state(self) -> None:
        """Call before reading ``param_list_cpu`` / the outer optimizer's state: with ``outer_state_resident`` they are
        brought up to date with the device copies only now, on demand."""
        with self._state_lock:
            if self._host_stale and self._dev is not None:
                outer, mom, _ = self._dev
                self.offloaded_data_flat_tensor.copy_(outer)
                self._momentum_flat().copy_(mom)
                self._host_stale = False
        waiter = getattr(self.elastic_device_mesh.global_pg, "wait_host_copies", None)
        if waiter is not None:
            waiter()

    def mark_host_state_written(self) -> None:
        """Call after writing ``param_list_cpu`` or loading the outer optimizer's state (checkpoint load, live
        recovery): the next outer step reads the host copies again, and the momentum view is rebuilt because
        ``load_state_dict`` replaces the optimizer's buffers."""
        waiter = getattr(self.elastic_device_mesh.global_pg, "wait_host_copies", None)
        if waiter is not None:
            waiter()
        with self._state_lock:
            self._host_stale = False       # whatever the device held is superseded by what was just written
            self._host_changed = True
            if hasattr(self, "_momentum"):
                del self._momentum

    def _device_state(self, model):
        """fp32 device copies of outer parameters and momentum plus a pseudo-gradient buffer for this rank's shard, for
        the fused engine on CUDA with ``outer_state_resident``: the outer step then costs one device-to-host copy of the
        pseudo-gradient and one copy back instead of host-side subtraction and a host-side optimizer step. Returns None
        when the mode does not apply or the 12 bytes per parameter are not available."""
        if not (self.config.outer_state_resident and self._engine_layout and model.device.type == "cuda") or \
                getattr(self, "_no_device_state", False):
            return None
        n = model.master.numel()
        if self._dev is None or self._dev[0].numel() != n:
            try:
                self._dev = tuple(torch.empty(n, dtype=torch.float32, device=model.device) for _ in range(3))
            except torch.cuda.OutOfMemoryError:
                self._logger.warning("no room for the outer state on the device (12 bytes per parameter): outer steps use the host path")
                self._no_device_state, self._dev = True, None
                return None
            self._host_changed = True
        if self._host_changed:
            self._dev[0].copy_(self.offloaded_data_flat_tensor, non_blocking=True)
            self._dev[1].copy_(self._momentum_flat(), non_blocking=True)
            self._host_changed = False
            self._host_stale = False
        return self._dev

    # ------------------------------------------------------------------ setup
    @torch.no_grad()
    def _init_offloaded_optimizer(self, model) -> None:
        self.param_list_cpu = self.get_offloaded_param(model)
        self.outer_optimizer = torch.optim.SGD(self.param_list_cpu, lr=self.config.outer_lr, momentum=0.9, nesterov=True)
        self._logger.debug("offload model to cpu")

    @torch.no_grad()
    def get_offloaded_param(self, model) -> list[nn.Parameter]:
        """Allocate the two flat host buffers (outer params, pseudo-gradient), copy the current
        local shards into the first and return one ``nn.Parameter`` view per model parameter with a
        pre-allocated ``.grad`` view. Buckets for the all-reduce are cut wherever the first integer
        in the parameter name changes: [embedding] [layer 0] ... [layer L-1] [norm, output]."""
        shards = _named_local_shards(model)
        pin = torch.cuda.is_available()
        self._engine_layout = _is_engine(model)
        if self._engine_layout:
            total = model.master.numel()
            base = model.master.data_ptr()
            offsets = [(t.data_ptr() - base) // 4 for _, t in shards]
        else:
            offsets, total = [], 0
            for _, t in shards:
                offsets.append(total)
                total += t.numel()
        self.offloaded_data_flat_tensor = torch.zeros(total, dtype=torch.float32, pin_memory=pin)
        self.offloaded_grad_flat_tensor = torch.zeros(total, dtype=torch.float32, pin_memory=pin)
        params, cutoffs, prev = [], [], object()
        for (name, t), off in zip(shards, offsets):
            key = _find_first_number(name)
            if key != prev:
                cutoffs.append(off)
                prev = key
            data = self.offloaded_data_flat_tensor[off: off + t.numel()].view(t.shape)
            grad = self.offloaded_grad_flat_tensor[off: off + t.numel()].view(t.shape)
            data.copy_(t)
            p = nn.Parameter(data, requires_grad=True)
            p.grad = grad
            params.append(p)
        cutoffs.append(total)
        self._offloaded_grad_grouped_tensor = [self.offloaded_grad_flat_tensor[i:j] for i, j in zip(cutoffs, cutoffs[1:]) if j > i]
        self._param_names = [n for n, _ in shards]
        return params

    # ------------------------------------------------------------------ pseudo-gradient
    @torch.no_grad()
    def _compute_pseudo_gradient(self, model, fake: bool, scale: float = 1.0) -> None:
        """offloaded_grad_flat_tensor := (outer - inner) * scale (zeros for a fake step)."""
        if fake:
            self.offloaded_grad_flat_tensor.zero_()
            self._device_state(model)      # a joiner's first outer step still needs its device copies in place
            return
        dev = self._device_state(model)
        if dev is not None:
            # outer - inner (and the 1 / workers factor) on the device, one bulk device->host copy of the result
            torch.sub(dev[0], model.master, out=dev[2])
            if scale != 1.0:
                dev[2].mul_(scale)
            self.offloaded_grad_flat_tensor.copy_(dev[2], non_blocking=False)
            return
        if self._engine_layout:
            # one bulk device->host copy of the whole fp32 shard, then grad = outer - inner on the host
            self.offloaded_grad_flat_tensor.copy_(model.master, non_blocking=False)
            torch.sub(self.offloaded_data_flat_tensor, self.offloaded_grad_flat_tensor, out=self.offloaded_grad_flat_tensor)
        else:
            for p_off, (_, t) in zip(self.param_list_cpu, _named_local_shards(model)):
                p_off.grad.copy_(t)
                torch.sub(p_off.data, p_off.grad, out=p_off.grad)
        if scale != 1.0:
            self.offloaded_grad_flat_tensor.mul_(scale)

    @torch.no_grad()
    def sync_pseudo_gradient(self, model, fake: bool = False, flag: str = "outer") -> None:
        """Average ``outer - inner`` over the workers. Failures of the collective re-resolve the
        worker group and retry ``retry_all_reduce`` times; after that the local pseudo-gradient is
        used un-reduced (the worker keeps training on its own)."""
        t_start = time.perf_counter()
        edm = self.elastic_device_mesh
        edm.maybe_reinit_global_pg(admit_joiners=False)
        global_pg = edm.global_pg
        self._logger.debug("sync pseudo gradient%s with world size %d", " fake" if fake else "", global_pg.size())
        for attempt in range(self.config.retry_all_reduce):
            self._compute_pseudo_gradient(model, fake, 1.0 / global_pg.size())
            try:
                t_coll = time.perf_counter()
                edm.monitored_barrier(flag)
                for j, bucket in enumerate(self._offloaded_grad_grouped_tensor):
                    t0 = time.perf_counter()
                    all_reduce(self.config.compression, bucket, dist.ReduceOp.SUM, global_pg)
                    self._logger.debug(f"{j}/{len(self._offloaded_grad_grouped_tensor)} all reduce bucket done in "
                                       f"{time.perf_counter() - t0:.6f} seconds, numel: {bucket.numel()}")
                self.last_all_reduce_seconds = time.perf_counter() - t_coll
                self._logger.debug(f"All reduce takes {self.last_all_reduce_seconds:.6f} seconds numels: "
                                   f"{self.offloaded_grad_flat_tensor.numel()}")
                break
            except Exception as e:  # noqa: BLE001
                self._logger.error(f"Error syncing pseudo gradient: {e}, retry {attempt + 1}/{self.config.retry_all_reduce}")
                global_pg = edm.get_global_pg(maybe_reinit=True)
        else:
            self._logger.error("Failed to sync pseudo gradient after %d retries. Resorting to calculating pseudo-gradient "
                               "without reduce", self.config.retry_all_reduce)
            self._compute_pseudo_gradient(model, fake)
        self._logger.info(f"Sync psuedo-gradient in {time.perf_counter() - t_start:.6f} seconds")

    # ------------------------------------------------------------------ inner model refresh
    @torch.no_grad()
    def sync_inner_model(self, model) -> None:
        """Copy the (updated) outer parameters back into the inner model's local shards."""
        if self._engine_layout:
            model.master.copy_(self.offloaded_data_flat_tensor, non_blocking=True)
            model.publish_params()
            return
        for p_off, (_, t) in zip(self.param_list_cpu, _named_local_shards(model)):
            t.copy_(p_off.data)

    @torch.no_grad()
    def set_outer_from_inner(self, model) -> None:
        """outer := inner (after a checkpoint load or live recovery)."""
        self.wait_host_state()
        self._host_changed = True
        if self._engine_layout:
            self.offloaded_data_flat_tensor.copy_(model.master)
            return
        for p_off, (_, t) in zip(self.param_list_cpu, _named_local_shards(model)):
            p_off.data.copy_(t)

    # ------------------------------------------------------------------ outer step
    @torch.no_grad()
    def step(self, model, fake: bool = False, flag: str = "outer") -> None:
        t0 = time.perf_counter()
        fused = getattr(self.elastic_device_mesh.global_pg, "fused_outer_step", None)
        if fused is not None and self._engine_layout and model.device.type == "cuda":
            self._fused_step(model, fused, fake, flag)
            return
        with self._state_lock:
            self.sync_pseudo_gradient(model, fake=fake, flag=flag)
            self._logger.info(f"all reduce pseudo gradient in: {time.perf_counter() - t0} seconds")
            dev = self._device_state(model) if self.outer_optimizer is not None else None
            if dev is not None:
                self._device_outer_update(model, dev)
                return
        if self.outer_optimizer is not None:
            self.outer_optimizer.step()
        self.sync_inner_model(model)

    def _device_outer_update(self, model, dev) -> None:
        """Nesterov SGD of the outer parameters on the device copies (what ``torch.optim.SGD(momentum, nesterov=True)``
        does to the host copies), then inner := outer. The host copies become stale; wait_host_state() refreshes them."""
        outer, mom, g = dev
        group = self.outer_optimizer.param_groups[0]
        lr, mu = float(group["lr"]), float(group["momentum"])
        g.copy_(self.offloaded_grad_flat_tensor, non_blocking=True)        # the averaged pseudo-gradient
        mom.mul_(mu).add_(g)
        outer.sub_(g.add_(mom, alpha=mu), alpha=lr)
        model.master.copy_(outer)
        self._host_stale = True
        model.publish_params()

    def _momentum_flat(self) -> torch.Tensor:
        """Flat host view of the SGD momentum buffers (allocated on first use, same layout as the data)."""
        if not hasattr(self, "_momentum"):
            self._momentum = torch.zeros_like(self.offloaded_data_flat_tensor, pin_memory=torch.cuda.is_available())
            base = self.offloaded_data_flat_tensor.data_ptr()
            for p in self.param_list_cpu:
                off = (p.data.data_ptr() - base) // 4
                buf = self._momentum[off: off + p.numel()].view(p.shape)
                st = self.outer_optimizer.state[p]
                if "momentum_buffer" in st and st["momentum_buffer"] is not None:
                    buf.copy_(st["momentum_buffer"])
                st["momentum_buffer"] = buf
        return self._momentum

    def _fused_step(self, model, fused, fake: bool, flag: str) -> None:
        """GPU path: stage outer params + momentum to HBM, run the fused int8 all-reduce + Nesterov
        kernels against the peers' symmetric buffers, bring the new outer state back."""
        edm = self.elastic_device_mesh
        edm.maybe_reinit_global_pg(admit_joiners=False)
        for attempt in range(self.config.retry_all_reduce):
            try:
                edm.monitored_barrier(flag)
                fused(model, self.offloaded_data_flat_tensor, self._momentum_flat(), lr=self.config.outer_lr, momentum=0.9,
                      fake=fake, compression=self.config.compression,
                      first_step=not getattr(self, "_fused_stepped", False),
                      resident=self.config.outer_state_resident, host_changed=self._host_changed)
                self._fused_stepped = True
                self._host_changed = False
                model.publish_params()
                return
            except Exception as e:  # noqa: BLE001
                self._logger.error(f"Error in fused outer step: {e}, retry {attempt + 1}/{self.config.retry_all_reduce}")
                edm.get_global_pg(maybe_reinit=True)
                fused = getattr(edm.global_pg, "fused_outer_step", None)
                if fused is None:
                    break
        # host path: the host copies are the truth again (and stay it: no second set of device copies beside the group's)
        self.wait_host_state()
        self._host_changed = True
        self._no_device_state = True
        self.sync_pseudo_gradient(model, fake=fake, flag=flag)
        self.outer_optimizer.step()
        self.sync_inner_model(model)
