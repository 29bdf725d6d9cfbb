"""Training backends: the object the training loop, DiLoCo and the checkpoint manager talk to.

Two implementations of one small surface:

* :class:`FusedBackend` — the B200 path: :class:`prime_b200.engine.fused_llama.FusedLlama`
  (hand-written kernels, ZeRO-3 flat shards over symmetric memory).
* :class:`EagerBackend` — an ``nn.Module`` with a torch optimizer; CPU ranks (gloo) use it, e.g. the
  tiny-Llama DiLoCo configuration and every CPU test. With more than one local rank gradients are
  averaged with an all-reduce (data parallel; every rank holds the full parameters).

Surface: ``train_step(batch, micro_bs) -> dict``, ``named_master_shards()``, ``publish_params()``,
``model_state_dict()/load_model_state_dict()``, ``optimizer_state_dict()/load_optimizer_state_dict()``,
``lr_scheduler`` (a real ``LambdaLR`` in both cases, so its checkpointed state has one format).
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist
from torch import nn
from torch.distributed.tensor import DTensor, Shard

from .loss import compute_cross_entropy_loss
from .ops import kernels as K


def _split_seq_start(seq_start, mb: int, micro_bs: int, T: int):
    if seq_start is None:
        return None
    lo = mb * micro_bs * T
    return seq_start[lo: lo + micro_bs * T] - lo


class EagerBackend:
    def __init__(self, model: nn.Module, optimizer: torch.optim.Optimizer, scheduler, local_pg=None, z_loss_weight: float | None = None,
                 num_chunks: int | None = None, fused_linear_ce: bool = False, max_norm: float = 1.0):
        self.model, self.optimizer, self.lr_scheduler = model, optimizer, scheduler
        self.local_pg = local_pg
        self.z_loss_weight, self.num_chunks, self.fused_linear_ce = z_loss_weight, num_chunks, fused_linear_ce
        self.max_norm = max_norm
        self.device = next(model.parameters()).device
        self.is_fused = False

    @property
    def local_world(self) -> int:
        return dist.get_world_size(self.local_pg) if (self.local_pg is not None and dist.is_initialized()) else 1

    def train_step(self, batch: dict, micro_bs: int) -> dict[str, float]:
        tokens, labels, seq_start = batch["input_ids"], batch["labels"], batch.get("seq_start")
        B, T = tokens.shape
        n_micro = max(1, B // micro_bs)
        loss_sum, z_sum = 0.0, 0.0
        for mb in range(n_micro):
            sl = slice(mb * micro_bs, (mb + 1) * micro_bs)
            out = self.model(tokens[sl], seq_start=_split_seq_start(seq_start, mb, micro_bs, T))
            weight = self.model.output.weight if self.fused_linear_ce else None
            ce, z = compute_cross_entropy_loss(out, labels[sl], z_weight=self.z_loss_weight, num_chunks=self.num_chunks,
                                               fused_linear_weight=weight)
            loss = (ce + z if z is not None else ce) / n_micro
            loss.backward()
            loss_sum += float(ce.detach()) / n_micro
            z_sum += float(z.detach()) / n_micro if z is not None else 0.0
        if self.local_world > 1:
            for p in self.model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.local_pg)
                    p.grad.div_(self.local_world)
            t = torch.tensor([loss_sum, z_sum], device=self.device)
            dist.all_reduce(t, group=self.local_pg)
            loss_sum, z_sum = (t / self.local_world).tolist()
        grad_norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_norm)
        self.optimizer.step()
        self.lr_scheduler.step()
        self.optimizer.zero_grad()
        return {"loss": loss_sum, "z_loss": z_sum, "grad_norm": float(grad_norm)}

    def named_master_shards(self):
        for n, p in self.model.named_parameters():
            if p.requires_grad:
                yield n, p.data

    def publish_params(self) -> None:
        pass

    def current_lr(self) -> float:
        return self.lr_scheduler.get_last_lr()[0]

    # ---- checkpoint state ----
    def model_state_dict(self) -> dict[str, Any]:
        from torch.distributed.checkpoint.state_dict import StateDictOptions, get_model_state_dict
        return get_model_state_dict(self.model, options=StateDictOptions(strict=False))

    def load_model_state_dict(self, sd: dict[str, Any]) -> None:
        from torch.distributed.checkpoint.state_dict import StateDictOptions, set_model_state_dict
        set_model_state_dict(self.model, sd, options=StateDictOptions(strict=False))

    def optimizer_state_dict(self) -> dict[str, Any]:
        from torch.distributed.checkpoint.state_dict import StateDictOptions, get_optimizer_state_dict
        return get_optimizer_state_dict(self.model, self.optimizer, options=StateDictOptions(flatten_optimizer_state_dict=True))

    def load_optimizer_state_dict(self, sd: dict[str, Any]) -> None:
        from torch.distributed.checkpoint.state_dict import StateDictOptions, set_optimizer_state_dict
        set_optimizer_state_dict(self.model, self.optimizer, sd, options=StateDictOptions(flatten_optimizer_state_dict=True))


class FusedBackend:
    """Adapter around :class:`FusedLlama`. ``scheduler`` is a ``LambdaLR`` on a one-parameter dummy
    optimizer: it only produces the learning rate the sharded update is launched with. With ``optim.type = "adam"`` the
    update is the engine's sharded AdamW kernel; with ``"soap"`` it is :class:`prime_b200.optimizers.SOAP` stepping this
    rank's fp32 shards (``FusedLlama.set_shard_optimizer``): forward, backward, reduce-scatter, clip and the bf16 all-gather
    stay on the engine's kernels, and every rank preconditions its own block of rows, as the reference's fully-sharded
    Shampoo does (src/zeroband/optimizers.py:31-48)."""

    def __init__(self, engine, optim_cfg, sched_factory, mesh=None, max_norm: float = 1.0):
        self.engine = engine
        self.cfg = optim_cfg
        self._dummy = nn.Parameter(torch.zeros(1))
        self.optimizer = torch.optim.SGD([self._dummy], lr=optim_cfg.lr)
        self.lr_scheduler = sched_factory(self.optimizer)
        self.mesh = mesh
        self.max_norm = max_norm
        self.device = engine.device
        self.is_fused = True
        self.shard_optimizer = None
        if getattr(optim_cfg, "type", "adam") == "soap":
            from .optimizers import SOAP
            c = optim_cfg
            self.shard_optimizer = engine.set_shard_optimizer(lambda params: SOAP(
                params, lr=c.lr, betas=(c.betas1, c.betas2), eps=1e-12, weight_decay=c.weight_decay,
                max_preconditioner_dim=c.max_preconditioner_dim, precondition_frequency=c.precondition_frequency))
            self.shard_optimizer.materialize_state()      # checkpoints load in place: the state must exist before the first step

    # surface used by Diloco
    def named_master_shards(self):
        return self.engine.named_master_shards()

    @property
    def master(self):
        return self.engine.master

    def publish_params(self):
        self.engine.publish_params()

    def current_lr(self) -> float:
        return self.lr_scheduler.get_last_lr()[0]

    def train_step(self, batch: dict, micro_bs: int) -> dict[str, Any]:
        c = self.cfg
        loss, norm = self.engine.train_step(batch["input_ids"], batch["labels"], self.current_lr(), micro_bs=micro_bs,
                                            betas=(c.betas1, c.betas2), weight_decay=c.weight_decay, max_norm=self.max_norm,
                                            seq_start=batch.get("seq_start"), sync_loss=True)
        self.optimizer.step()          # the dummy optimizer only carries the schedule; stepping it keeps the scheduler's bookkeeping quiet
        self.lr_scheduler.step()
        z = float(self.engine._ws["step.loss"][1]) if self.engine.z_weight else 0.0
        return {"loss": loss, "z_loss": z, "grad_norm": norm}

    # ---- checkpoint state: this rank's dim-0 shards presented as DTensors ----
    def _dt(self, buf: torch.Tensor, name: str):
        eng = self.engine
        local = eng.shard_view(buf, name)
        if self.mesh is None:
            return local
        p = eng.layout.params[eng.layout.by_name[name]]
        stride = [1] * len(p.shape)
        for i in range(len(p.shape) - 2, -1, -1):
            stride[i] = stride[i + 1] * p.shape[i + 1]
        return DTensor.from_local(local, self.mesh, [Shard(0)], run_check=False, shape=torch.Size(p.shape), stride=tuple(stride))

    def model_state_dict(self) -> dict[str, Any]:
        eng = self.engine
        sd = {p.name: self._dt(eng.master, p.name) for p in eng.layout.params}
        a = eng.args
        from .models.llama import precompute_freqs_cis
        sd["freqs_cis"] = precompute_freqs_cis(a.head_dim, a.max_seq_len * 2, a.rope_theta)
        return sd

    def load_model_state_dict(self, sd: dict[str, Any]) -> None:
        # DCP loads in place into the DTensor locals, which are views of the master shard
        self.engine.publish_params()

    def _soap_key(self, i: int, k: str) -> str:
        # the state of a shard optimizer belongs to this rank's rows (its factors have the shard's shape, not a slice of a
        # global tensor's), so it is stored under keys of this rank
        return f"state.rank{self.engine.rank}.{self.engine.layout.params[i].name}.{k}"

    def optimizer_state_dict(self) -> dict[str, Any]:
        eng, c = self.engine, self.cfg
        out: dict[str, Any] = {}
        if self.shard_optimizer is not None:
            out["state.step"] = torch.tensor(float(eng.opt_step))
            for i, q in enumerate(eng._shard_params):
                for k, v in self.shard_optimizer.state.get(q, {}).items():
                    if v is None:                                # a side wider than max_preconditioner_dim: identity factor
                        continue
                    if torch.is_tensor(v):
                        out[self._soap_key(i, k)] = v
                    else:
                        out[self._soap_key(i, k)] = torch.tensor(float(v))
            return out
        for p in eng.layout.params:
            out[f"state.{p.name}.step"] = torch.tensor(float(eng.opt_step))
            out[f"state.{p.name}.exp_avg"] = self._dt(eng.exp_avg, p.name)
            out[f"state.{p.name}.exp_avg_sq"] = self._dt(eng.exp_avg_sq, p.name)
            for k, v in (("lr", c.lr), ("betas", (c.betas1, c.betas2)), ("eps", 1e-8), ("weight_decay", c.weight_decay),
                         ("amsgrad", False), ("maximize", False)):
                out[f"param_groups.{p.name}.{k}"] = v
        return out

    def load_optimizer_state_dict(self, sd: dict[str, Any]) -> None:
        if self.shard_optimizer is not None:
            # DCP loads tensors in place into the objects optimizer_state_dict() handed out; plain numbers come back here
            step = sd.get("state.step")
            if step is not None:
                self.engine.opt_step = int(float(step))
            for i, q in enumerate(self.engine._shard_params):
                st = self.shard_optimizer.state.get(q)
                if st is not None and self._soap_key(i, "step") in sd:
                    st["step"] = int(float(sd[self._soap_key(i, "step")]))
            return
        first = self.engine.layout.params[0].name
        step = sd.get(f"state.{first}.step")
        if step is not None:
            self.engine.opt_step = int(float(step))
