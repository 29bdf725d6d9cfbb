"""Inner optimizers for the eager path (reference: src/zeroband/optimizers.py:17-52).

AdamW maps to ``torch.optim.AdamW`` (the fused engine has its own sharded AdamW kernel). SOAP -- Adam run
in the eigenbasis of Shampoo's Kronecker-factored second-moment statistics, which is what the reference
gets from ``DistributedShampoo(preconditioner_config=DefaultEigenvalueCorrectedShampooConfig)`` -- uses that
package when it is installed and the self-contained :class:`SOAP` below otherwise, so
``optim.optim.type = "soap"`` trains either way."""
from __future__ import annotations

from typing import Iterable

import torch

from .config import AdamConfig, OptimizersConfig, SoapConfig


class SOAP(torch.optim.Optimizer):
    """Eigenvalue-corrected Shampoo (SOAP, Vyas et al. 2024), one process / one shard at a time.

    For every parameter with two or more dimensions the gradient is viewed as a matrix ``G`` (leading
    dimensions merged). Exponential averages ``L = E[G G^T]`` and ``R = E[G^T G]`` are kept for every side not
    larger than ``max_preconditioner_dim``; their eigenvectors ``Q_L``, ``Q_R`` are refreshed every
    ``precondition_frequency`` steps by one power-iteration + QR step from the previous basis. Adam's
    second moment lives in the rotated space (``Q_L^T G Q_R``), its first moment in the original one, and the
    normalised step is rotated back. Vectors and over-wide sides fall back to plain AdamW / an identity
    factor. Weight decay is decoupled. With FSDP-style row shards each rank preconditions its own shard, the
    same block-diagonal approximation the reference's fully-sharded Shampoo makes."""

    def __init__(self, params, lr: float = 4e-4, betas=(0.9, 0.95), eps: float = 1e-12, weight_decay: float = 1e-5,
                 max_preconditioner_dim: int = 8192, precondition_frequency: int = 100, shampoo_beta: float | None = None):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, max_preconditioner_dim=max_preconditioner_dim,
                        precondition_frequency=precondition_frequency,
                        shampoo_beta=betas[1] if shampoo_beta is None else shampoo_beta)
        super().__init__(params, defaults)

    @staticmethod
    def _rotate(x: torch.Tensor, qs, back: bool) -> torch.Tensor:
        ql, qr = qs
        if ql is not None:
            x = (ql if back else ql.t()) @ x
        if qr is not None:
            x = x @ (qr.t() if back else qr)
        return x

    @staticmethod
    def _eigvecs(m: torch.Tensor) -> torch.Tensor:
        # symmetric PSD: eigh in fp64 on a jittered copy, eigenvectors by decreasing eigenvalue
        a = m.double()
        a = a + 1e-30 * torch.eye(a.shape[0], dtype=a.dtype, device=a.device)
        _, v = torch.linalg.eigh(a)
        return v.flip(1).to(m.dtype)

    @staticmethod
    def _init_state(st: dict, local: torch.Tensor, max_dim: int, with_bases: bool) -> None:
        st["step"] = 0
        st["exp_avg"] = torch.zeros_like(local)
        st["exp_avg_sq"] = torch.zeros_like(local)
        if local.dim() >= 2:
            g2 = local.reshape(local.shape[0], -1)
            for side, n in (("L", g2.shape[0]), ("R", g2.shape[1])):
                keep = n <= max_dim
                st["GG_" + side] = torch.zeros(n, n, dtype=torch.float32, device=local.device) if keep else None
                # the first step replaces the basis by the eigenvectors of the first statistics; a placeholder of the right
                # shape only matters to a checkpoint loader that fills existing tensors in place
                st["Q_" + side] = torch.eye(n, dtype=torch.float32, device=local.device) if (keep and with_bases) else None

    @torch.no_grad()
    def materialize_state(self) -> None:
        """Create every parameter's state now (zeros, identity bases) instead of at its first step, so that a checkpoint
        loader that loads in place finds tensors of the final shapes."""
        for group in self.param_groups:
            for p in group["params"]:
                if not self.state[p]:
                    local = p._local_tensor if hasattr(p, "_local_tensor") else p
                    self._init_state(self.state[p], local.detach().float(), group["max_preconditioner_dim"], with_bases=True)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            sb, eps, lr, wd = group["shampoo_beta"], group["eps"], group["lr"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g_full = p.grad.float()
                local = g_full._local_tensor if hasattr(g_full, "_local_tensor") else g_full      # DTensor shard
                target = p._local_tensor if hasattr(p, "_local_tensor") else p
                st = self.state[p]
                if not st:
                    self._init_state(st, local, group["max_preconditioner_dim"], with_bases=False)
                st["step"] += 1
                t = st["step"]
                if wd:
                    target.mul_(1.0 - lr * wd)
                if local.dim() < 2:      # norms, biases: AdamW
                    st["exp_avg"].mul_(b1).add_(local, alpha=1 - b1)
                    st["exp_avg_sq"].mul_(b2).addcmul_(local, local, value=1 - b2)
                    denom = (st["exp_avg_sq"] / (1 - b2 ** t)).sqrt_().add_(eps)
                    target.add_((st["exp_avg"] / (1 - b1 ** t) / denom).to(target.dtype), alpha=-lr)
                    continue
                shape = local.shape
                g2 = local.reshape(shape[0], -1)
                # statistics; the very first gradient also defines the first eigenbasis
                if st["GG_L"] is not None:
                    st["GG_L"].mul_(sb).addmm_(g2, g2.t(), alpha=1 - sb)
                if st["GG_R"] is not None:
                    st["GG_R"].mul_(sb).addmm_(g2.t(), g2, alpha=1 - sb)
                if t == 1:
                    for side in ("L", "R"):
                        if st["GG_" + side] is not None:
                            st["Q_" + side] = self._eigvecs(st["GG_" + side])
                elif t % group["precondition_frequency"] == 0:
                    v2 = st["exp_avg_sq"].reshape(shape[0], -1)
                    for dim, side in enumerate(("L", "R")):
                        gg, q = st["GG_" + side], st["Q_" + side]
                        if gg is None:
                            continue
                        est = torch.einsum("ij,ij->j", q, gg @ q)              # diag(Q^T GG Q)
                        order = torch.argsort(est, descending=True)
                        q = q[:, order]
                        v2 = v2.index_select(dim, order)                       # the second moment follows its axes
                        st["Q_" + side] = torch.linalg.qr(gg @ q).Q             # one power-iteration step
                    st["exp_avg_sq"] = v2.reshape(shape).contiguous()
                qs = (st["Q_L"], st["Q_R"])
                g_rot = self._rotate(g2, qs, back=False)
                st["exp_avg"].mul_(b1).add_(local, alpha=1 - b1)
                v2 = st["exp_avg_sq"].reshape(shape[0], -1)
                v2.mul_(b2).addcmul_(g_rot, g_rot, value=1 - b2)
                m_rot = self._rotate(st["exp_avg"].reshape(shape[0], -1), qs, back=False)
                n_rot = (m_rot / (1 - b1 ** t)) / ((v2 / (1 - b2 ** t)).sqrt() + eps)
                upd = self._rotate(n_rot, qs, back=True).reshape(shape)
                target.add_(upd.to(target.dtype), alpha=-lr)
        return loss


def get_optimizer(params: Iterable[torch.nn.Parameter], config: OptimizersConfig) -> torch.optim.Optimizer:
    if isinstance(config, AdamConfig):
        return torch.optim.AdamW(params, lr=config.lr, weight_decay=config.weight_decay, betas=(config.betas1, config.betas2))
    if isinstance(config, SoapConfig):
        try:
            from distributed_shampoo import DefaultEigenvalueCorrectedShampooConfig, DistributedShampoo, FullyShardShampooConfig
        except ImportError:
            return SOAP(params, lr=config.lr, betas=(config.betas1, config.betas2), eps=1e-12, weight_decay=config.weight_decay,
                        max_preconditioner_dim=config.max_preconditioner_dim, precondition_frequency=config.precondition_frequency)
        return DistributedShampoo(
            params, lr=config.lr, betas=(config.betas1, config.betas2), epsilon=1e-12, weight_decay=config.weight_decay,
            max_preconditioner_dim=config.max_preconditioner_dim, precondition_frequency=config.precondition_frequency,
            use_decoupled_weight_decay=True, preconditioner_config=DefaultEigenvalueCorrectedShampooConfig,
            distributed_config=FullyShardShampooConfig())
    raise ValueError(f"Unknown optimizer {config}")


__all__ = ["OptimizersConfig", "SOAP", "get_optimizer"]
