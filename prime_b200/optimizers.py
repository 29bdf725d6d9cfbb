"""Inner optimizers for the eager path (reference: src/zeroband/optimizers.py:17-52).

AdamW maps to ``torch.optim.AdamW`` on CPU parameters (the fused engine has its own sharded AdamW
kernel). SOAP needs the optional ``distributed_shampoo`` package; when it is absent a clear error is
raised at construction time instead of at import time."""
from __future__ import annotations

from typing import Iterable

import torch

from .config import AdamConfig, OptimizersConfig, SoapConfig


def get_optimizer(params: Iterable[torch.nn.Parameter], config: OptimizersConfig) -> torch.optim.Optimizer:
    if isinstance(config, AdamConfig):
        return torch.optim.AdamW(params, lr=config.lr, weight_decay=config.weight_decay, betas=(config.betas1, config.betas2))
    if isinstance(config, SoapConfig):
        try:
            from distributed_shampoo import DefaultEigenvalueCorrectedShampooConfig, DistributedShampoo, FullyShardShampooConfig
        except ImportError as e:
            raise ImportError("optim.optim.type = 'soap' needs the distributed_shampoo package (facebookresearch/optimizers)") from e
        return DistributedShampoo(
            params, lr=config.lr, betas=(config.betas1, config.betas2), epsilon=1e-12, weight_decay=config.weight_decay,
            max_preconditioner_dim=config.max_preconditioner_dim, precondition_frequency=config.precondition_frequency,
            use_decoupled_weight_decay=True, preconditioner_config=DefaultEigenvalueCorrectedShampooConfig,
            distributed_config=FullyShardShampooConfig())
    raise ValueError(f"Unknown optimizer {config}")


__all__ = ["OptimizersConfig", "get_optimizer"]
