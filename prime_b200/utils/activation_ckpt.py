"""Activation checkpointing for the eager module (reference: src/zeroband/utils/activation_ckpt.py:8-24).

``num`` selects every ``num``-th transformer block (1 = all). The reference increments its block
counter only inside the branch that wraps, so with ``num > 1`` it wraps just the first block; the
behaviour here is the documented one. The fused engine has its own recompute path
(``FusedLlama(ac_ckpt=...)``) with the same selection rule."""
from __future__ import annotations

import torch
from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import checkpoint_wrapper

from .logger import get_logger


def apply_ac_ckpt(model: torch.nn.Module, num: int) -> None:
    """Wrap every ``num``-th block of ``model.layers`` so its activations are recomputed in backward."""
    logger = get_logger()
    wrapped = 0
    for idx, (layer_id, block) in enumerate(list(model.layers.named_children())):
        if idx % max(1, num) == 0:
            model.layers.register_module(layer_id, checkpoint_wrapper(block, preserve_rng_state=False))
            wrapped += 1
    logger.debug(f"Applied activation checkpointing to {wrapped} layers")
