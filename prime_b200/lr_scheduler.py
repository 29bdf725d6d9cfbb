"""Learning-rate schedules as pure functions of the step plus a LambdaLR factory
(reference: src/zeroband/lr_scheduler.py:10-55; cosine / linear there come from transformers)."""
from __future__ import annotations

import math
from functools import partial

from torch.optim import Optimizer
from torch.optim.lr_scheduler import LambdaLR

SCHED_TYPES = ("cosine", "linear", "wsd-sqrt")


def linear_factor(step: int, *, num_warmup_steps: int, num_training_steps: int) -> float:
    if step < num_warmup_steps:
        return step / max(1, num_warmup_steps)
    return max(0.0, (num_training_steps - step) / max(1, num_training_steps - num_warmup_steps))


def cosine_factor(step: int, *, num_warmup_steps: int, num_training_steps: int, num_cycles: float = 0.5) -> float:
    if step < num_warmup_steps:
        return step / max(1, num_warmup_steps)
    progress = (step - num_warmup_steps) / max(1, num_training_steps - num_warmup_steps)
    return max(0.0, 0.5 * (1.0 + math.cos(math.pi * num_cycles * 2.0 * progress)))


def wsd_sqrt_factor(step: int, *, num_warmup_steps: int, num_stable_steps: int, num_training_steps: int,
                    min_lr_ratio: float = 0.0) -> float:
    """Warmup -> stable -> (1 - sqrt) decay."""
    if step < num_warmup_steps:
        return step / max(1, num_warmup_steps)
    if step < num_stable_steps:
        return 1.0
    if step < num_training_steps:
        progress = (step - num_stable_steps) / max(1, num_training_steps - num_stable_steps)
        return max(min_lr_ratio, 1 - math.sqrt(progress))
    return min_lr_ratio


def get_factor_fn(sched_type: str, num_warmup_steps: int, num_stable_steps: int, num_training_steps: int):
    if sched_type == "cosine":
        return partial(cosine_factor, num_warmup_steps=num_warmup_steps, num_training_steps=num_training_steps)
    if sched_type == "linear":
        return partial(linear_factor, num_warmup_steps=num_warmup_steps, num_training_steps=num_training_steps)
    if sched_type == "wsd-sqrt":
        return partial(wsd_sqrt_factor, num_warmup_steps=num_warmup_steps, num_stable_steps=num_stable_steps,
                       num_training_steps=num_training_steps)
    raise ValueError(f"Unknown scheduler type: {sched_type}")


def get_scheduler(sched_type: str, optimizer: Optimizer, num_warmup_steps: int, num_stable_steps: int,
                  num_training_steps: int) -> LambdaLR:
    return LambdaLR(optimizer, get_factor_fn(sched_type, num_warmup_steps, num_stable_steps, num_training_steps))
