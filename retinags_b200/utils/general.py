"""Small numeric helpers shared by trainer and models.

Parity: ``utils/general_utils.py:18-151`` of the reference (inverse sigmoid, the log-linear
learning-rate schedule with optional warm-up delay, the batch-aware "every N iterations" tests
used because one step advances the iteration counter by the batch size, seeding).
"""
from __future__ import annotations

import math
import random

import numpy as np
import torch


def inverse_sigmoid(x: torch.Tensor) -> torch.Tensor:
    return torch.log(x / (1 - x))


def expon_lr(step: float, lr_init: float, lr_final: float, lr_delay_steps: int = 0, lr_delay_mult: float = 1.0,
             max_steps: int = 1_000_000) -> float:
    """Log-linear interpolation from ``lr_init`` to ``lr_final`` over ``max_steps``; 0 when disabled."""
    if step < 0 or lr_init <= 0.0 or lr_final <= 0.0:
        return 0.0
    if lr_delay_steps > 0:
        delay = lr_delay_mult + (1 - lr_delay_mult) * math.sin(0.5 * math.pi * min(max(step / lr_delay_steps, 0.0), 1.0))
    else:
        delay = 1.0
    t = min(max(step / max_steps, 0.0), 1.0)
    return delay * math.exp(math.log(lr_init) * (1 - t) + math.log(lr_final) * t)


def is_interval_in_batch(start_iter: int, batch_size: int, interval: int, low_limit: int = 0) -> bool:
    """True when a multiple of ``interval`` falls inside [start_iter, start_iter + batch_size)."""
    assert batch_size > 0 and interval > 0
    if start_iter <= low_limit:
        return False
    if batch_size >= interval:
        return True
    if batch_size == 1:
        return start_iter % interval == 0
    head, tail = start_iter % interval, (start_iter + batch_size - 1) % interval
    return head == 0 or head > tail


def is_point_in_batch(start_iter: int, batch_size: int, point: int) -> bool:
    return start_iter <= point < start_iter + batch_size


def seed_everything(seed: int = 0):
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
