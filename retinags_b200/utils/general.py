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


def build_rotation(q: torch.Tensor) -> torch.Tensor:
    """(N,3,3) rotation matrices of (N,4) quaternions (w,x,y,z), normalised first (``general_utils.py:73-95``)."""
    q = q / q.norm(dim=1, keepdim=True)
    r, x, y, z = q[:, 0], q[:, 1], q[:, 2], q[:, 3]
    R = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - r * z), 2 * (x * z + r * y),
                     2 * (x * y + r * z), 1 - 2 * (x * x + z * z), 2 * (y * z - r * x),
                     2 * (x * z - r * y), 2 * (y * z + r * x), 1 - 2 * (x * x + y * y)], dim=-1)
    return R.view(-1, 3, 3)


def build_scaling_rotation(s: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """L = R diag(s): the factor of the 3-D covariance Sigma = L L^T (``general_utils.py:97-107``)."""
    return build_rotation(q) * s[:, None, :]


def strip_symmetric(m: torch.Tensor) -> torch.Tensor:
    """Upper triangle (xx, xy, xz, yy, yz, zz) of (N,3,3) symmetric matrices (``general_utils.py:60-71``)."""
    return torch.stack([m[:, 0, 0], m[:, 0, 1], m[:, 0, 2], m[:, 1, 1], m[:, 1, 2], m[:, 2, 2]], dim=1)


def covariance_3d(scale: torch.Tensor, rot: torch.Tensor, scale_modifier: float = 1.0) -> torch.Tensor:
    """(N,6) packed 3-D covariances from activated scales and raw quaternions."""
    L = build_scaling_rotation(scale_modifier * scale, rot)
    return strip_symmetric(L @ L.transpose(1, 2))


def safe_state(silent: bool = False, seed: int = 0):
    """Seed every generator and stamp each line written to stdout with the time (``general_utils.py:113-133``);
    ``silent`` drops the output instead."""
    import sys
    from datetime import datetime
    real = sys.stdout

    class _Stamped:
        def write(self, text):
            if silent:
                return
            if text.endswith("\n"):
                real.write(text.replace("\n", " [{}]\n".format(datetime.now().strftime("%d/%m %H:%M:%S"))))
            else:
                real.write(text)

        def flush(self):
            real.flush()

    sys.stdout = _Stamped()
    seed_everything(seed)
    return real
