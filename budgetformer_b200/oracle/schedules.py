"""The two learning-rate schedules in closed form (utils/lr.py:5-52), as functions of the scheduler's step count."""
from __future__ import annotations

import math


def cosine_with_warmup(step: int, warmup: int, total: int, peak_lr: float) -> float:
    warmup = max(1, warmup)
    if step <= warmup:
        return peak_lr * step / warmup
    progress = (step - warmup) / max(1, total - warmup)
    return 0.5 * peak_lr * (1.0 + math.cos(math.pi * progress))       # not clamped: past `total` the cosine turns back up


def polynomial_decay(step: int, warmup: int, total: int, peak_lr: float, end_lr: float, power: float = 1.0) -> float:
    if step <= warmup:
        return peak_lr * step / float(warmup)
    if step >= total:
        return end_lr
    span = total - warmup
    remaining = 1.0 - (step - warmup) / span
    return (peak_lr - end_lr) * remaining ** power + end_lr
