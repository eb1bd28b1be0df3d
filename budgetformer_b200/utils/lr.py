"""Learning-rate schedules keyed on the scheduler's step count (one step = one epoch in full-graph
mode).  Same curves as the reference's ``utils/lr.py``: linear warm-up then cosine to zero
(:5-23) or polynomial decay to ``end_lr`` (:26-52), written as ``LambdaLR``-free closed forms."""
from __future__ import annotations

import math

from torch.optim.lr_scheduler import LRScheduler


def cosine_with_warmup_value(step: int, warmup: int, tot: int, lr: float) -> float:
    warmup = max(1, warmup)
    if step <= warmup:
        return lr * step / float(warmup)
    progress = (step - warmup) / max(1, tot - warmup)
    return lr * 0.5 * (1.0 + math.cos(math.pi * progress))


def polynomial_decay_value(step: int, warmup: int, tot: int, lr: float, end_lr: float, power: float) -> float:
    if step <= warmup:
        return lr * step / float(warmup)
    if step >= tot:
        return end_lr
    remaining = 1 - (step - warmup) / (tot - warmup)
    return (lr - end_lr) * remaining ** power + end_lr


class CosineWithWarmupLR(LRScheduler):
    def __init__(self, optimizer, warmup, tot, lr, last_epoch=-1):
        self.warmup, self.tot, self.lr = max(1, warmup), tot, lr
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        v = cosine_with_warmup_value(self._step_count, self.warmup, self.tot, self.lr)
        return [v for _ in self.optimizer.param_groups]


class PolynomialDecayLR(LRScheduler):
    def __init__(self, optimizer, warmup, tot, lr, end_lr, power, last_epoch=-1):
        self.warmup, self.tot, self.lr, self.end_lr, self.power = warmup, tot, lr, end_lr, power
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        v = polynomial_decay_value(self._step_count, self.warmup, self.tot, self.lr, self.end_lr, self.power)
        return [v for _ in self.optimizer.param_groups]


def schedule_epochs(args, n_train=None):
    """(warmup_epochs, total_epochs): ``--tot_updates > 0`` rescales mini-batch step counts into epochs
    using ``ceil(n_train / lr_ref_batch_size)`` (utils/fullgraph_sp_support.py:2368-2375)."""
    warm, tot = int(args.warmup_updates), int(args.epochs)
    tot_updates = int(getattr(args, "tot_updates", 0) or 0)
    if tot_updates > 0 and n_train:
        ref = max(1, int(getattr(args, "lr_ref_batch_size", 1000)))
        per_epoch = max(1, (int(n_train) + ref - 1) // ref)
        warm = max(1, round(args.warmup_updates / per_epoch))
        tot = max(warm + 1, round(tot_updates / per_epoch))
    return warm, tot


def build_lr_scheduler(args, optimizer, n_train=None):
    warm, tot = schedule_epochs(args, n_train)
    if getattr(args, "lr_schedule", "polynomial") == "cosine_with_warmup":
        return CosineWithWarmupLR(optimizer, warmup=warm, tot=tot, lr=args.peak_lr)
    return PolynomialDecayLR(optimizer, warmup=warm, tot=tot, lr=args.peak_lr, end_lr=args.end_lr, power=1.0)
