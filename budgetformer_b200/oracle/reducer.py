"""Gradient averaging and the per-rank loss rule (gt_sp/reducer.py:120-146, main_node_fullgraph_sp.py:1233-1239)."""
from __future__ import annotations

from typing import Sequence

import torch


def mean_of_rank_gradients(per_rank: Sequence[torch.Tensor]) -> torch.Tensor:
    """Each rank divides its gradient by the world size, then the ranks are summed."""
    p = float(len(per_rank))
    out = torch.zeros_like(per_rank[0], dtype=torch.float32)
    for g in per_rank:
        out += g.float() / p
    return out


def rank_loss(log_probs: torch.Tensor, labels: torch.Tensor, local_train_idx: torch.Tensor) -> torch.Tensor:
    """Mean negative log-likelihood over the rank's own training rows; a rank without any contributes a zero that
    still depends on the output (so that every collective of the backward pass runs)."""
    if local_train_idx.numel() == 0:
        return log_probs.sum() * 0
    return -log_probs.float()[local_train_idx, labels[local_train_idx]].mean()
