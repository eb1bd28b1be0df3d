"""Edge-list attention as the reference computes it, in float32 on COO edges.

``edge_index[0]`` is the key/value node, ``edge_index[1]`` the query node
(models/gt_dist_node_level.py:224-262).  Shapes: ``q, k, v`` are ``[n, H, hn]``; the result is ``[n, H, hn]``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

CLAMP = 5.0
EPS = 1e-6


def _scatter_sum(values: torch.Tensor, index: torch.Tensor, n: int) -> torch.Tensor:
    out = torch.zeros((n,) + tuple(values.shape[1:]), dtype=values.dtype, device=values.device)
    return out.index_add_(0, index, values)


def edge_scores(q, k, edge_index, edge_factor: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``clamp(sum_d k[src] * q[dst] / sqrt(hn) [* E], -5, 5)`` per edge and head: ``[E, H]``."""
    src, dst = edge_index[0].long(), edge_index[1].long()
    prod = k.float()[src] * q.float()[dst] / math.sqrt(q.size(-1))
    if edge_factor is not None:
        prod = prod * edge_factor.float()
    return prod.sum(-1).clamp(-CLAMP, CLAMP)


def sparse_attention(q, k, v, edge_index, edge_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Graphormer / GT: ``out_i = sum_j w_ij v_j / (sum_j w_ij + 1e-6)`` with ``w = exp(score [+ bias])``; the bias is
    added after the clamp (models/graphormer_dist_node_level.py:231-263).  A query without in-edges gets zeros."""
    n = q.size(0)
    src, dst = edge_index[0].long(), edge_index[1].long()
    s = edge_scores(q, k, edge_index)
    if edge_bias is not None:
        s = s + edge_bias.float()
    w = torch.exp(s)
    z = _scatter_sum(w, dst, n)
    wv = _scatter_sum(w.unsqueeze(-1) * v.float()[src], dst, n)
    return wv / (z.unsqueeze(-1) + EPS)


def gps_attention(q, k, v, edge_index, keep: Optional[torch.Tensor] = None, dropout_p: float = 0.0) -> torch.Tensor:
    """GraphGPS: the weights are normalised per edge first, ``alpha = w / (Z[dst] + 1e-6)``, dropout acts on ``alpha``
    (``keep`` is the ``[E, H]`` boolean mask, rescaled by ``1 / (1 - p)``), then ``sum alpha v``
    (models/graphgps_dist_node_level.py:161-177)."""
    n = q.size(0)
    src, dst = edge_index[0].long(), edge_index[1].long()
    w = torch.exp(edge_scores(q, k, edge_index))
    z = _scatter_sum(w, dst, n)
    alpha = w / (z[dst] + EPS)
    if keep is not None and dropout_p > 0:
        alpha = alpha * keep.to(alpha.dtype) / (1.0 - dropout_p)
    return _scatter_sum(alpha.unsqueeze(-1) * v.float()[src], dst, n)


def exphormer_attention(q, k, v, edge_index, edge_type_emb: torch.Tensor, edge_proj_weight: torch.Tensor,
                        head_lo: int = 0, head_hi: Optional[int] = None) -> torch.Tensor:
    """Exphormer: ``E = edge_proj(edge_type_emb[type])`` reshaped ``[E, H_total, hn]`` and sliced to the heads
    ``[head_lo, head_hi)`` this rank owns; it multiplies ``k * q / sqrt(hn)`` element-wise before the sum over ``hn``
    (models/exphormer_dist_node_level.py:92-121).  ``edge_index`` carries the type in row 2."""
    n, h_local, hn = q.shape
    emb = edge_type_emb.float()[edge_index[2].long()]                     # [E, hidden]
    e_all = emb @ edge_proj_weight.float().t()                             # Linear without bias
    e_all = e_all.view(emb.size(0), -1, hn)
    head_hi = head_lo + h_local if head_hi is None else head_hi
    s = edge_scores(q, k, edge_index, e_all[:, head_lo:head_hi])
    src, dst = edge_index[0].long(), edge_index[1].long()
    w = torch.exp(s)
    z = _scatter_sum(w, dst, n)
    wv = _scatter_sum(w.unsqueeze(-1) * v.float()[src], dst, n)
    return wv / (z.unsqueeze(-1) + EPS)
