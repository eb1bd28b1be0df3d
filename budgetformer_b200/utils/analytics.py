"""Research analytics that ride along with training: attention mass per hop / per head and edge-set statistics.

* ``HopMassTracker`` / ``HeadMassStats`` restate the trackers the reference keeps inside its attention modules
  (models/gt_dist_node_level.py:75-139,264-429; models/graphormer_dist_node_level.py:102-151,340-507): how much
  normalised attention weight falls on keys at hop distance d from the query, how many hops are needed to collect a
  target share of it, and the mean attention mass per head.  ``write_hop_stats`` is the JSON dump of the legacy
  driver (main_node_sp.py:194-276).
* The edge-set helpers are the small analytics of gt_sp/utils.py (:548-617 ``slice_edge_index``,
  ``edge_index_new_edge_ratio``, ``edge_index_jaccard``; :2389-2515 ``calc_power_edge_index``,
  ``calculate_sparsity[_csr]``, ``make_strongly_connected``) on integer edge keys instead of Python sets.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch


# ----------------------------------------------------------------------------------------------- mass trackers
class HeadMassStats:
    """Running mean of the attention mass each local head puts on the given edges."""

    def __init__(self, num_heads: int):
        self.sum = torch.zeros(int(num_heads), dtype=torch.float32)
        self.count = torch.zeros(int(num_heads), dtype=torch.float32)

    def reset(self) -> None:
        self.sum.zero_()
        self.count.zero_()

    def add(self, weights: torch.Tensor) -> None:
        """``weights`` ``[E, H]`` normalised attention weights of one call."""
        if weights.numel():
            w = weights.detach().float().cpu()
            self.sum += w.sum(0)
            self.count += float(w.size(0))

    def mean(self) -> torch.Tensor:
        return self.sum / self.count.clamp_min(1.0)


class HopMassTracker:
    """Share of attention weight per hop distance, averaged over calls (``max_batches`` calls at most)."""

    def __init__(self, mass: float = 0.95, max_hop: int = 15, max_batches: int = 1):
        self.mass, self.max_hop, self.max_batches = float(mass), int(max_hop), int(max_batches)
        self.reset()

    def reset(self) -> None:
        self.hop_sum: List[float] = []
        self.calls = 0
        self.seen = 0
        self.hops_needed_sum = 0.0
        self.hops_needed_count = 0
        self.hops_needed_max = 0

    def add_sparse(self, dst: torch.Tensor, hops: torch.Tensor, weights: torch.Tensor) -> None:
        """One sparse attention call: per edge its query ``dst``, its hop distance (``< 0`` = unknown) and its
        normalised weight ``[E]`` or ``[E, H]`` (averaged over heads)."""
        if self.max_batches > 0 and self.seen >= self.max_batches:
            return
        self.seen += 1
        w = weights.detach().float()
        if w.dim() > 1:
            w = w.reshape(w.size(0), -1).mean(1)
        hops = hops.to(w.device).long()
        ok = hops >= 0
        if self.max_hop > 0:
            ok &= hops <= self.max_hop
        if not bool(ok.any()):
            return
        per_hop = torch.zeros(int(hops[ok].max()) + 1, dtype=torch.float32, device=w.device)
        per_hop.index_add_(0, hops[ok], w[ok])
        total = float(per_hop.sum())
        if total <= 0.0:
            return
        self._accumulate((per_hop / total).cpu())

    def add_dense(self, probs: torch.Tensor, hop_matrix: torch.Tensor) -> None:
        """One dense attention call: ``probs`` ``[Q, K]`` (already averaged over heads), ``hop_matrix`` ``[Q, K]``."""
        q, k = probs.shape
        dst = torch.arange(q, device=probs.device).repeat_interleave(k)
        self.add_sparse(dst, hop_matrix.reshape(-1), probs.reshape(-1))

    def _accumulate(self, share: torch.Tensor) -> None:
        if len(self.hop_sum) < share.numel():
            self.hop_sum.extend([0.0] * (share.numel() - len(self.hop_sum)))
        for i, v in enumerate(share.tolist()):
            self.hop_sum[i] += v
        self.calls += 1
        target = min(max(self.mass, 0.0), 1.0)
        if target > 0.0:
            hit = torch.nonzero(share.cumsum(0) >= target)
            if hit.numel():
                need = int(hit[0])
                self.hops_needed_sum += need
                self.hops_needed_count += 1
                self.hops_needed_max = max(self.hops_needed_max, need)

    def summary(self) -> Optional[Dict[str, object]]:
        if self.calls == 0:
            return None
        return {"hop_mass": [v / self.calls for v in self.hop_sum], "calls": self.calls,
                "hops_for_target_mean": self.hops_needed_sum / max(1, self.hops_needed_count),
                "hops_for_target_max": self.hops_needed_max, "target": self.mass}


def hop_stats_dirname(args) -> str:
    name = f"attn{float(getattr(args, 'full_attn_hop_mass', 0.95)):g}_maxhop{int(getattr(args, 'full_attn_hop_max_hop', 64))}"
    tag = str(getattr(args, "full_attn_hop_stats_tag", "") or "").strip()
    return f"{name}_{tag}" if tag else name


def write_hop_stats(args, epoch: int, per_layer: List[Optional[Dict[str, object]]]) -> str:
    """``<stats_dir>/<dataset>/<model>/<dirname>/epoch_<e>.json`` with the tracker settings and one entry per layer."""
    root = os.path.join(str(getattr(args, "full_attn_hop_stats_dir", "./plot/hop_stats")), str(getattr(args, "dataset", "data")),
                        str(getattr(args, "model", "model")), hop_stats_dirname(args))
    os.makedirs(root, exist_ok=True)
    path = os.path.join(root, f"epoch_{int(epoch)}.json")
    payload = {"epoch": int(epoch), "mass": float(getattr(args, "full_attn_hop_mass", 0.95)),
               "max_queries": int(getattr(args, "full_attn_hop_max_queries", 64)),
               "query_sampling": str(getattr(args, "full_attn_hop_query_sampling", "random")),
               "max_batches": int(getattr(args, "full_attn_hop_max_batches", 1)),
               "max_hop_limit": int(getattr(args, "full_attn_hop_max_hop", 64)), "layers": per_layer}
    with open(path, "w") as f:
        json.dump(payload, f)
    return path


def bfs_hop_matrix(edge_index: torch.Tensor, num_nodes: int, queries: torch.Tensor, max_hop: int = 64) -> torch.Tensor:
    """Hop distance from every query to every node along in-edges (``-1`` = unreachable within ``max_hop``)."""
    n = int(num_nodes)
    adj = torch.zeros(n, n, dtype=torch.bool)
    adj[edge_index[1].long(), edge_index[0].long()] = True         # row = query side, col = key side
    dist = torch.full((queries.numel(), n), -1, dtype=torch.long)
    frontier = torch.zeros(queries.numel(), n, dtype=torch.bool)
    frontier[torch.arange(queries.numel()), queries.long()] = True
    dist[frontier] = 0
    limit = max_hop if max_hop > 0 else n
    for d in range(1, limit + 1):
        nxt = (frontier.float() @ adj.float()) > 0
        nxt &= dist < 0
        if not bool(nxt.any()):
            break
        dist[nxt] = d
        frontier = nxt
    return dist


# ----------------------------------------------------------------------------------------------- edge-set statistics
def edge_ids(edge_index: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """Sorted unique int64 key ``src * n + dst`` of every edge."""
    return torch.unique(edge_index[0].long() * int(num_nodes) + edge_index[1].long())


def slice_edge_index(edge_index: torch.Tensor, start: int, end: int) -> torch.Tensor:
    """Edges with both endpoints in ``[start, end)``, re-based to 0."""
    s, d = edge_index[0], edge_index[1]
    keep = (s >= start) & (s < end) & (d >= start) & (d < end)
    return edge_index[:, keep] - int(start)


def edge_index_new_edge_ratio(previous: torch.Tensor, current: torch.Tensor, num_nodes: int) -> float:
    """Fraction of the current edge set that was not in the previous one."""
    cur = edge_ids(current, num_nodes)
    if cur.numel() == 0:
        return 0.0
    old = edge_ids(previous, num_nodes)
    return float((~torch.isin(cur, old)).sum()) / float(cur.numel())


def edge_index_jaccard(a: torch.Tensor, b: torch.Tensor, num_nodes: int) -> float:
    ia, ib = edge_ids(a, num_nodes), edge_ids(b, num_nodes)
    inter = int(torch.isin(ia, ib).sum())
    union = ia.numel() + ib.numel() - inter
    return 1.0 if union == 0 else inter / union


def calculate_sparsity(edge_index: torch.Tensor, num_nodes: int) -> float:
    """Share of the ``n x n`` attention matrix that is empty."""
    n = int(num_nodes)
    return 1.0 - edge_ids(edge_index, n).numel() / float(n * n) if n else 0.0


def calculate_sparsity_csr(rowptr: torch.Tensor, num_nodes: int) -> float:
    n = int(num_nodes)
    return 1.0 - float(rowptr[-1]) / float(n * n) if n else 0.0


def calc_power_edge_index(edge_index: torch.Tensor, num_nodes: int, power: int) -> torch.Tensor:
    """Edges of ``A + A^2 + ... + A^power`` (reachability within ``power`` steps), without self loops."""
    n = int(num_nodes)
    a = torch.sparse_coo_tensor(edge_index.long(), torch.ones(edge_index.size(1)), (n, n)).coalesce()
    reach, cur = a, a
    for _ in range(max(0, int(power) - 1)):
        cur = torch.sparse.mm(cur, a).coalesce()
        reach = (reach + cur).coalesce()
    idx = reach.indices()
    return idx[:, idx[0] != idx[1]]


def make_strongly_connected(edge_index: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """Adds the ring ``i -> (i + 1) mod n`` so that every node reaches every other (duplicates removed)."""
    n = int(num_nodes)
    ring = torch.stack([torch.arange(n), (torch.arange(n) + 1) % n]).to(edge_index)
    keys = edge_ids(torch.cat([edge_index, ring], 1), n)
    return torch.stack([keys // n, keys % n]).to(edge_index.dtype)
