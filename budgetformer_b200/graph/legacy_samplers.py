"""Per-batch subgraph samplers and per-head edge views of the legacy mini-batch path.

Counterparts of ``SubgraphSampler`` / ``IdentitySubgraphSampler`` / ``EdgeDropSubgraphSampler`` and of the
``HeadSubgraphProvider`` family with their two factories (gt_sp/utils.py:1539-1667 in the reference).  Here a head
view is described by one rule - "head h reads edge set ``assign[h]``" - and the three providers only differ in how
the edge sets and the assignment are made; grouping edges by source id is a vectorised mask instead of a Python loop
over edges.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

Edges = Union[torch.Tensor, Sequence[Optional[torch.Tensor]]]


class SubgraphSampler:
    """Maps (edge_index of the batch, seed nodes, node count) to the edge_index attention should use."""

    def sample(self, edge_index: torch.Tensor, seed_nodes: torch.Tensor, num_nodes: int) -> torch.Tensor:
        raise NotImplementedError


class IdentitySubgraphSampler(SubgraphSampler):
    def sample(self, edge_index, seed_nodes, num_nodes):
        return edge_index


class EdgeDropSubgraphSampler(SubgraphSampler):
    """Keeps each edge with probability ``1 - drop_ratio``; never returns an empty graph."""

    def __init__(self, drop_ratio: float, generator: Optional[torch.Generator] = None):
        self.drop_ratio = min(1.0, max(0.0, float(drop_ratio)))
        self.generator = generator

    def sample(self, edge_index, seed_nodes, num_nodes):
        if self.drop_ratio <= 0.0 or edge_index.numel() == 0:
            return edge_index
        u = torch.rand(edge_index.size(1), device=edge_index.device, generator=self.generator)
        keep = u > self.drop_ratio
        return edge_index[:, keep] if bool(keep.any()) else edge_index


def _first(edges: Edges) -> torch.Tensor:
    if isinstance(edges, (list, tuple)):
        for e in edges:
            if e is not None:
                return e
        raise ValueError("no edge set given")
    return edges


def _head_to_group(num_heads: int, groups: int) -> List[int]:
    """Consecutive heads share a group: ceil(num_heads / groups) heads per group."""
    per = -(-num_heads // groups)
    return [min(h // per, groups - 1) for h in range(num_heads)]


class HeadSubgraphProvider:
    """``build(edges, num_heads)`` returns one edge_index per head."""

    def build(self, edges: Edges, num_heads: int) -> List[torch.Tensor]:
        raise NotImplementedError


class SharedHeadSubgraphProvider(HeadSubgraphProvider):
    def build(self, edges, num_heads):
        e = _first(edges)
        return [e] * num_heads


class GroupedHeadSubgraphProvider(HeadSubgraphProvider):
    """Edges are partitioned by ``src % groups``; the heads of group g attend over partition g."""

    def __init__(self, num_groups: int):
        self.num_groups = max(1, int(num_groups))

    def build(self, edges, num_heads):
        e = _first(edges)
        if e.numel() == 0:
            return [e] * num_heads
        groups = min(self.num_groups, num_heads)
        part = e[0].to(torch.long) % groups
        sets = [e[:, part == g] for g in range(groups)]
        return [sets[g] for g in _head_to_group(num_heads, groups)]


class HopMappedHeadSubgraphProvider(HeadSubgraphProvider):
    """Head group g attends over hop bucket ``hop_sequence[g % len]`` (missing or empty buckets fall back to bucket 0)."""

    def __init__(self, hop_sequence: Sequence[int], num_groups: int):
        self.hop_sequence = [int(h) for h in hop_sequence] or [0]
        self.num_groups = max(1, int(num_groups))

    def build(self, edges, num_heads):
        if not isinstance(edges, (list, tuple)) or len(edges) == 0:
            return [edges] * num_heads
        groups = min(self.num_groups, num_heads)
        sets = []
        for g in range(groups):
            hop = self.hop_sequence[g % len(self.hop_sequence)]
            bucket = edges[hop] if hop < len(edges) else None
            sets.append(bucket if bucket is not None else edges[0])
        return [sets[g] for g in _head_to_group(num_heads, groups)]


def build_subgraph_sampler(args) -> SubgraphSampler:
    if str(getattr(args, "subgraph_sampler", "identity")) == "edge_drop":
        return EdgeDropSubgraphSampler(float(getattr(args, "edge_drop_ratio", 0.0)))
    return IdentitySubgraphSampler()


def build_head_subgraph_provider(args) -> HeadSubgraphProvider:
    groups = max(1, int(getattr(args, "head_groups", 4)))
    kind = str(getattr(args, "head_subgraph_provider", "hop"))
    if kind == "hop":
        return HopMappedHeadSubgraphProvider(list(range(groups)), groups)
    if kind == "grouped":
        return GroupedHeadSubgraphProvider(groups)
    return SharedHeadSubgraphProvider()
