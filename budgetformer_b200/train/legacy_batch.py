"""Mini-batch sequence-parallel batching (legacy mode of the reference's ``main_node_sp.py``).

The node set is cut into sequences of ``--seq_len`` nodes; each step trains on one sequence whose rows are sharded
over the SP ranks.  The attention graph of a step is the subgraph induced by the sequence
(``--batch_subgraph_mode induced``) or by the sequence's seeds plus the nodes their random walks visit
(``seed_rw``); restates ``get_batch_blockize`` / ``sample_seed_rw_subgraph`` / ``_compute_local_spd_bias``
(gt_sp/utils.py:1669-1966, :939-1010, :64-110) on the CSR containers of this package.  ``--batch_reorder_parts k``
(``get_batch_reorder_blockize``, gt_sp/utils.py:1969-2090) first reorders the sequence so that each of k locality
clusters is contiguous, which keeps most attention edges inside one rank's rows."""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..graph.attn_graph import AttnGraph, Topology, add_virtual_node
from ..graph.builder_spec import random_walks
from ..parallel.initialize import set_global_token_indices


def induced_subgraph(edge_index: torch.Tensor, idx: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """Edges with both endpoints in ``idx``, relabelled to positions in ``idx`` (PyG ``subgraph(relabel_nodes=True)``)."""
    remap = torch.full((int(num_nodes),), -1, dtype=torch.long)
    remap[idx] = torch.arange(idx.numel())
    s, d = remap[edge_index[0]], remap[edge_index[1]]
    m = (s >= 0) & (d >= 0)
    return torch.stack([s[m], d[m]], 0)


def map_global_nodes_to_local(nodes_global: torch.Tensor, sampled_nodes: torch.Tensor) -> torch.Tensor:
    """Position in ``sampled_nodes`` of every id of ``nodes_global`` (which must all be sampled) by binary search over
    the sorted sample: no table of the size of the whole graph is needed (gt_sp/utils.py:939-948)."""
    sample, ids = sampled_nodes.long(), nodes_global.long()
    if ids.numel() == 0:
        return torch.empty(0, dtype=torch.long, device=sample.device)
    ordered, order = torch.sort(sample)
    pos = torch.searchsorted(ordered, ids).clamp_(max=max(int(ordered.numel()) - 1, 0))
    return order[pos]


def reorder_by_partition(edge_index: torch.Tensor, idx: torch.Tensor, num_nodes: int, k: int) -> torch.Tensor:
    """``idx`` permuted so that the k parts of its induced subgraph are contiguous.  The partitioner is
    deterministic, so every rank computes the same order and nothing is broadcast."""
    from ..graph.partition import reformat_graph
    sub = induced_subgraph(edge_index, idx, num_nodes)
    _edges, old_of_new = reformat_graph(sub, k, num_nodes=int(idx.numel()))
    return idx[old_of_new]


def sample_seed_rw_subgraph(topo: Topology, seeds: torch.Tensor, walk_length: int, walks_per_node: int, seed: int,
                            max_nodes: Optional[int] = None) -> torch.Tensor:
    """Seeds first, then the distinct nodes visited by their walks (truncated to ``max_nodes``)."""
    walks = random_walks(topo, walks_per_node, walk_length, seed)
    w = max(1, int(walks_per_node))
    rows = (seeds.numpy()[:, None] * w + np.arange(w)[None, :]).reshape(-1)
    visited = np.unique(walks[rows].reshape(-1))
    extra = np.setdiff1d(visited, seeds.numpy(), assume_unique=False)
    nodes = torch.cat([seeds, torch.from_numpy(extra).long()])
    return nodes[:max_nodes] if max_nodes else nodes


def compute_local_spd_bias(edge_index: torch.Tensor, n: int, max_dist: int) -> torch.Tensor:
    """One-hot shortest-path-distance bias ``[n, n, max_dist + 1]`` of the batch subgraph (distances clamped)."""
    from scipy.sparse import csr_matrix
    from scipy.sparse.csgraph import shortest_path

    a = csr_matrix((np.ones(edge_index.size(1)), (edge_index[0].numpy(), edge_index[1].numpy())), shape=(n, n))
    dist = shortest_path(a, directed=False, unweighted=True)
    dist = np.where(np.isinf(dist), max_dist, dist).clip(0, max_dist).astype(np.int64)
    return torch.nn.functional.one_hot(torch.from_numpy(dist), max_dist + 1).float()


def get_batch_blockize(args, feature: torch.Tensor, y: torch.Tensor, idx_batch: torch.Tensor, edge_index_global: torch.Tensor,
                       num_nodes: int, sp_rank: int, sp_world: int, topo: Optional[Topology] = None, epoch_seed: int = 0,
                       ) -> Tuple[torch.Tensor, torch.Tensor, AttnGraph, Optional[torch.Tensor], torch.Tensor]:
    """Returns (x_local, y_local, attention graph over the whole sequence, attn_bias rows of this rank or None,
    mask of local rows that carry a label to train on)."""
    mode = getattr(args, "batch_subgraph_mode", "induced")
    seeds = idx_batch
    if mode == "seed_rw":
        assert topo is not None
        nodes = sample_seed_rw_subgraph(topo, seeds, int(args.walk_length), int(args.walks_per_node), epoch_seed,
                                        max_nodes=int(args.seq_len) if int(args.seq_len) > 0 else None)
    else:
        nodes = seeds
        parts = int(getattr(args, "batch_reorder_parts", 0) or 0)
        if parts > 1 and nodes.numel() > parts:
            nodes = reorder_by_partition(edge_index_global, nodes, num_nodes, parts)
    n = int(nodes.numel())
    pad = (-n) % max(1, sp_world)
    ei = induced_subgraph(edge_index_global, nodes, num_nodes)
    loops = torch.arange(n)
    ei = torch.cat([ei, torch.stack([loops, loops])], 1)              # every query attends at least to itself
    n_pad = n + pad
    s = n_pad // sp_world
    graph = AttnGraph.from_edge_index(ei, n_pad)
    virtual = str(args.model) == "graphormer" and int(getattr(args, "num_global_node", 0)) > 0
    if virtual:
        graph = add_virtual_node(graph, n_pad, s)
        set_global_token_indices([r * (s + 1) for r in range(sp_world)])
    else:
        set_global_token_indices(None)
    x = feature[nodes]
    yy = y[nodes]
    label_ok = torch.zeros(n_pad, dtype=torch.bool)
    label_ok[: seeds.numel()] = True                                   # only the seeds carry a training label
    if pad:
        x = torch.cat([x, x.new_zeros(pad, x.size(1))], 0)
        yy = torch.cat([yy, yy.new_full((pad,), -1)], 0)
    sl = slice(sp_rank * s, (sp_rank + 1) * s)
    attn_bias = None
    if getattr(args, "attn_bias_mode", "none") == "local_spd":
        attn_bias = compute_local_spd_bias(ei, n_pad, int(args.attn_bias_max_dist))[sl]
    return x[sl], yy[sl], graph, attn_bias, label_ok[sl]


def get_batch_reorder_blockize(args, feature, y, idx_batch, edge_index_global, num_nodes, sp_rank, sp_world, k: int = 0,
                               topo: Optional[Topology] = None, epoch_seed: int = 0):
    """``get_batch_blockize`` on the sequence reordered into ``k`` locality clusters (``k <= 1``: unchanged order)."""
    import copy
    a = copy.copy(args)
    a.batch_reorder_parts = int(k)
    a.batch_subgraph_mode = "induced"
    return get_batch_blockize(a, feature, y, idx_batch, edge_index_global, num_nodes, sp_rank, sp_world, topo=topo,
                              epoch_seed=epoch_seed)
