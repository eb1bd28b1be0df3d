"""Dataset loading and CPU-side preprocessing.

Data contract (utils/fullgraph_sp_support.py:637-642): ``<dataset_dir>/<dataset>/x.pt`` float
``[N, d]``, ``y.pt`` int ``[N]`` (or ``[N, C]`` multi-hot with ``--multilabel``), ``edge_index.pt`` int64
``[2, E]``; optional split files (``utils/split_utils.py``), else a seeded random 60/20/20 split
(gt_sp/utils.py:746-758)."""
from __future__ import annotations

import os
import random
import time
from dataclasses import dataclass, replace
from typing import Optional
import numpy as np
import torch

from ..utils.split_utils import load_default_split, safe_torch_load


@dataclass
class GraphData:
    x: torch.Tensor
    y: torch.Tensor
    edge_index: torch.Tensor
    split_idx: dict
    num_nodes: int          # before padding
    output_dim: int
    multilabel: bool = False
    node_order: Optional[torch.Tensor] = None   # set by reorder_for_locality: original id of every (new) node id


def random_split_idx(num_nodes: int, seed: int, frac_train: float = 0.6, frac_valid: float = 0.2) -> dict:
    """Python ``random.shuffle`` under ``seed``, 60/20/20 (gt_sp/utils.py:746-758)."""
    rnd = random.Random(int(seed))
    idx = list(range(int(num_nodes)))
    rnd.shuffle(idx)
    n_tr, n_va = int(frac_train * num_nodes), int(frac_valid * num_nodes)
    return {"train": torch.tensor(idx[:n_tr], dtype=torch.long),
            "valid": torch.tensor(idx[n_tr:n_tr + n_va], dtype=torch.long),
            "test": torch.tensor(idx[n_tr + n_va:], dtype=torch.long)}


def to_bidirected_edge_index(edge_index: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """Union of the graph and its reverse, duplicates removed (utils/fullgraph_sp_support.py:570-573)."""
    ei = torch.cat([edge_index, edge_index.flip(0)], dim=1).to(torch.int64)
    key = torch.unique(ei[0] * int(num_nodes) + ei[1])
    return torch.stack([torch.div(key, int(num_nodes), rounding_mode="floor"), key % int(num_nodes)], 0)


def sample_induced_subgraph(x, y, edge_index, split_idx, ratio: float, seed: int):
    """``--node_sample_ratio``: keep a uniform node sample and its induced subgraph."""
    n = x.size(0)
    g = torch.Generator().manual_seed(int(seed))
    keep = torch.randperm(n, generator=g)[: max(1, int(round(n * ratio)))].sort().values
    remap = torch.full((n,), -1, dtype=torch.long)
    remap[keep] = torch.arange(keep.numel())
    m = (remap[edge_index[0]] >= 0) & (remap[edge_index[1]] >= 0)
    ei = torch.stack([remap[edge_index[0][m]], remap[edge_index[1][m]]], 0)
    split = None
    if split_idx is not None:
        split = {k: remap[v][remap[v] >= 0] for k, v in split_idx.items()}
    return x[keep], y[keep], ei, split


def load_data(args, dist_module=None) -> GraphData:
    root = os.path.join(args.dataset_dir, args.dataset)
    x = safe_torch_load(os.path.join(root, "x.pt"), mmap=True).float()      # no copy when already fp32
    y = safe_torch_load(os.path.join(root, "y.pt"), mmap=True)
    edge_index = safe_torch_load(os.path.join(root, "edge_index.pt"), mmap=True).to(torch.int64)
    multilabel = bool(getattr(args, "multilabel", False)) or (y.dim() == 2 and y.size(1) > 1)
    if not multilabel:
        y = y.reshape(-1).to(torch.long)
    n = x.size(0)
    split = None
    if not getattr(args, "force_random_split", False):
        split = load_default_split(args.dataset, args.dataset_dir, dist_module, wait_for_rank0=True,
                                   split_id=int(getattr(args, "split_id", 0)))
    if getattr(args, "to_bidirected", False):
        edge_index = to_bidirected_edge_index(edge_index, n)
    ratio = float(getattr(args, "node_sample_ratio", 1.0))
    if ratio < 1.0:
        x, y, edge_index, split = sample_induced_subgraph(x, y, edge_index, split, ratio, args.seed)
        n = x.size(0)
    if split is None:
        split = random_split_idx(n, args.seed)
    out_dim = int(y.size(1)) if multilabel else int(y.max().item()) + 1
    data = GraphData(x, y, edge_index, split, n, out_dim, multilabel)
    parts = int(getattr(args, "locality_reorder_parts", 0) or 0)
    return reorder_for_locality(data, parts) if parts > 1 else data


def reorder_for_locality(data: GraphData, parts: int, imbalance: float = 0.03) -> GraphData:
    """``--locality_reorder_parts K``: relabel the nodes once, at load time, so that each of K clusters of the
    multilevel partition (graph/partition.py) owns a contiguous id range.  Neighbours then sit close together in the
    feature / key / value matrices, which is what the edge-attention gathers read; the model sees an isomorphic
    graph, so accuracy is unaffected (the sampled attention edges differ, since their hash ranks node ids).
    ``node_order[new] = old`` maps results back."""
    from ..graph.partition import partition_assignment
    n = int(data.num_nodes)
    part = partition_assignment(data.edge_index, n, int(parts), imbalance)
    old_of_new = torch.argsort(part, stable=True)
    new_of_old = torch.empty(n, dtype=torch.long)
    new_of_old[old_of_new] = torch.arange(n, dtype=torch.long)
    tail = torch.arange(n, data.x.size(0), dtype=torch.long)           # padding rows (if any) stay at the end
    rows = torch.cat([old_of_new, tail])
    split = {k: new_of_old[v.long()] for k, v in data.split_idx.items()} if data.split_idx is not None else None
    return replace(data, x=data.x[rows], y=data.y[rows], edge_index=new_of_old[data.edge_index.long()], split_idx=split,
                   node_order=old_of_new)


def pad_to_sequence_parallel_world(data: GraphData, world: int) -> GraphData:
    """Pad N to a multiple of P with zero feature rows and label -1 (utils/fullgraph_sp_runtime.py:819-826)."""
    n = data.x.size(0)
    pad = (-n) % max(1, int(world))
    if pad == 0:
        return data
    x = torch.cat([data.x, data.x.new_zeros((pad,) + tuple(data.x.shape[1:]))], 0)
    if data.multilabel:
        y = torch.cat([data.y, data.y.new_zeros((pad, data.y.size(1)))], 0)
    else:
        y = torch.cat([data.y, data.y.new_full((pad,), -1)], 0)
    return replace(data, x=x, y=y)


def _bidirected_self_loop_coo(edge_index: torch.Tensor, n: int):
    ei = to_bidirected_edge_index(edge_index.cpu(), n)
    self_nodes = torch.arange(n, dtype=torch.long)
    return torch.cat([ei[0], self_nodes]), torch.cat([ei[1], self_nodes])


def compute_laplacian_pe(row: torch.Tensor, col: torch.Tensor, num_nodes: int, pe_dim: int) -> torch.Tensor:
    """Eigenvectors 1..pe_dim of I - D^-1/2 A D^-1/2 on the unweighted structure
    (utils/fullgraph_sp_support.py:69-106: scipy ``eigs(which="SR", tol=1e-2)`` with a dense fallback)."""
    import scipy.sparse as sp
    from scipy.sparse.linalg import eigs

    n = int(num_nodes)
    a = sp.csr_matrix((np.ones(row.numel()), (row.numpy(), col.numpy())), shape=(n, n))
    a.data[:] = 1.0
    deg = np.asarray(a.sum(axis=0)).reshape(-1).clip(1)
    d = sp.diags(deg ** -0.5)
    lap = sp.eye(n, format="csr") - d @ a @ d
    try:
        val, vec = eigs(lap, k=pe_dim + 1, which="SR", tol=1e-2)
    except Exception:
        val, vec = np.linalg.eigh(lap.toarray())
        val, vec = val[: pe_dim + 1], vec[:, : pe_dim + 1]
    vec = vec[:, val.real.argsort()]
    return torch.from_numpy(np.ascontiguousarray(vec[:, 1:pe_dim + 1].real)).float()


def compute_multihop_features(edge_index, num_nodes: int, features: torch.Tensor, hops: int, pe_dim: int = 0,
                              rank: int = 0) -> torch.Tensor:
    """``[N, hops+1, d+pe_dim]``: h_0 = [x | PE], h_k = D^-1/2 (A_bi + I) D^-1/2 h_{k-1}
    (utils/fullgraph_sp_support.py:109-190)."""
    t0 = time.time()
    n = int(num_nodes)
    row, col = _bidirected_self_loop_coo(edge_index, n)
    x = features.float().cpu()[:n]
    if pe_dim > 0:
        x = torch.cat([x, compute_laplacian_pe(row, col, n, pe_dim)], dim=1)
    deg = torch.bincount(col, minlength=n).float()
    dis = deg.pow(-0.5)
    dis[torch.isinf(dis)] = 0.0
    adj = torch.sparse_coo_tensor(torch.stack([row, col]), dis[row] * dis[col], (n, n)).coalesce()
    feats = [x]
    for _ in range(int(hops)):
        x = torch.sparse.mm(adj, x)
        feats.append(x)
    out = torch.stack(feats, dim=1)
    if rank == 0:
        print(f"[nagphormer] {hops}-hop features ready in {time.time() - t0:.2f}s "
              f"({out.numel() * 4 / 2**20:.1f} MiB)")
    return out


def preprocess_hop_features(args, data: GraphData, rank: int = 0) -> GraphData:
    """``--hops/--pe_dim`` for Graphormer/GT: concatenate the hop stack into ``(hops+1)*(d+pe)`` input features
    (utils/fullgraph_sp_runtime.py:829-860).  NAGphormer keeps the same flattened layout and un-flattens it."""
    hops, pe = int(getattr(args, "hops", 0)), int(getattr(args, "pe_dim", 0))
    if hops <= 0 and pe <= 0:
        return data
    n_pad = data.x.size(0)
    mh = compute_multihop_features(data.edge_index, data.num_nodes, data.x, max(hops, 0), pe, rank)
    flat = mh.reshape(mh.size(0), -1)
    if n_pad > flat.size(0):
        flat = torch.cat([flat, flat.new_zeros(n_pad - flat.size(0), flat.size(1))], 0)
    return replace(data, x=flat)


def generate_expander_edges(num_nodes: int, degree: int, seed: int = 0) -> torch.Tensor:
    """``degree`` random Hamiltonian cycles, both directions, self loops removed
    (utils/fullgraph_sp_support.py:193-215)."""
    rng = np.random.default_rng(int(seed))
    src, dst = [], []
    for _ in range(int(degree)):
        perm = rng.permutation(int(num_nodes))
        prev = np.roll(perm, 1)
        src.append(np.stack([perm, prev], 1).reshape(-1))
        dst.append(np.stack([prev, perm], 1).reshape(-1))
    row = torch.from_numpy(np.concatenate(src)).long()
    col = torch.from_numpy(np.concatenate(dst)).long()
    m = row != col
    return torch.stack([row[m], col[m]], 0)
