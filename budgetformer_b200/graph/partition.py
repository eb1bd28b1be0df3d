"""Locality reordering of the legacy mini-batch path: k-way partition, contiguous ids per part, induced subgraphs.

``reformat_graph(edge_index, k)`` has the return contract of the reference (gt_sp/utils.py:787-819: edges relabelled
and sorted by new source id, plus the old node ids in new order), and ``gen_sub_edge_index`` that of
gt_sp/utils.py:761-773 (edges among the nodes of one batch, relabelled to positions in the batch).  The reference
gets its partition from METIS through DGL; here it comes from the native multilevel partitioner
(csrc/cpu/partition.cpp: heavy-edge-matching coarsening, breadth-first initial partition of the coarsest graph,
balance-constrained boundary refinement at every level), with a SciPy reverse-Cuthill-McKee ordering as the stand-in
when the extension is not built.
"""
from __future__ import annotations

from typing import Tuple

import torch


def symmetric_csr(edge_index: torch.Tensor, num_nodes: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """int32 CPU CSR of the undirected, de-duplicated graph without self loops."""
    n = int(num_nodes)
    s, d = edge_index[0].long().cpu(), edge_index[1].long().cpu()
    keep = s != d
    s, d = s[keep], d[keep]
    keys = torch.unique(torch.cat([s * n + d, d * n + s]))
    row, col = keys // n, keys % n
    rowptr = torch.zeros(n + 1, dtype=torch.int64)
    rowptr[1:] = torch.cumsum(torch.bincount(row, minlength=n), 0)
    return rowptr.to(torch.int32).contiguous(), col.to(torch.int32).contiguous()


def partition_assignment(edge_index: torch.Tensor, num_nodes: int, k: int, imbalance: float = 0.03,
                         refine_passes: int = 8) -> torch.Tensor:
    """Part id ``[num_nodes]`` (int64) of a balanced k-way partition that keeps neighbours together."""
    n, k = int(num_nodes), max(1, min(int(k), max(1, int(num_nodes))))
    if n == 0:
        return torch.zeros(0, dtype=torch.long)
    rowptr, col = symmetric_csr(edge_index, n)
    from ..ops import _ext
    if _ext.available():
        part, _moved = _ext.load().partition_cpu(rowptr, col, n, k, float(imbalance), int(refine_passes))
        return part.long()
    return _rcm_ranges(rowptr, col, n, k)


def _rcm_ranges(rowptr: torch.Tensor, col: torch.Tensor, n: int, k: int) -> torch.Tensor:
    import numpy as np
    from scipy.sparse import csr_matrix
    from scipy.sparse.csgraph import reverse_cuthill_mckee
    a = csr_matrix((np.ones(col.numel(), dtype=np.int8), col.numpy(), rowptr.numpy()), shape=(n, n))
    order = torch.from_numpy(np.ascontiguousarray(reverse_cuthill_mckee(a, symmetric_mode=True)).astype(np.int64))
    part = torch.empty(n, dtype=torch.long)
    part[order] = (torch.arange(n, dtype=torch.long) * k) // n
    return part


def edge_cut(edge_index: torch.Tensor, part: torch.Tensor) -> int:
    """Number of directed edges whose endpoints lie in different parts."""
    return int((part[edge_index[0].long()] != part[edge_index[1].long()]).sum())


def reformat_graph(edge_index: torch.Tensor, k: int, num_nodes: int = None, imbalance: float = 0.03,
                   refine_passes: int = 8) -> Tuple[torch.Tensor, torch.Tensor]:
    """Relabel nodes so that part p owns a contiguous id range (parts in ascending order, old order kept inside a
    part).  Returns ``(edge_index in new ids sorted by source, old id of every new id)``."""
    n = int(num_nodes) if num_nodes is not None else (int(edge_index.max()) + 1 if edge_index.numel() else 0)
    part = partition_assignment(edge_index, n, k, imbalance, refine_passes)
    old_of_new = torch.argsort(part, stable=True)                    # new id -> old id
    new_of_old = torch.empty(n, dtype=torch.long)
    new_of_old[old_of_new] = torch.arange(n, dtype=torch.long)
    src, dst = new_of_old[edge_index[0].long().cpu()], new_of_old[edge_index[1].long().cpu()]
    by_src = torch.argsort(src, stable=True)
    return torch.stack([src[by_src], dst[by_src]]), old_of_new


def gen_sub_edge_index(edge_index: torch.Tensor, idx_batch: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """Edges with both endpoints in ``idx_batch``, relabelled to the position of the endpoint in ``idx_batch``."""
    n = int(num_nodes)
    pos = torch.full((n,), -1, dtype=torch.long, device=edge_index.device)
    idx = idx_batch.long().to(edge_index.device)
    pos[idx] = torch.arange(idx.numel(), device=edge_index.device)
    s, d = pos[edge_index[0].long()], pos[edge_index[1].long()]
    keep = (s >= 0) & (d >= 0)
    return torch.stack([s[keep], d[keep]])
