"""Attention-graph construction rules, restated by brute force on int64 COO (NumPy).

* per-query sampling: group candidate edges by query, rank by
  ``(src*1103515245 + dst*214013 + seed'*2654435761 + 12345) mod 2^31`` with ``seed' = seed + 17`` (real edges) or
  ``+ 37`` (walk edges), keep the K smallest; ties go to the smaller source id; fewer than K candidates are all kept
  (utils/fullgraph_sp_support.py:970-1004);
* random-walk edges from given walks: hop ``d >= 1`` of a walk from ``s`` emits ``(walk[d] -> s)`` unless ``d > 1`` and
  the walk stood still (gt_sp/utils.py:1232-1248);
* merge = sorted unique union (gt_sp/utils.py:877-887);
* Graphormer's virtual node: ``fix_edge_index`` + ``adjust_edge_index_nomerge`` (gt_sp/utils.py:113-130, :540-545).
"""
from __future__ import annotations

import numpy as np

REAL_SEED_OFFSET = 17
WALK_SEED_OFFSET = 37


def edge_hash(src, dst, seed):
    s = np.asarray(src, dtype=np.int64)
    d = np.asarray(dst, dtype=np.int64)
    with np.errstate(over="ignore"):
        return (s * 1103515245 + d * 214013 + np.int64(seed) * 2654435761 + 12345) % (1 << 31)


def sample_per_query(src, dst, k: int, seed: int):
    """Indices (into the candidate arrays) of the edges kept: for every query the ``k`` smallest (hash, src)."""
    src = np.asarray(src, dtype=np.int64)
    dst = np.asarray(dst, dtype=np.int64)
    if k <= 0:
        return np.zeros(0, dtype=np.int64)
    key = edge_hash(src, dst, seed)
    keep = []
    for q in np.unique(dst):
        idx = np.nonzero(dst == q)[0]
        # duplicates of one (src, dst) pair share hash and source: the first occurrence represents them
        order = sorted(idx.tolist(), key=lambda i: (int(key[i]), int(src[i]), i))
        keep.extend(order[:k])
    return np.asarray(sorted(keep), dtype=np.int64)


def walk_edges(walks):
    """``walks``: int array ``[n_walks, L + 1]`` (column 0 = start).  Returns the emitted ``(src, dst)`` arrays."""
    walks = np.asarray(walks, dtype=np.int64)
    srcs, dsts = [], []
    for d in range(1, walks.shape[1]):
        ok = walks[:, d] >= 0
        if d > 1:
            ok &= walks[:, d] != walks[:, d - 1]
        srcs.append(walks[ok, d])
        dsts.append(walks[ok, 0])
    if not srcs:
        return np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.int64)
    return np.concatenate(srcs), np.concatenate(dsts)


def merge_unique(*edge_sets):
    """Sorted unique union of ``(src, dst)`` pairs, ordered by (query, key) like a CSR over queries."""
    pairs = set()
    for s, d in edge_sets:
        pairs.update(zip(np.asarray(s).tolist(), np.asarray(d).tolist()))
    out = sorted(pairs, key=lambda p: (p[1], p[0]))
    if not out:
        return np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.int64)
    a = np.asarray(out, dtype=np.int64)
    return a[:, 0], a[:, 1]


def budgeted_edges(real_src, real_dst, walk_src, walk_dst, b_real: int, b_walk: int, seed: int):
    r = sample_per_query(real_src, real_dst, b_real, seed + REAL_SEED_OFFSET)
    w = sample_per_query(walk_src, walk_dst, b_walk, seed + WALK_SEED_OFFSET)
    return merge_unique((np.asarray(real_src)[r], np.asarray(real_dst)[r]), (np.asarray(walk_src)[w], np.asarray(walk_dst)[w]))


def add_virtual_node(src, dst, num_nodes: int, nodes_per_rank: int):
    """Ids shifted by one, node <-> virtual node (id 0) edges in both directions, then every id ``j > 0`` moved to
    ``j + (j - 1) // nodes_per_rank`` so that it lands behind the per-rank copies of the token in the gathered
    sequence."""
    src = np.asarray(src, dtype=np.int64) + 1
    dst = np.asarray(dst, dtype=np.int64) + 1
    nodes = np.arange(1, num_nodes + 1, dtype=np.int64)
    zeros = np.zeros(num_nodes, dtype=np.int64)
    src = np.concatenate([src, nodes, zeros])
    dst = np.concatenate([dst, zeros, nodes])
    move = lambda j: np.where(j > 0, j + (j - 1) // nodes_per_rank, j)
    return move(src), move(dst)
