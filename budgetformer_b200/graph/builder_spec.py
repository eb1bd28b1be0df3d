"""Executable specification of the per-epoch attention-graph build (numpy, CPU).

This is the oracle that the C++/OpenMP builder and the CUDA builder are tested against
bit for bit.  It restates the reference pipeline
(utils/fullgraph_sp_support.py:2943-3026, gt_sp/utils.py:1198-1248, :877-887):

1. real edges: per query keep the ``b_real`` in-edges with the smallest
   ``edge_hash31(src, dst, seed + 17)``; ties broken by smaller ``src``;
2. random-walk edges: ``W`` walks of length ``L`` from every node over the coalesced
   out-edge CSR, uniform neighbour, dead ends stay in place; hop ``d`` emits
   ``(walk[d] -> walk[0])`` unless ``d > 1 and walk[d] == walk[d-1]``; per query keep the
   ``b_rw`` candidates (with multiplicity, as in the reference's un-coalesced pool) with
   the smallest ``edge_hash31(src, dst, seed + 37)``;
3. merge: sorted unique union per query; Exphormer instead keeps both lists apart with an
   edge type (0 real, 1 random walk) and appends a type-0 self loop
   (main_node_fullgraph_sp.py:1186-1201).

``None`` as a budget means "all candidates", ``0`` means "drop that side"
(utils/fullgraph_sp_support.py:1289-1307).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .attn_graph import AttnGraph, Topology
from .rng import REAL_SEED_OFFSET, RW_SEED_OFFSET, edge_hash31, walk_uniform32


def random_walks(topo: Topology, walks_per_node: int, walk_length: int, seed: int) -> np.ndarray:
    """[N*W, L+1] int64 walk matrix; walk id = node*W + w."""
    n, w, l = topo.num_nodes, int(walks_per_node), int(walk_length)
    rowptr = topo.out_rowptr.cpu().numpy().astype(np.int64)
    col = topo.out_col.cpu().numpy().astype(np.int64)
    walk_id = np.arange(n * w, dtype=np.uint64)
    cur = (np.arange(n * w, dtype=np.int64) // max(w, 1))
    walks = np.empty((n * w, l + 1), dtype=np.int64)
    walks[:, 0] = cur
    for step in range(1, l + 1):
        deg = rowptr[cur + 1] - rowptr[cur]
        r = walk_uniform32(walk_id, step, seed)
        pick = ((r * deg.astype(np.uint64)) >> np.uint64(32)).astype(np.int64)
        has = deg > 0
        nxt = cur.copy()
        if has.any():
            nxt[has] = col[rowptr[cur[has]] + pick[has]]
        walks[:, step] = nxt
        cur = nxt
    return walks


def rw_candidates(walks: np.ndarray):
    """(src, dst) of every emitted random-walk edge, hop-major like the reference."""
    q = walks[:, 0]
    srcs, dsts = [], []
    for d in range(1, walks.shape[1]):
        kv = walks[:, d]
        valid = kv >= 0
        if d > 1:
            valid &= kv != walks[:, d - 1]
        srcs.append(kv[valid])
        dsts.append(q[valid])
    if not srcs:
        return np.zeros(0, np.int64), np.zeros(0, np.int64)
    return np.concatenate(srcs), np.concatenate(dsts)


def select_per_query(src: np.ndarray, dst: np.ndarray, k: Optional[int], seed: int):
    """Keep the ``k`` smallest (hash, src) per ``dst``.  Returns (src, dst) sorted by (dst, src)."""
    if k is not None and int(k) <= 0:
        return np.zeros(0, np.int64), np.zeros(0, np.int64)
    if src.size == 0:
        return src, dst
    if k is None:
        order = np.lexsort((src, dst))
        return src[order], dst[order]
    comp = (edge_hash31(src, dst, seed) << np.uint64(32)) | src.astype(np.uint64)
    order = np.lexsort((comp, dst))
    d_sorted = dst[order]
    is_new = np.ones(d_sorted.size, dtype=bool)
    is_new[1:] = d_sorted[1:] != d_sorted[:-1]
    starts = np.maximum.accumulate(np.where(is_new, np.arange(d_sorted.size), 0))
    keep = (np.arange(d_sorted.size) - starts) < int(k)
    sel = order[keep]
    s, d = src[sel], dst[sel]
    o2 = np.lexsort((s, d))
    return s[o2], d[o2]


def khop_neighbor_candidates(topo: Topology, fanout, seed: int):
    """``--rw_edge_mode dgl_neighbor``: fan-out k-hop expansion with origin tracking (gt_sp/utils.py:1281-1384).
    From every node, hop h keeps at most ``fanout[h]`` out-neighbours of each frontier node (-1 = all) and emits
    ``(reached node -> origin)``.  Neighbour choice is a seeded hash ranking, so it is reproducible on every rank."""
    n = topo.num_nodes
    rowptr = topo.out_rowptr.cpu().numpy().astype(np.int64)
    col = topo.out_col.cpu().numpy().astype(np.int64)
    deg = np.diff(rowptr)
    e_src = np.repeat(np.arange(n, dtype=np.int64), deg)
    origin = np.arange(n, dtype=np.int64)
    frontier = np.arange(n, dtype=np.int64)
    srcs, dsts = [], []
    for h, f in enumerate(fanout):
        # expand every (origin, frontier) pair along the frontier node's out-edges
        cnt = deg[frontier]
        rep_o = np.repeat(origin, cnt)
        rep_f = np.repeat(frontier, cnt)
        starts = np.repeat(rowptr[frontier], cnt)
        within = np.arange(rep_f.size) - np.repeat(np.cumsum(cnt) - cnt, cnt)
        nbr = col[starts + within]
        if f is not None and int(f) >= 0:
            key = edge_hash31(nbr, rep_f, int(seed) + 101 * (h + 1)) ^ (rep_o.astype(np.uint64) * np.uint64(2654435761) & np.uint64(0x7FFFFFFF))
            pair = rep_o * n + rep_f
            order = np.lexsort((key, pair))
            p_sorted = pair[order]
            new = np.ones(p_sorted.size, dtype=bool)
            new[1:] = p_sorted[1:] != p_sorted[:-1]
            first = np.maximum.accumulate(np.where(new, np.arange(p_sorted.size), 0))
            keep = order[(np.arange(p_sorted.size) - first) < int(f)]
            rep_o, nbr = rep_o[keep], nbr[keep]
        uniq = np.unique(rep_o * n + nbr)
        origin, frontier = uniq // n, uniq % n
        srcs.append(frontier.copy())
        dsts.append(origin.copy())
        if frontier.size == 0:
            break
    if not srcs:
        return np.zeros(0, np.int64), np.zeros(0, np.int64)
    return np.concatenate(srcs), np.concatenate(dsts)


def khop_neighbor_candidates_native(topo: Topology, fanout, seed: int, num_threads: int = 0):
    """The same candidate multiset from the C++/OpenMP expansion (csrc/cpu/edge_builder.cpp), origin-major; ``None``
    when the extension is not available or the topology does not live on the CPU."""
    if topo.out_rowptr.is_cuda:
        return None
    try:
        from ..ops import _ext
        ext = _ext.load()
    except Exception:
        return None
    src, dst = ext.khop_candidates_cpu(topo.out_rowptr.to(torch.int32).contiguous(), topo.out_col.to(torch.int32).contiguous(),
                                       int(topo.num_nodes), [int(f) if f is not None else -1 for f in fanout], int(seed),
                                       int(num_threads))
    return src.numpy(), dst.numpy()


def parse_fanout(text) -> list:
    return [int(t) for t in str(text).split(",") if t.strip()]


def build_attn_graph_spec(
    topo: Topology,
    b_real: Optional[int],
    b_rw: Optional[int],
    walks_per_node: int,
    walk_length: int,
    seed: int,
    *,
    use_real: bool = True,
    use_rw: bool = True,
    exphormer: bool = False,
    fanout=None,
) -> AttnGraph:
    n = topo.num_nodes
    in_rowptr = topo.in_rowptr.cpu().numpy().astype(np.int64)
    in_src = topo.in_src.cpu().numpy().astype(np.int64)
    real_dst = np.repeat(np.arange(n, dtype=np.int64), np.diff(in_rowptr))
    if use_real:
        rs, rd = select_per_query(in_src, real_dst, b_real, int(seed) + REAL_SEED_OFFSET)
    else:
        rs, rd = np.zeros(0, np.int64), np.zeros(0, np.int64)
    if use_rw and (fanout or (walks_per_node > 0 and walk_length > 0)) and (b_rw is None or b_rw > 0):
        if fanout:
            native = khop_neighbor_candidates_native(topo, fanout, seed)
            ws, wd = native if native is not None else khop_neighbor_candidates(topo, fanout, seed)
        else:
            ws, wd = rw_candidates(random_walks(topo, walks_per_node, walk_length, seed))
        ws, wd = select_per_query(ws, wd, b_rw, int(seed) + RW_SEED_OFFSET)
    else:
        ws, wd = np.zeros(0, np.int64), np.zeros(0, np.int64)

    if exphormer:
        self_ids = np.arange(n, dtype=np.int64)
        src = np.concatenate([rs, ws, self_ids])
        dst = np.concatenate([rd, wd, self_ids])
        typ = np.concatenate([np.zeros(rs.size, np.int64), np.ones(ws.size, np.int64), np.zeros(n, np.int64)])
        part = np.concatenate([np.zeros(rs.size, np.int64), np.ones(ws.size, np.int64), np.full(n, 2, np.int64)])
        order = np.lexsort((src, part, dst))
        src, dst, typ = src[order], dst[order], typ[order]
        etype = torch.from_numpy(typ.astype(np.uint8))
    else:
        key = np.unique(np.concatenate([rd, wd]) * n + np.concatenate([rs, ws]))
        dst = key // n
        src = key - dst * n
        etype = None
    rowptr = np.zeros(n + 1, dtype=np.int64)
    if dst.size:
        rowptr[1:] = np.cumsum(np.bincount(dst, minlength=n))
    return AttnGraph(
        n,
        torch.from_numpy(rowptr.astype(np.int32)),
        torch.from_numpy(src.astype(np.int32)),
        etype,
        n_real=int(rs.size),
        n_rw=int(ws.size),
    )
