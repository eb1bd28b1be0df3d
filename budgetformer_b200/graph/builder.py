"""Per-epoch attention-graph construction: dispatch between the CUDA builder, its C++/OpenMP
twin and the numpy specification.

All three implement the same rules (see ``builder_spec``) and return identical ``AttnGraph``
objects for identical ``(topology, budgets, seed)``, which is why no rank ever has to
broadcast edges: every rank calls ``build_attn_graph`` with the epoch seed
(utils/fullgraph_sp_runtime.py:221-226 in the reference) and gets the same graph.
"""
from __future__ import annotations

from typing import Optional

import torch

from .attn_graph import AttnGraph, Topology, add_virtual_node
from .builder_spec import build_attn_graph_spec

MAX_SIDE_BUDGET = 32
MAX_WALK_LEN = 16


def native_supported(b_real: Optional[int], b_rw: Optional[int], walk_length: int) -> bool:
    if b_real is None or b_rw is None:
        return False
    return 0 <= b_real <= MAX_SIDE_BUDGET and 0 <= b_rw <= MAX_SIDE_BUDGET and walk_length <= MAX_WALK_LEN


def build_attn_graph(
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
    num_threads: int = 0,
    force_spec: bool = False,
    fanout=None,
) -> AttnGraph:
    """Build on whatever device ``topo`` lives on.  ``None`` budgets (unsampled, the legacy
    ``--include_real_edges`` path) and budgets above 32 per side fall back to the specification."""
    br = 0 if not use_real else b_real
    bw = 0 if (not use_rw or (not fanout and (walks_per_node <= 0 or walk_length <= 0))) else b_rw
    if fanout and not force_spec and br is not None and bw is not None and topo.device.type == "cpu":
        g = _build_fanout_native(topo, int(br), int(bw), fanout, seed, exphormer, num_threads)
        if g is not None:
            return g
    if force_spec or fanout or not native_supported(br, bw, walk_length):
        g = build_attn_graph_spec(topo, b_real, b_rw, walks_per_node, walk_length, seed,
                                  use_real=use_real, use_rw=use_rw, exphormer=exphormer, fanout=fanout)
        return g.to(topo.device) if topo.device.type != "cpu" else g
    from ..ops import _ext
    ext = _ext.load()
    rowptr, col, etype, totals = ext.build_attn_graph(
        topo.in_rowptr, topo.in_src, topo.out_rowptr, topo.out_col, int(topo.num_nodes),
        int(br), int(bw), int(walks_per_node), int(walk_length), bool(exphormer), int(seed), int(num_threads))
    if topo.device.type == "cuda":
        _ext.count_launches(2)
    g = AttnGraph(int(topo.num_nodes), rowptr, col, etype if exphormer else None,
                  max_degree=int(br) + int(bw) + (1 if exphormer else 0))
    g._totals = totals  # device tensor; read lazily to avoid a sync on the hot path
    return g


def _build_fanout_native(topo: Topology, br: int, bw: int, fanout, seed: int, exphormer: bool,
                         num_threads: int) -> Optional[AttnGraph]:
    """``--rw_edge_mode dgl_neighbor`` on the C++/OpenMP builder (expansion, per-query selection and merge in one pass
    per query); ``None`` when the extension is not available."""
    try:
        from ..ops import _ext
        ext = _ext.load()
    except Exception:
        return None
    i32 = lambda t: t.to(torch.int32).contiguous()
    rowptr, col, etype, totals = ext.build_attn_graph_fanout_cpu(
        i32(topo.in_rowptr), i32(topo.in_src), i32(topo.out_rowptr), i32(topo.out_col), int(topo.num_nodes), br, bw,
        [int(f) if f is not None else -1 for f in fanout], bool(exphormer), int(seed), int(num_threads))
    r, w = (int(x) for x in totals.tolist())
    return AttnGraph(int(topo.num_nodes), rowptr, col, etype if exphormer else None, n_real=r, n_rw=w,
                     max_degree=br + bw + (1 if exphormer else 0))


def graph_totals(g: AttnGraph):
    """(selected real edges, selected walk edges) of a natively built graph."""
    t = getattr(g, "_totals", None)
    if t is not None:
        r, w = (int(x) for x in t.tolist())
        g.n_real, g.n_rw = r, w
    return g.n_real, g.n_rw


__all__ = ["build_attn_graph", "graph_totals", "add_virtual_node", "native_supported"]
