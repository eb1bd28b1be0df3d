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
    ``--include_real_edges`` path), budgets above 32 per side, walks longer than 16 and the fan-out mode go to the
    general C++ builder on the CPU (to the numpy specification only when the extension is missing or
    ``force_spec`` asks for it)."""
    br = 0 if not use_real else b_real
    bw = 0 if (not use_rw or (not fanout and (walks_per_node <= 0 or walk_length <= 0))) else b_rw
    if not force_spec and (fanout or not native_supported(br, bw, walk_length)):
        g = _build_rows_native(topo, b_real, b_rw, walks_per_node, walk_length, seed, use_real, use_rw, exphormer,
                               fanout, num_threads)
        if g is not None:
            return g.to(topo.device) if topo.device.type != "cpu" else g
    if force_spec or fanout or not native_supported(br, bw, walk_length):
        g = build_attn_graph_spec(topo, b_real, b_rw, walks_per_node, walk_length, seed,
                                  use_real=use_real, use_rw=use_rw, exphormer=exphormer, fanout=fanout)
        return g.to(topo.device) if topo.device.type != "cpu" else g
    from ..ops import _ext
    ext = _ext.load()
    rowptr, col, etype, totals = ext.build_attn_graph(
        topo.in_rowptr, topo.in_src, topo.out_rowptr, topo.out_col, int(topo.num_nodes),
        int(br), int(bw), int(walks_per_node), int(walk_length), bool(exphormer), int(seed), int(num_threads),
        _long_rows(topo, ext))
    if topo.device.type == "cuda":
        _ext.count_launches(2)
    g = AttnGraph(int(topo.num_nodes), rowptr, col, etype if exphormer else None,
                  max_degree=int(br) + int(bw) + (1 if exphormer else 0))
    g._totals = totals  # device tensor; read lazily to avoid a sync on the hot path
    return g


def _long_rows(topo: Topology, ext) -> Optional[torch.Tensor]:
    """Queries whose in-edge row the device builder ranks with a whole thread block instead of one lane group (power-law
    graphs have rows of 10^5 - 10^6 in-edges that would otherwise be the tail of the selection kernel).
    ``BF_BUILD_HUB_BLOCKS=0`` switches the pre-pass off (measurements)."""
    import os
    if topo.device.type != "cuda" or os.environ.get("BF_BUILD_HUB_BLOCKS", "1") == "0":
        return None
    return topo.in_hub_rows(int(ext.BUILD_HUB_DEGREE))


def _build_rows_native(topo: Topology, b_real: Optional[int], b_rw: Optional[int], walks_per_node: int, walk_length: int,
                       seed: int, use_real: bool, use_rw: bool, exphormer: bool, fanout, num_threads: int,
                       rows: Optional[tuple] = None) -> Optional[AttnGraph]:
    """The cases the fixed-width builders do not take - a side without budget (``None``: every candidate) or above
    ``MAX_SIDE_BUDGET``, walks longer than ``MAX_WALK_LEN`` - on the general two-pass C++/OpenMP builder.  It runs on
    the CPU copy of the topology (the specification it replaces does too); ``None`` without the extension.
    ``rows = (begin, end)`` builds only those queries: the result has ``end - begin`` rows (keys keep their global ids),
    which is what a rank contributes to a sharded build (``build_attn_graph_shard``)."""
    try:
        from ..ops import _ext
        ext = _ext.load()
    except Exception:
        return None
    cpu = topo if topo.device.type == "cpu" else topo.to("cpu")
    i32 = lambda t: t.to(torch.int32).contiguous()
    walk_side = bool(use_rw) and (bool(fanout) or (walks_per_node > 0 and walk_length > 0))
    code = lambda b: -1 if b is None else int(b)
    rowptr, col, etype, totals = ext.build_attn_graph_rows_cpu(
        i32(cpu.in_rowptr), i32(cpu.in_src), i32(cpu.out_rowptr), i32(cpu.out_col), int(topo.num_nodes),
        code(b_real), code(b_rw), bool(use_real), walk_side, int(walks_per_node), int(walk_length),
        [int(f) if f is not None else -1 for f in (fanout or [])], bool(exphormer), int(seed), int(num_threads),
        int(rows[0]) if rows else 0, int(rows[1]) if rows else -1)
    r, w = (int(x) for x in totals.tolist())
    bound = None
    if b_real is not None and b_rw is not None:
        bound = max(0, int(b_real)) + max(0, int(b_rw)) + (1 if exphormer else 0)
    n_rows = int(rows[1] - rows[0]) if rows else int(topo.num_nodes)
    return AttnGraph(n_rows, rowptr, col, etype if exphormer else None, n_real=r, n_rw=w, max_degree=bound)


def build_attn_graph_shard(topo: Topology, rows: tuple, b_real: Optional[int], b_rw: Optional[int], walks_per_node: int,
                           walk_length: int, seed: int, *, use_real: bool = True, use_rw: bool = True,
                           exphormer: bool = False, num_threads: int = 0, fanout=None) -> AttnGraph:
    """The rows ``[rows[0], rows[1])`` of the graph ``build_attn_graph`` would return, as a graph over those queries
    only.  Rows are independent of one another, so the shards of all ranks concatenate to the full graph."""
    g = _build_rows_native(topo, b_real, b_rw, walks_per_node, walk_length, seed, use_real, use_rw, exphormer, fanout,
                           num_threads, rows=rows)
    if g is not None:
        return g
    full = build_attn_graph_spec(topo, b_real, b_rw, walks_per_node, walk_length, seed, use_real=use_real,
                                 use_rw=use_rw, exphormer=exphormer, fanout=fanout)          # no extension: cut it out
    lo, hi = int(full.rowptr[rows[0]]), int(full.rowptr[rows[1]])
    return AttnGraph(int(rows[1] - rows[0]), (full.rowptr[rows[0]:rows[1] + 1] - lo).contiguous(), full.col[lo:hi].contiguous(),
                     None if full.etype is None else full.etype[lo:hi].contiguous(), max_degree=full.max_degree)


class ShardedDeviceBuild:
    """Device build split over the sequence-parallel ranks by query range.

    Every rank runs the selection kernel (hash-ranked real edges, Philox walks, merge) for its own ``N / P`` queries
    only and leaves the fixed-width rows in a symmetric buffer; after one device barrier each rank fetches all shards
    with coalesced peer loads and finishes locally (prefix sum, compaction to CSR).  Rows do not depend on one another,
    so the result is bit-identical to the whole build - the reference reaches the same end by broadcasting the edge
    list from one rank (utils/fullgraph_sp_support.py:3262-3338); here the work is divided instead of repeated.

    Two shard buffers alternate: a rank overwrites a buffer only after it has passed the barrier of the build in
    between, which every peer reaches after it finished fetching, so no second barrier is needed.  One instance serves
    one host thread and one barrier channel (the ranks must issue its builds in the same order)."""

    def __init__(self, world, channel: int):
        self.sw, self.channel = world, int(channel)
        self.bufs = [None, None]
        self.nbytes = 0
        self.turn = 0

    @staticmethod
    def _layout(rows: int, cap: int):
        a16 = lambda b: (b + 15) // 16 * 16
        col, cnt, typ = a16(rows * cap * 4), a16(rows * 4), a16(rows * cap)
        return col, cnt, typ, col + cnt + typ + 16

    def ensure(self, rows: int, cap: int) -> None:
        """Make the two shard buffers large enough for ``rows`` x ``cap``.  Allocation is a collective of the group:
        call it from the thread that owns the group's other collectives, with the same arguments on every rank."""
        need = self._layout(rows, cap)[3]
        if need > self.nbytes:
            self.bufs = [self.sw.alloc((need,), torch.uint8) for _ in range(2)]
            self.nbytes, self.turn = need, 0

    def ready(self, rows: int, cap: int) -> bool:
        return self._layout(rows, cap)[3] <= self.nbytes

    def build(self, topo: Topology, br: int, bw: int, walks_per_node: int, walk_length: int, seed: int,
              exphormer: bool) -> AttnGraph:
        from ..ops import _ext
        ext = _ext.load()
        sw = self.sw
        n, p = int(topo.num_nodes), sw.world
        rows = n // p
        cap = max(int(br) + int(bw) + (1 if exphormer else 0), 1)
        buf = self.bufs[self.turn]
        self.turn ^= 1
        o_col, o_cnt, o_typ, _total = self._layout(rows, cap)
        t = buf.tensor
        ell_col = t[:rows * cap * 4].view(torch.int32)
        ell_cnt = t[o_col:o_col + rows * 4].view(torch.int32)
        ell_typ = t[o_col + o_cnt:o_col + o_cnt + rows * cap] if exphormer else None
        totals = t[o_col + o_cnt + o_typ:o_col + o_cnt + o_typ + 16].view(torch.int64)
        ext.budget_select_rows(topo.in_rowptr, topo.in_src, topo.out_rowptr, topo.out_col, n, int(br), int(bw),
                               int(walks_per_node), int(walk_length), bool(exphormer), int(seed), sw.rank * rows, rows,
                               ell_col, ell_cnt, ell_typ, totals, _long_rows(topo, ext))
        sw.barrier(self.channel)                                  # every rank's shard is complete
        dev = t.device
        full_col = torch.empty(n * cap, dtype=torch.int32, device=dev)
        full_cnt = torch.empty(n, dtype=torch.int32, device=dev)
        ext.peer_concat(buf.ptrs, rows * cap, full_col)
        ext.peer_concat([ptr + o_col for ptr in buf.ptrs], rows, full_cnt)
        full_typ = None
        if exphormer:
            full_typ = torch.empty(n * cap, dtype=torch.uint8, device=dev)
            ext.peer_concat([ptr + o_col + o_cnt for ptr in buf.ptrs], rows * cap, full_typ)
        all_tot = torch.empty(2 * p, dtype=torch.int64, device=dev)
        ext.peer_concat([ptr + o_col + o_cnt + o_typ for ptr in buf.ptrs], 2, all_tot)
        rowptr, col, etype = ext.ell_rows_to_csr(full_col, full_cnt, full_typ, n, cap)
        _ext.count_launches(7 if exphormer else 6)
        g = AttnGraph(n, rowptr, col, etype if exphormer else None, max_degree=int(br) + int(bw) + (1 if exphormer else 0))
        g._totals = all_tot.view(p, 2).sum(0)
        return g


def graph_totals(g: AttnGraph):
    """(selected real edges, selected walk edges) of a natively built graph."""
    t = getattr(g, "_totals", None)
    if t is not None:
        r, w = (int(x) for x in t.tolist())
        g.n_real, g.n_rw = r, w
    return g.n_real, g.n_rw


__all__ = ["build_attn_graph", "build_attn_graph_shard", "graph_totals", "add_virtual_node", "native_supported",
           "ShardedDeviceBuild"]
