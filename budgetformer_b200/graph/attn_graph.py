"""Attention-graph containers.

``Topology`` is the raw graph in the two int32 CSR forms the builders need (out-edges
for random walks, in-edges for per-query real-edge sampling).  ``AttnGraph`` is one
epoch's sampled attention graph stored as a CSR over *queries* (destination nodes)
plus, lazily, its transpose over *keys* for the atomics-free backward pass.

The reference carries this object as an int64 COO ``edge_index[2|3, E]`` with
``edge_index[0]`` = key/value node and ``edge_index[1]`` = query node
(models/gt_dist_node_level.py:224-262) and re-sorts it inside every scatter.  Because
every query holds at most ``B`` sampled in-edges by construction, grouping by query
once at build time is free and lets the attention kernels run gather-only.
``AttnGraph.edge_index()`` / ``AttnGraph.from_edge_index()`` convert to and from the
reference's COO form so both representations are accepted by every model.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

HUB_DEGREE = 1024  # rows longer than this take the chunked hub path in the kernels
KV_TASK_EDGES = 64  # edges per work item of the dK/dV pass (32 and 128 both measured slower on the 2.9 M-node graph)


@dataclass
class Topology:
    """Raw graph, int32 CSR both ways.  ``out_*`` is coalesced (sorted, unique) like the
    reference's random-walk CSR (gt_sp/utils.py:926-931); ``in_*`` keeps multiplicity
    like the reference's real-edge sampler input (utils/fullgraph_sp_support.py:262-298)."""

    num_nodes: int
    out_rowptr: torch.Tensor  # [N+1] int32/int64
    out_col: torch.Tensor     # [E'] int32
    in_rowptr: torch.Tensor   # [N+1]
    in_src: torch.Tensor      # [E] int32

    @property
    def device(self):
        return self.out_col.device

    @property
    def num_edges(self) -> int:
        return int(self.in_src.numel())

    def to(self, device, non_blocking: bool = False) -> "Topology":
        f = lambda t: t.to(device, non_blocking=non_blocking)
        return Topology(self.num_nodes, f(self.out_rowptr), f(self.out_col), f(self.in_rowptr), f(self.in_src))

    def pin_memory(self) -> "Topology":
        f = lambda t: t.pin_memory() if not t.is_cuda else t
        return Topology(self.num_nodes, f(self.out_rowptr), f(self.out_col), f(self.in_rowptr), f(self.in_src))

    def nbytes(self) -> int:
        return sum(int(t.numel()) * t.element_size() for t in (self.out_rowptr, self.out_col, self.in_rowptr, self.in_src))

    def in_hub_rows(self, min_degree: int) -> Optional[torch.Tensor]:
        """Ascending int32 ids of the nodes with more than ``min_degree`` in-edges (``None`` when there are none).  The
        topology does not change during a run, so the list is computed once per threshold and kept."""
        cache = self.__dict__.setdefault("_hub_rows", {})
        if min_degree not in cache:
            deg = self.in_rowptr[1:] - self.in_rowptr[:-1]
            rows = torch.nonzero(deg > int(min_degree)).flatten().to(torch.int32).contiguous()
            cache[min_degree] = rows if rows.numel() > 0 else None
        return cache[min_degree]

    @staticmethod
    def from_edge_index(edge_index: torch.Tensor, num_nodes: int) -> "Topology":
        """Build both CSRs from an int64 COO ``[2, E]`` (row 0 = source, row 1 = destination)."""
        ei = edge_index[:2].to(torch.int64)
        src, dst = ei[0], ei[1]
        n = int(num_nodes)
        dev = ei.device
        # in-CSR: stable sort by (dst, src), multiplicity kept
        key_in = dst * n + src
        order = torch.argsort(key_in, stable=True)
        in_src = src[order].to(torch.int32)
        in_rowptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
        in_rowptr[1:] = torch.cumsum(torch.bincount(dst, minlength=n), 0)
        # out-CSR: unique (src, dst)
        key_out = torch.unique(src * n + dst)
        o_src = torch.div(key_out, n, rounding_mode="floor")
        out_col = (key_out - o_src * n).to(torch.int32)
        out_rowptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
        out_rowptr[1:] = torch.cumsum(torch.bincount(o_src, minlength=n), 0)
        return Topology(n, out_rowptr.to(torch.int32), out_col, in_rowptr.to(torch.int32), in_src)


@dataclass
class AttnGraph:
    """Sampled attention graph: CSR over queries.

    ``num_rows`` is the length of the post-all-to-all sequence the ids address
    (``N`` for GT/GraphGPS/Exphormer, ``N + P`` for Graphormer whose every rank carries
    a copy of the virtual node: main_node_fullgraph_sp.py:251-257)."""

    num_rows: int
    rowptr: torch.Tensor                 # [num_rows+1] int32
    col: torch.Tensor                    # [E] int32 — key/value node per edge
    etype: Optional[torch.Tensor] = None  # [E] uint8 (Exphormer edge type)
    # transpose over keys, built lazily
    t_rowptr: Optional[torch.Tensor] = field(default=None, repr=False)
    t_row: Optional[torch.Tensor] = field(default=None, repr=False)   # query id per transposed slot
    t_eid: Optional[torch.Tensor] = field(default=None, repr=False)   # position in ``col``
    # balanced work list over the transpose (chunks of <= KV_TASK_EDGES edges); see ensure_transpose
    t_task: Optional[torch.Tensor] = field(default=None, repr=False)        # [T, 4] int32: row, beg, end, partial slot
    t_split: Optional[torch.Tensor] = field(default=None, repr=False)       # [S, 3] int32: row, first slot, n slots
    max_degree: Optional[int] = None     # known upper bound on query in-degree (None = unknown)
    n_real: int = -1
    n_rw: int = -1
    kv_slots: int = 0                    # number of fp32 partial slots the dK/dV pass needs

    @property
    def device(self):
        return self.col.device

    @property
    def num_edges(self) -> int:
        return int(self.col.numel())

    def nbytes(self) -> int:
        tot = 0
        for t in (self.rowptr, self.col, self.etype, self.t_rowptr, self.t_row, self.t_eid, self.t_task, self.t_split):
            if t is not None:
                tot += int(t.numel()) * t.element_size()
        return tot

    def to(self, device, non_blocking: bool = False) -> "AttnGraph":
        f = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)
        return AttnGraph(self.num_rows, f(self.rowptr), f(self.col), f(self.etype), f(self.t_rowptr),
                         f(self.t_row), f(self.t_eid), f(self.t_task), f(self.t_split), self.max_degree,
                         self.n_real, self.n_rw, self.kv_slots)

    def record_stream(self, stream) -> None:
        """Tell the caching allocator that ``stream`` uses every tensor of the graph (they were allocated on another)."""
        for t in (self.rowptr, self.col, self.etype, self.t_rowptr, self.t_row, self.t_eid, self.t_task, self.t_split,
                  getattr(self, "_totals", None)):
            if t is not None and t.is_cuda:
                t.record_stream(stream)

    def row_ids(self) -> torch.Tensor:
        """Query id of every edge (int64), i.e. ``edge_index[1]`` of the COO form."""
        deg = (self.rowptr[1:] - self.rowptr[:-1]).to(torch.int64)
        return torch.repeat_interleave(torch.arange(self.num_rows, device=self.device), deg,
                                       output_size=self.num_edges)

    def edge_index(self) -> torch.Tensor:
        """COO ``[2|3, E]`` int64 in the reference's convention (row 0 key, row 1 query)."""
        rows = [self.col.to(torch.int64), self.row_ids()]
        if self.etype is not None:
            rows.append(self.etype.to(torch.int64))
        return torch.stack(rows, 0)

    def ensure_transpose(self) -> "AttnGraph":
        """Build the by-key CSR (deterministic: stable sort keeps query order inside a key's row)."""
        if self.t_rowptr is not None:
            return self
        if self.col.is_cuda and self.col.dtype == torch.int32 and self.rowptr.dtype == torch.int32:
            # device graphs: radix sort over the node-id bits + compaction kernels (csrc/graph_transpose.cu)
            from ..ops import _ext
            t_rowptr, t_row, t_eid, tasks, splits, sizes = _ext.load().graph_transpose(
                self.rowptr.contiguous(), self.col.contiguous(), int(self.num_rows), int(KV_TASK_EDGES))
            _ext.count_launches(9)
            self.t_rowptr, self.t_row, self.t_eid = t_rowptr, t_row, t_eid
            self.t_task, self.t_split, self.kv_slots = tasks, splits, int(sizes[1])
            return self
        col64 = self.col.to(torch.int64)
        _, perm = torch.sort(col64, stable=True)
        rows = self.row_ids()
        self.t_eid = perm.to(torch.int32)
        self.t_row = rows[perm].to(torch.int32)
        t_rowptr = torch.zeros(self.num_rows + 1, dtype=torch.int64, device=self.device)
        if self.num_edges:
            t_rowptr[1:] = torch.cumsum(torch.bincount(col64, minlength=self.num_rows), 0)
        self.t_rowptr = t_rowptr.to(torch.int32)
        self._build_kv_tasks(t_rowptr)
        return self

    def _build_kv_tasks(self, t_rowptr: torch.Tensor) -> None:
        """Work list of the dK/dV pass.  Key popularity is heavy-tailed (a hub is the key of 10^4-10^5 edges), so a
        row-per-lane-group mapping leaves most of the GPU idle behind a few long rows.  Every key row is cut into
        chunks of at most ``KV_TASK_EDGES`` edges; rows with one chunk store their result directly, rows with
        several write fp32 partials that a second small kernel adds up in a fixed order (deterministic, no atomics)."""
        dev = self.device
        deg = t_rowptr[1:] - t_rowptr[:-1]
        n_chunks = torch.clamp((deg + KV_TASK_EDGES - 1) // KV_TASK_EDGES, min=1)
        first = torch.zeros(self.num_rows + 1, dtype=torch.int64, device=dev)
        first[1:] = torch.cumsum(n_chunks, 0)
        total = int(first[-1].item()) if self.num_rows else 0
        rows = torch.repeat_interleave(torch.arange(self.num_rows, device=dev), n_chunks, output_size=total)
        chunk = torch.arange(total, device=dev) - first[rows]
        beg = t_rowptr[rows] + chunk * KV_TASK_EDGES
        end = torch.minimum(beg + KV_TASK_EDGES, t_rowptr[rows + 1])
        split_row = n_chunks > 1
        is_split = split_row[rows]
        slot = torch.cumsum(is_split.to(torch.int64), 0) - 1
        slot = torch.where(is_split, slot, torch.full_like(slot, -1))
        tasks = torch.stack([rows, beg, end, slot], 1)
        # items of split keys first (long work is scheduled first), then one item per remaining key, both in key order
        tasks = torch.cat([tasks[is_split], tasks[~is_split]], 0)
        self.t_task = tasks.to(torch.int32).contiguous()
        srows = torch.nonzero(split_row).flatten()
        nsl = n_chunks[srows]
        sfirst = torch.cumsum(nsl, 0) - nsl
        self.t_split = torch.stack([srows, sfirst, nsl], 1).to(torch.int32).contiguous()
        self.kv_slots = int(nsl.sum().item()) if srows.numel() else 0

    @staticmethod
    def from_edge_index(edge_index: torch.Tensor, num_rows: int) -> "AttnGraph":
        """Group an arbitrary COO by query (stable, so the reference's within-query order is kept)."""
        ei = edge_index.to(torch.int64)
        dst = ei[1]
        order = torch.argsort(dst, stable=True)
        col = ei[0][order].to(torch.int32)
        rowptr = torch.zeros(num_rows + 1, dtype=torch.int64, device=ei.device)
        if dst.numel():
            rowptr[1:] = torch.cumsum(torch.bincount(dst, minlength=num_rows), 0)
        etype = ei[2][order].to(torch.uint8) if ei.size(0) >= 3 else None
        return AttnGraph(int(num_rows), rowptr.to(torch.int32), col, etype)


def as_attn_graph(edges, num_rows: int) -> AttnGraph:
    """Accept either container; models call this on whatever the caller passed as ``edge_index``."""
    if isinstance(edges, AttnGraph):
        if edges.num_rows != num_rows:
            raise ValueError(f"attention graph has {edges.num_rows} rows, sequence has {num_rows}")
        return edges
    if isinstance(edges, torch.Tensor):
        return AttnGraph.from_edge_index(edges, num_rows)
    raise TypeError(f"unsupported edge container {type(edges)!r}")


def add_virtual_node(graph: AttnGraph, num_nodes: int, nodes_per_rank: int) -> AttnGraph:
    """Graphormer virtual node in the post-all-to-all index space.

    Equivalent to the reference's ``fix_edge_index`` (gt_sp/utils.py:113-130: shift ids by +1,
    add node->0 and 0->node for every node) followed by ``adjust_edge_index_nomerge``
    (gt_sp/utils.py:540-545: id j>0 moves to j + (j-1)//nodes_per_rank so that it skips the P
    per-rank copies of the virtual node).  Row 0 gets all N nodes (a hub row); every real row
    gets the extra key 0 appended; rows of the other P-1 token copies stay empty.
    """
    n, s = int(num_nodes), int(nodes_per_rank)
    p = (n + s - 1) // s
    dev = graph.device
    ids = torch.arange(n, device=dev, dtype=torch.int64)
    new_id = ids + 1 + torch.div(ids, s, rounding_mode="floor")          # real node -> sequence row
    deg = (graph.rowptr[1:] - graph.rowptr[:-1]).to(torch.int64)
    total = n + p
    new_deg = torch.zeros(total, dtype=torch.int64, device=dev)
    new_deg[new_id] = deg + 1
    new_deg[0] = n
    rowptr = torch.zeros(total + 1, dtype=torch.int64, device=dev)
    rowptr[1:] = torch.cumsum(new_deg, 0)
    e_new = int(graph.num_edges + 2 * n)
    col = torch.empty(e_new, dtype=torch.int32, device=dev)
    # row 0: all real nodes in id order
    col[:n] = new_id.to(torch.int32)
    # real rows: virtual key (0) first — the reference's coalesced order is irrelevant to the math
    starts = rowptr[new_id]
    col[starts] = 0
    if graph.num_edges:
        rows = graph.row_ids()
        pos_in_row = torch.arange(graph.num_edges, device=dev) - graph.rowptr[:-1].to(torch.int64)[rows]
        col[starts[rows] + 1 + pos_in_row] = new_id[graph.col.to(torch.int64)].to(torch.int32)
    return AttnGraph(total, rowptr.to(torch.int32), col, None, max_degree=None,
                     n_real=graph.n_real, n_rw=graph.n_rw)
