"""Attention-graph construction: C++ builder vs the numpy specification, structural properties."""
import numpy as np
import pytest
import torch

from budgetformer_b200.graph.attn_graph import AttnGraph, Topology, add_virtual_node
from budgetformer_b200.graph.builder import build_attn_graph
from budgetformer_b200.graph.builder_spec import random_walks, rw_candidates, select_per_query
from budgetformer_b200.graph.rng import edge_hash31
from tests.helpers import random_topology


@pytest.mark.parametrize("exph", [False, True])
@pytest.mark.parametrize("cfg", [(4, 4, 2, 4), (2, 6, 3, 5), (8, 0, 2, 4), (0, 5, 2, 3), (32, 32, 8, 8)])
def test_native_cpu_builder_equals_spec(cfg, exph):
    br, bw, w, l = cfg
    topo, _ = random_topology(400, 3500, hub_in=500, seed=4)
    a = build_attn_graph(topo, br, bw, w, l, 45, exphormer=exph)
    b = build_attn_graph(topo, br, bw, w, l, 45, exphormer=exph, force_spec=True)
    assert torch.equal(a.rowptr, b.rowptr) and torch.equal(a.col, b.col)
    if exph:
        assert torch.equal(a.etype, b.etype)


def test_budget_is_respected_and_rows_sorted_unique():
    topo, _ = random_topology(300, 4000, seed=1)
    g = build_attn_graph(topo, 3, 5, 4, 4, 9)
    deg = g.rowptr[1:] - g.rowptr[:-1]
    assert int(deg.max()) <= 8
    rows = g.row_ids()
    key = rows * 300 + g.col.long()
    assert torch.all(key[1:] > key[:-1])


def test_real_edges_are_real_and_nested_in_budget():
    """Common random numbers: the top-K set is contained in the top-(K+2) set for the same seed
    (the budget controller relies on this)."""
    topo, ei = random_topology(300, 5000, seed=2)
    real = set((int(s), int(d)) for s, d in ei.t().tolist())
    prev = None
    for k in (2, 4, 6, 8):
        g = build_attn_graph(topo, k, 0, 2, 4, 13)
        cur = set(zip(g.col.tolist(), g.row_ids().tolist()))
        assert cur <= real
        if prev is not None:
            assert prev <= cur
        prev = cur


def test_hash_matches_reference_formula():
    src, dst, seed = np.array([5, 123456789]), np.array([7, 987654321]), 59
    want = [(int(s) * 1103515245 + int(d) * 214013 + seed * 2654435761 + 12345) % (1 << 31) for s, d in zip(src, dst)]
    assert edge_hash31(src, dst, seed).tolist() == want


def test_walk_rules():
    # path 0 -> 1 -> 2 (2 is a sink): a walk from 0 reaches 1, 2, then stays at 2
    ei = torch.tensor([[0, 1], [1, 2]])
    topo = Topology.from_edge_index(ei, 3)
    walks = random_walks(topo, 1, 4, seed=0)
    assert walks[0].tolist() == [0, 1, 2, 2, 2]
    assert walks[2].tolist() == [2, 2, 2, 2, 2]
    s, d = rw_candidates(walks)
    pairs = sorted(zip(s.tolist(), d.tolist()))
    # sink emits the hop-1 self edge only; stalled steps are dropped
    assert (2, 2) in pairs and pairs.count((2, 2)) == 1
    assert (2, 0) in pairs and pairs.count((2, 0)) == 1


def test_select_per_query_bruteforce():
    rng = np.random.default_rng(0)
    src, dst = rng.integers(0, 50, 600), rng.integers(0, 20, 600)
    s, d = select_per_query(src, dst, 3, 99)
    for q in range(20):
        cand = src[dst == q]
        comp = sorted(((int(edge_hash31(np.array([c]), np.array([q]), 99)[0]) << 32) | int(c)) for c in cand)[:3]
        assert sorted(s[d == q].tolist()) == sorted(c & 0xFFFFFFFF for c in comp)


def test_every_rank_builds_the_same_graph():
    topo, _ = random_topology(256, 2000, seed=8)
    a = build_attn_graph(topo, 4, 4, 2, 4, 100, num_threads=1)
    b = build_attn_graph(topo, 4, 4, 2, 4, 100, num_threads=4)
    assert torch.equal(a.col, b.col) and torch.equal(a.rowptr, b.rowptr)


def test_virtual_node_index_map():
    """Equivalent to fix_edge_index + adjust_edge_index_nomerge of the reference."""
    n, s = 8, 4
    ei = torch.tensor([[1, 2, 7, 5], [0, 0, 3, 6]])
    g = add_virtual_node(AttnGraph.from_edge_index(ei, n), n, s)
    got = set(zip(g.col.tolist(), g.row_ids().tolist()))
    shifted = ei + 1
    virt = torch.arange(1, n + 1)
    full = torch.cat([shifted, torch.stack([virt, torch.zeros(n, dtype=torch.long)]),
                      torch.stack([torch.zeros(n, dtype=torch.long), virt])], 1)
    adj = full.clone()
    m = adj > 0
    adj[m] = adj[m] + torch.div(adj[m] - 1, s, rounding_mode="floor")
    want = set(zip(adj[0].tolist(), adj[1].tolist()))
    assert got == want and g.num_rows == n + 2


def test_coo_roundtrip_and_transpose():
    ei = torch.tensor([[3, 1, 2, 0, 3], [0, 0, 1, 2, 2]])
    g = AttnGraph.from_edge_index(ei, 4).ensure_transpose()
    back = g.edge_index()
    assert set(zip(back[0].tolist(), back[1].tolist())) == set(zip(ei[0].tolist(), ei[1].tolist()))
    for key in range(4):
        sl = slice(int(g.t_rowptr[key]), int(g.t_rowptr[key + 1]))
        assert all(int(g.col[e]) == key for e in g.t_eid[sl].tolist())


@pytest.mark.parametrize("fanout", [[3, 2], [-1, 2], [2, 2, 2]])
def test_native_fanout_expansion_equals_spec(fanout):
    """C++/OpenMP k-hop fan-out expansion (--rw_edge_mode dgl_neighbor) against the numpy specification: the same
    candidate multiset, and therefore the same attention graph."""
    import numpy as np
    from budgetformer_b200.graph import builder_spec as spec
    topo, _ = random_topology(400, 3000, hub_out=60, seed=4)
    ws, wd = spec.khop_neighbor_candidates(topo, fanout, 77)
    native = spec.khop_neighbor_candidates_native(topo, fanout, 77, num_threads=3)
    assert native is not None
    ns, nd = native
    a = np.sort(wd.astype(np.int64) * 400 + ws.astype(np.int64))
    b = np.sort(nd.astype(np.int64) * 400 + ns.astype(np.int64))
    assert a.size == b.size and bool((a == b).all())
    g1 = spec.build_attn_graph_spec(topo, 3, 4, 2, 3, 77, fanout=fanout)
    orig = spec.khop_neighbor_candidates_native
    spec.khop_neighbor_candidates_native = lambda *a, **k: None          # force the numpy expansion
    try:
        g2 = spec.build_attn_graph_spec(topo, 3, 4, 2, 3, 77, fanout=fanout)
    finally:
        spec.khop_neighbor_candidates_native = orig
    assert torch.equal(g1.rowptr, g2.rowptr) and torch.equal(g1.col, g2.col)


@pytest.mark.parametrize("exphormer", [False, True])
@pytest.mark.parametrize("fanout,b_real,b_rw", [([3, 2], 3, 4), ([-1, 2], 0, 5), ([2, 2, 2], 4, 0), ([4], 2, 40)])
def test_native_fanout_build_equals_spec(fanout, b_real, b_rw, exphormer):
    """The one-pass C++ build of the fan-out mode (expansion + per-query top-K + merge) is bit-identical to the numpy
    specification, type row and edge totals included."""
    from budgetformer_b200.graph import builder_spec as spec
    from budgetformer_b200.graph.builder import build_attn_graph
    topo, _ = random_topology(400, 3000, hub_out=60, seed=9)
    want = spec.build_attn_graph_spec(topo, b_real, b_rw, 2, 3, 123, exphormer=exphormer, fanout=fanout)
    got = build_attn_graph(topo, b_real, b_rw, 2, 3, 123, exphormer=exphormer, fanout=fanout, num_threads=3)
    assert got.max_degree is not None                                   # came from the native path
    assert torch.equal(got.rowptr, want.rowptr) and torch.equal(got.col, want.col)
    if exphormer:
        assert torch.equal(got.etype, want.etype)
    assert (got.n_real, got.n_rw) == (want.n_real, want.n_rw)
    deg = got.rowptr[1:] - got.rowptr[:-1]
    assert int(deg.max()) <= got.max_degree


def test_fanout_mode_is_not_gated_by_walks_per_node():
    """--rw_edge_mode dgl_neighbor builds its pool from the fan-out: walks_per_node = 0 keeps the walk side."""
    import types
    from budgetformer_b200.graph import builder_spec as spec
    from budgetformer_b200.graph.builder import build_attn_graph
    from budgetformer_b200.graph.engine import resolve_budget_state
    args = types.SimpleNamespace(walk_length=4, walks_per_node=0, rw_edge_mode="dgl_neighbor", include_real_edges=1)
    assert resolve_budget_state(args).use_rw
    assert resolve_budget_state(args, {"real_edges_per_query": 2, "rw_edges_per_query": 3}).use_rw
    args.rw_edge_mode = "random_walk"
    assert not resolve_budget_state(args).use_rw
    assert not resolve_budget_state(args, {"real_edges_per_query": 2, "rw_edges_per_query": 3}).use_rw
    topo, _ = random_topology(200, 1200, seed=2)
    g = build_attn_graph(topo, 2, 3, 0, 0, 5, fanout=[3, 2])
    s = spec.build_attn_graph_spec(topo, 2, 3, 0, 0, 5, fanout=[3, 2])
    assert g.n_rw > 0 and torch.equal(g.col, s.col) and torch.equal(g.rowptr, s.rowptr)


@pytest.mark.parametrize("exphormer", [False, True])
@pytest.mark.parametrize("b_real,b_rw,walks,length,fanout,use_real,use_rw", [
    (None, None, 2, 3, None, True, True),        # the reference's default: all real edges + the whole walk pool
    (None, 4, 2, 3, None, True, True),
    (40, 50, 6, 10, None, True, True),           # above the fixed-width limit
    (3, 3, 2, 20, None, True, True),             # walks longer than the CUDA builder takes
    (None, None, 2, 3, [3, 2], True, True),      # fan-out pool without budget
    (None, None, 2, 3, None, False, True),
    (None, None, 0, 0, None, True, True),        # no walks at all
    (0, None, 2, 3, None, True, True),
])
def test_general_native_build_equals_spec(b_real, b_rw, walks, length, fanout, use_real, use_rw, exphormer):
    from budgetformer_b200.graph import builder_spec as spec
    from budgetformer_b200.graph import builder
    topo, _ = random_topology(300, 2500, hub_out=50, seed=11)
    want = spec.build_attn_graph_spec(topo, b_real, b_rw, walks, length, 31, use_real=use_real, use_rw=use_rw,
                                      exphormer=exphormer, fanout=fanout)
    got = builder._build_rows_native(topo, b_real, b_rw, walks, length, 31, use_real, use_rw, exphormer, fanout, 3)
    assert got is not None
    assert torch.equal(got.rowptr, want.rowptr) and torch.equal(got.col, want.col)
    if exphormer:
        assert torch.equal(got.etype, want.etype)
    assert (got.n_real, got.n_rw) == (want.n_real, want.n_rw)
    via_dispatch = builder.build_attn_graph(topo, b_real, b_rw, walks, length, 31, use_real=use_real, use_rw=use_rw,
                                            exphormer=exphormer, fanout=fanout)
    assert torch.equal(via_dispatch.col, want.col)
