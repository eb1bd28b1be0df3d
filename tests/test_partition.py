"""Locality partition / reordering of the legacy mini-batch path (graph/partition.py, csrc/cpu/partition.cpp)."""
import types

import pytest
import torch

from budgetformer_b200.graph import partition as P
from budgetformer_b200.train.legacy_batch import get_batch_blockize, get_batch_reorder_blockize, induced_subgraph


def _clustered_graph(k=4, per=60, p_in=0.25, n_cross=12, seed=0):
    """k dense clusters with a few cross edges; node ids shuffled so that id order carries no locality."""
    g = torch.Generator().manual_seed(seed)
    n = k * per
    src, dst = [], []
    for c in range(k):
        a = torch.rand(per, per, generator=g) < p_in
        s, d = torch.nonzero(a, as_tuple=True)
        src.append(s + c * per)
        dst.append(d + c * per)
    cs = torch.randint(0, n, (n_cross,), generator=g)
    cd = torch.randint(0, n, (n_cross,), generator=g)
    ei = torch.stack([torch.cat(src + [cs]), torch.cat(dst + [cd])])
    ei = ei[:, ei[0] != ei[1]]
    shuffle = torch.randperm(n, generator=g)
    truth = torch.empty(n, dtype=torch.long)
    truth[shuffle] = torch.arange(n) // per
    return shuffle[ei], n, truth


def test_partition_is_balanced_and_cuts_few_edges():
    ei, n, truth = _clustered_graph()
    part = P.partition_assignment(ei, n, 4)
    assert part.shape == (n,) and int(part.min()) >= 0 and int(part.max()) <= 3
    sizes = torch.bincount(part, minlength=4)
    assert int(sizes.max()) <= int(1.03 * n / 4) + 1 and int(sizes.min()) >= int(0.97 * n / 4) - 1
    cut, planted, naive = P.edge_cut(ei, part), P.edge_cut(ei, truth), P.edge_cut(ei, torch.arange(n) * 4 // n)
    assert cut <= 3 * planted + 8, (cut, planted)           # close to the planted clusters
    assert cut < naive // 4, (cut, naive)                   # far better than cutting the shuffled id order
    # deterministic
    assert torch.equal(part, P.partition_assignment(ei, n, 4))


def test_partition_handles_isolated_nodes_components_and_large_k():
    ei = torch.tensor([[0, 1, 2, 5, 6], [1, 2, 0, 6, 5]])
    part = P.partition_assignment(ei, 9, 3)                  # nodes 3, 4, 7, 8 have no edge
    sizes = torch.bincount(part, minlength=3)
    assert int(sizes.sum()) == 9 and int(sizes.min()) >= 2 and int(sizes.max()) <= 4
    assert len(set(part[[0, 1, 2]].tolist())) == 1           # the triangle stays together
    assert P.partition_assignment(ei, 9, 50).unique().numel() == 9      # k clipped to n
    assert P.partition_assignment(torch.zeros(2, 0, dtype=torch.long), 0, 4).numel() == 0
    assert torch.equal(P.partition_assignment(ei, 9, 1), torch.zeros(9, dtype=torch.long))


def test_rcm_stand_in_gives_a_balanced_partition():
    ei, n, _ = _clustered_graph(seed=3)
    rowptr, col = P.symmetric_csr(ei, n)
    part = P._rcm_ranges(rowptr, col, n, 4)
    assert torch.bincount(part, minlength=4).tolist() == [n // 4] * 4
    assert P.edge_cut(ei, part) < P.edge_cut(ei, torch.arange(n) * 4 // n)


def test_reformat_graph_contract():
    ei, n, _ = _clustered_graph(seed=1)
    new_ei, old_of_new = P.reformat_graph(ei, 4, num_nodes=n)
    assert new_ei.shape == ei.shape and torch.equal(torch.sort(old_of_new).values, torch.arange(n))
    assert bool((new_ei[0][1:] >= new_ei[0][:-1]).all())                  # sorted by new source id
    back = old_of_new[new_ei]                                               # the same edge set in old ids
    assert torch.equal(torch.unique(back[0] * n + back[1]), torch.unique(ei[0] * n + ei[1]))
    part = P.partition_assignment(ei, n, 4)
    assert bool((part[old_of_new][1:] >= part[old_of_new][:-1]).all())     # contiguous id range per part


def test_gen_sub_edge_index_matches_the_batcher_helper():
    ei, n, _ = _clustered_graph(seed=2)
    idx = torch.randperm(n, generator=torch.Generator().manual_seed(5))[:70]
    a, b = P.gen_sub_edge_index(ei, idx, n), induced_subgraph(ei, idx, n)
    assert torch.equal(a, b)
    assert torch.equal(idx[a], ei[:, torch.isin(ei[0], idx) & torch.isin(ei[1], idx)])


def test_reordered_batch_keeps_more_edges_inside_a_rank():
    ei, n, _ = _clustered_graph(seed=4)
    feature = torch.arange(n, dtype=torch.float32)[:, None].repeat(1, 3)   # row i carries its own node id
    y = torch.arange(n) % 7
    args = types.SimpleNamespace(batch_subgraph_mode="induced", model="gt", num_global_node=0, attn_bias_mode="none",
                                 seq_len=n, batch_reorder_parts=0)
    idx = torch.arange(n)
    world = 4

    def local_share(fn, **kw):
        rows, inside, total = [], 0, 0
        for r in range(world):
            x, yy, graph, _bias, ok = fn(args, feature, y, idx, ei, n, r, world, **kw)
            assert bool(ok.all()) and torch.equal(yy, x[:, 0].long() % 7)  # labels travel with their features
            rows.append(x[:, 0].long())
        order = torch.cat(rows)
        assert torch.equal(torch.sort(order).values, idx)                  # a permutation of the batch
        pos = torch.empty(n, dtype=torch.long)
        pos[order] = torch.arange(n)
        s = n // world
        return float((pos[ei[0]] // s == pos[ei[1]] // s).float().mean()), graph

    plain, g0 = local_share(get_batch_blockize)
    reordered, g1 = local_share(get_batch_reorder_blockize, k=world)
    assert g0.num_edges == g1.num_edges
    assert reordered > 0.9 and plain < 0.5, (plain, reordered)


def test_multilevel_partition_recovers_planted_communities():
    """Shuffled ids, 8 planted blocks of a stochastic block model: the multilevel partitioner finds a cut as small as
    the planted one (a breadth-first ordering alone cannot: the frontier leaves a block after two hops)."""
    from budgetformer_b200.graph.synthetic import sbm_graph
    from budgetformer_b200.ops import _ext
    if not _ext.available():
        pytest.skip("needs the native partitioner")
    n, blocks = 8000, 8
    _, y, ei = sbm_graph(n, blocks=blocks, p_in=0.01, p_out=0.0003, feat_dim=4, seed=1)
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(0))
    ei, truth = perm[ei], torch.empty(n, dtype=torch.long)
    truth[perm] = y
    part = P.partition_assignment(ei, n, blocks)
    sizes = torch.bincount(part, minlength=blocks)
    assert int(sizes.max()) <= int(1.03 * n / blocks) + 1 and int(sizes.min()) >= int(0.97 * n / blocks) - 1
    assert P.edge_cut(ei, part) <= 1.1 * P.edge_cut(ei, truth)


def test_host_bench_cases_run(capsys):
    import json
    from budgetformer_b200.utils import host_bench
    host_bench.main(["build", "--nodes", "3000", "--edges", "12000", "--iters", "1", "--spec"])
    host_bench.main(["partition", "--nodes", "4000", "--parts", "4"])
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert len(lines) == 8 and all(l["seconds"] >= 0 for l in lines)
    assert all(l["identical"] for l in lines if "identical" in l)
    assert lines[-2]["cut"] < lines[-2]["cut_id_order"]
