"""Helpers of the legacy mini-batch / graph-level paths (train/legacy_utils.py)."""
import random
import types

import numpy as np
import pytest
import scipy.sparse as sp
import torch

from budgetformer_b200.graph.attn_graph import Topology
from budgetformer_b200.parallel import initialize as init
from budgetformer_b200.train import legacy_utils as L


@pytest.fixture(autouse=True)
def _clean_state():
    init.reset_state()
    yield
    init.reset_state()


def test_scoped_seeding_restores_every_generator():
    random.seed(1); np.random.seed(1); torch.manual_seed(1)
    expect = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    random.seed(1); np.random.seed(1); torch.manual_seed(1)
    for ctx in (L.fixed_random_seed, L.fixed_random_seed_cpu):
        with ctx(99):
            a = (random.random(), float(np.random.rand()), float(torch.rand(1)))
        with ctx(99):
            b = (random.random(), float(np.random.rand()), float(torch.rand(1)))
        assert a == b
    assert (random.random(), float(np.random.rand()), float(torch.rand(1))) == expect


def test_padding_family():
    assert L.pad_y(torch.tensor([1, 2]), 4).tolist() == [1, 2, -100, -100]
    assert L.pad_y(torch.tensor([1, 2]), 1).tolist() == [1, 2]                      # never truncates
    x = torch.ones(2, 3)
    assert L.pad_2d(x, 5).shape == (5, 3) and float(L.pad_2d(x, 5).sum()) == 6.0
    assert L.pad_attn_bias(torch.ones(2, 2, 4), 3).shape == (3, 3, 4)
    assert L.pad_2d_bs(torch.ones(2, 3), 5).shape == (2, 5)
    assert L.pad_x_bs(torch.ones(2, 3, 7), 5).shape == (2, 5, 7)
    assert L.pad_4d_bs(torch.ones(2, 3, 4, 5), 6).shape == (2, 6, 4, 5)
    # world size 1 outside an initialised SP group
    assert L.pad_3d_bs(torch.ones(2, 3, 3), 4).shape == (2, 4, 4)
    assert L.pad_5d_bs(torch.ones(2, 3, 3, 2, 2), 4).shape == (2, 4, 4, 2, 2)
    assert L.pad_attn_bias_bs(torch.ones(2, 3, 3), 4).shape == (2, 4, 4)
    assert L.pad_spatial_pos_bs_unsplit(torch.ones(2, 3, 3), 4).shape == (2, 4, 4)
    assert L.pad_edge_input_bs_unsplit(torch.ones(2, 3, 3, 1, 1), 4).shape == (2, 4, 4, 1, 1)
    b = L.pad_attn_bias_bs_unsplit(torch.zeros(2, 3, 3), 4, torch.tensor([2, 3]))
    assert b.shape == (2, 5, 5)
    assert torch.isinf(b[0, :3, 3:]).all() and (b[0, 3:, :2] == 0).all() and torch.isinf(b[0, 3:, 2:]).all()
    assert (b[1, 3:, :3] == 0).all()
    assert torch.softmax(b[0], -1).isfinite().all()


def test_virtual_node_edge_lists_match_the_csr_construction():
    ei = torch.tensor([[0, 1, 2], [1, 2, 0]])
    fixed = L.fix_edge_index(ei, 3)
    assert fixed.shape == (2, 3 + 6)
    assert fixed[:, :3].tolist() == [[1, 2, 3], [2, 3, 1]]
    assert set(map(tuple, fixed[:, 3:].t().tolist())) == {(1, 0), (2, 0), (3, 0), (0, 1), (0, 2), (0, 3)}
    # 4 real nodes, 2 per rank: rows are [tok, n1, n2, tok, n3, n4]
    ids = torch.tensor([[0, 1, 2, 3, 4]])
    assert L.adjust_edge_index_nomerge(ids, 2).tolist() == [[0, 1, 2, 4, 5]]


def _adjs(n, d=3, seed=0):
    rng = np.random.default_rng(seed)
    a = sp.random(n, n, density=0.3, random_state=rng, format="csr", dtype=np.float32)
    out = [a]
    for _ in range(d - 1):
        out.append((out[0] @ out[-1]).tocsr())
    return out


def test_get_batch_dense_bias_single_rank_and_short_sequence():
    n = 12
    adjs = _adjs(n)
    x, y = torch.randn(n, 5), torch.arange(n)
    args = types.SimpleNamespace(seq_len=6)
    idx = torch.tensor([3, 1, 7, 9, 0, 4])
    xi, yi, bias = L.get_batch(args, x, y, idx, adjs)
    assert torch.equal(xi, x[idx]) and torch.equal(yi, y[idx]) and bias.shape == (6, 6, 3)
    assert torch.allclose(bias[2, 4, 1], torch.tensor(float(adjs[1][7, 0])))
    assert init.get_last_batch_flag() is False
    short = torch.tensor([2, 5, 8])
    xi, yi, bias = L.get_batch(args, x, y, short, adjs, rest_split_sizes=[3])
    assert xi.shape == (3, 5) and bias.shape == (3, 3, 3) and init.get_last_batch_flag() is True


def test_get_batch_papers100m_shapes_and_token_reindexing():
    n = 10
    ei = torch.tensor([[0, 1, 2, 3, 4, 5], [1, 2, 3, 4, 5, 0]])
    x, y = torch.randn(n, 4), torch.arange(n)
    args = types.SimpleNamespace(seq_len=4, world_size=2, model="graphormer")
    idx = torch.tensor([0, 1, 2, 3])
    xi, yi, bias, e = L.get_batch_papers100m(args, x, y, idx, None, None, "cpu", ei, n)
    assert xi.shape == (4, 4) and bias is None
    # induced edges 0->1, 1->2, 2->3 become (1,2), (2,4), (4,5) in the [tok, a, b, tok, c, d] row numbering
    assert e[:, :3].tolist() == [[1, 2, 4], [2, 4, 5]]
    short = torch.tensor([4, 5, 6])
    xi, yi, _, e = L.get_batch_papers100m(args, x, y, short, None, [2, 1], "cpu", ei, n)
    assert xi.shape == (4, 4) and yi.tolist() == [4, 5, 6, -100]
    args.model = "gt"
    _, _, _, e = L.get_batch_papers100m(args, x, y, idx, None, None, "cpu", ei, n)
    assert e.tolist() == [[0, 1, 2], [1, 2, 3]]


def test_graph_level_loader_batches():
    def make():
        return types.SimpleNamespace(x=torch.arange(2 * 7 * 1).reshape(2, 7, 1), in_degree=torch.ones(2, 7, dtype=torch.long),
                                     out_degree=torch.ones(2, 7, dtype=torch.long), attn_bias=torch.zeros(2, 8, 8),
                                     sub_split_seq_lens=[4, 3])
    args = types.SimpleNamespace(num_global_node=1, dummy_bias=True, world_size=2)
    b = make()
    xs, ins, outs, tokens = L.get_batch_from_loader_malnet(args, b)
    assert [t.shape for t in xs] == [(2, 4, 1), (2, 4, 1)] and tokens == [0, 5] and b.attn_bias is None
    assert xs[1][0, :, 0].tolist() == [4, 5, 6, 0] and ins[1][0].tolist() == [1, 1, 1, 0]
    b = make()
    L.get_batch_from_loader(args, b)                      # one rank: the first slice, tokens for a world of one
    assert b.x.shape == (2, 4, 1) and b.global_token_indices == [0] and not hasattr(b, "sub_split_seq_lens")


def test_global_token_merge_and_extend():
    init.set_global_token_indices([0, 3])
    x = torch.arange(6, dtype=torch.float32).reshape(1, 6, 1)       # rows: tok a b tok c d
    assert L.merge_global_token(x, 1).flatten().tolist() == [1, 2, 4, 5, 1.5]
    assert L.merge_global_token0(x, 1).flatten().tolist() == [1.5, 1, 2, 4, 5]
    # world size 1: extend keeps one chunk and appends / prepends the token
    y = torch.arange(5, dtype=torch.float32).reshape(1, 5, 1)
    assert L.extend_global_token0(y, 1).flatten().tolist() == [0, 1, 2, 3, 4]
    assert len(L.split_tensor_along_second_dim(torch.zeros(1, 6, 2), 3)) == 3
    assert L.split_tensor_along_second_dim(torch.zeros(1, 6, 2), 3, True)[0].is_contiguous()


def _ring_topology(n=24):
    s = torch.arange(n)
    ei = torch.stack([torch.cat([s, s]), torch.cat([(s + 1) % n, (s + 5) % n])])
    return Topology.from_edge_index(ei, n), ei


def test_random_walk_groups():
    topo, ei = _ring_topology()
    n = topo.num_nodes
    buckets = L.compute_hops_random_walk(topo, walk_length=4, walks_per_node=2, num_groups=2, seed=3)
    assert len(buckets) == 2 and all(b.shape[0] == 2 for b in buckets)
    assert buckets[0].numel() > 0
    # a node is an end point in one hop only, and hops alternate between the groups
    assert not bool(torch.isin(buckets[0][1].unique(), buckets[1][1].unique()).any())
    again = L.compute_hops_random_walk(topo, walk_length=4, walks_per_node=2, num_groups=2, seed=3)
    assert all(torch.equal(a, b) for a, b in zip(buckets, again))
    groups = L.compute_group_nodes_random_walk(topo, walk_length=3, walks_per_node=2, num_groups=4,
                                               max_nodes_per_group=10, seed=1)
    assert len(groups) == 4
    for g, nodes in enumerate(groups):
        assert nodes.numel() <= 10 and nodes.unique().numel() == nodes.numel()
        assert nodes[:6].tolist() == list(range(g, n, 4))                           # the seeds come first


def test_check_conditions():
    _, ei = _ring_topology(8)
    loops = torch.arange(8).repeat(2, 1)
    assert not L.check_conditions(ei, 8)                                            # no self loops
    assert L.check_conditions(torch.cat([ei, loops], 1), 8)
    two = torch.tensor([[0, 1, 2, 3], [1, 0, 3, 2]])
    assert not L.check_conditions(torch.cat([two, torch.arange(4).repeat(2, 1)], 1), 4)   # two components


def test_legacy_sequence_files(tmp_path):
    import os
    from budgetformer_b200.utils import preprocess_data as pd
    n = 30
    s = torch.arange(n)
    ei = torch.stack([torch.cat([s, (s + 1) % n]), torch.cat([(s + 1) % n, s])])
    pd.save_dataset(str(tmp_path), "ring", torch.randn(n, 4), s % 3, ei)
    a = pd.adjacency(ei, n)
    norm = pd.adj_normalize(a)
    assert abs(float(norm[0, 0]) - 1 / 3) < 1e-6 and abs(float(norm[0, 1]) - 1 / 3) < 1e-6     # degree 2 (+1) everywhere
    assert abs(float(pd.column_normalize(a).sum(0).max()) - 1.0) < 1e-6
    assert pd.eigenvector(np.eye(n) - np.asarray(norm.todense()), 4).shape == (n, 4)
    path = pd.process_data(str(tmp_path), "ring", k1=5, seed=1)
    recs = torch.load(path)
    assert len(recs) == n
    bias, ids, y = recs[7][0]
    assert ids[0] == 7 and ids.numel() == 6 and ids.unique().numel() == 6 and bias.shape == (6, 6, 6)
    assert torch.equal(y, ids % 3)
    assert bool(torch.isin(torch.tensor([6, 8]), ids).all())         # nearest neighbours carry most PPR mass
    path = pd.rand_nodes_seq(str(tmp_path), "ring", k1=8, seed=2)
    recs = torch.load(path)
    assert [r[0][1].numel() for r in recs] == [8, 8, 8, 6]
    assert torch.cat([r[0][1] for r in recs]).unique().numel() == n
    assert os.path.basename(path) == "data_rand8.pt"
    # the records feed the dense-bias batcher
    args = types.SimpleNamespace(seq_len=8)
    powers = pd.power_adjacency_list(norm, 6)
    xi, yi, b = L.get_batch(args, torch.randn(n, 4), s % 3, recs[0][0][1], powers)
    assert torch.allclose(b, recs[0][0][0])


def test_preprocess_cli_writes_sequence_files(tmp_path):
    import os
    from budgetformer_b200.utils import preprocess_data as pd
    pd.main(["--dataset", "synthetic:sbm2k", "--dataset_dir", str(tmp_path), "--sequences", "rand", "--k1", "512"])
    recs = torch.load(os.path.join(str(tmp_path), "sbm2k", "data_rand512.pt"))
    assert len(recs) == 4 and recs[0][0][0].shape == (512, 512, 6)


def test_hop_buckets_feed_the_per_head_group_attention_path():
    """Legacy per-head subgraphs end to end: random-walk hop buckets -> hop-mapped head views -> a GT forward whose
    head groups attend over their own bucket."""
    from budgetformer_b200.config import parse_fullgraph_args
    from budgetformer_b200.graph.legacy_samplers import HopMappedHeadSubgraphProvider
    from budgetformer_b200.train.engine import build_model
    topo, ei = _ring_topology(32)
    n = topo.num_nodes
    buckets = L.compute_hops_random_walk(topo, walk_length=4, walks_per_node=2, num_groups=2, seed=4)
    loops = torch.arange(n).repeat(2, 1)
    # walk edges are (start, reached): the start node is the query, so flip them into (key, query) and add self loops
    buckets = [torch.cat([b.flip(0), loops], 1) for b in buckets]
    views = HopMappedHeadSubgraphProvider([0, 1], 2).build(buckets, 4)
    assert len(views) == 4 and views[0] is views[1] and views[2] is views[3] and views[0] is not views[2]
    a = parse_fullgraph_args(["--dataset", "x", "--model", "gt", "--n_layers", "1", "--hidden_dim", "32", "--num_heads", "4"])
    m = build_model(a, 6, 3).eval()
    with torch.no_grad():
        out = m(torch.randn(n, 6), None, [views[0], views[2]], attn_type="sparse")
    assert out.shape == (n, 3) and torch.isfinite(out).all()


def test_hop_buckets_and_shared_pool_match_the_builder_candidates():
    import numpy as np
    from budgetformer_b200.graph.builder_spec import random_walks, rw_candidates
    topo, _ = _ring_topology(40)
    pool = L.build_head_hop_edges(topo, walk_length=4, walks_per_node=2, seed=9)
    src, dst = rw_candidates(random_walks(topo, 2, 4, 9))               # what the full-graph builder samples from
    key = lambda s, d: np.sort(np.asarray(d) * 40 + np.asarray(s))
    assert np.array_equal(key(pool[0].numpy(), pool[1].numpy()), key(src, dst))
    buckets = L.compute_hop_buckets_random_walk(topo, 3, walk_length=4, walks_per_node=2, seed=9)
    assert len(buckets) == 3 and sum(b.size(1) for b in buckets) == pool.size(1)
    far = L.build_head_hop_edges(topo, walk_length=4, walks_per_node=2, min_hop=2, seed=9)
    assert far.size(1) == pool.size(1) - buckets[0].size(1)             # hop 1 left out


def test_map_global_nodes_to_local():
    from budgetformer_b200.train.legacy_batch import map_global_nodes_to_local
    sample = torch.tensor([40, 7, 19, 3])
    assert map_global_nodes_to_local(torch.tensor([3, 40, 19, 19, 7]), sample).tolist() == [3, 0, 2, 2, 1]
    assert map_global_nodes_to_local(torch.zeros(0, dtype=torch.long), sample).numel() == 0
