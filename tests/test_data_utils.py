import os

import numpy as np
import pytest
import torch

from budgetformer_b200.train.data import (GraphData, compute_multihop_features, generate_expander_edges,
                                          pad_to_sequence_parallel_world, random_split_idx, to_bidirected_edge_index)
from budgetformer_b200.utils.prepare_snap_patents import even_quantile_labels, prepare_labels
from budgetformer_b200.utils.preprocess_data import get_dataset, rand_train_test_idx
from budgetformer_b200.utils.split_utils import load_default_split


def test_random_split_is_seeded_60_20_20():
    a, b = random_split_idx(1000, 42), random_split_idx(1000, 42)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert (a["train"].numel(), a["valid"].numel(), a["test"].numel()) == (600, 200, 200)
    assert torch.cat(list(a.values())).unique().numel() == 1000


def test_padding_and_bidirected():
    d = GraphData(torch.randn(10, 3), torch.arange(10), torch.tensor([[0, 1], [1, 2]]), random_split_idx(10, 0), 10, 10)
    p = pad_to_sequence_parallel_world(d, 4)
    assert p.x.size(0) == 12 and p.y[-1] == -1 and float(p.x[-1].abs().sum()) == 0
    bi = to_bidirected_edge_index(torch.tensor([[0, 1, 1], [1, 0, 2]]), 3)
    assert set(map(tuple, bi.t().tolist())) == {(0, 1), (1, 0), (1, 2), (2, 1)}


def test_multihop_features_and_expander():
    ei = torch.tensor([[0, 1, 2], [1, 2, 3]])
    x = torch.eye(4)
    mh = compute_multihop_features(ei, 4, x, hops=2, rank=1)
    assert mh.shape == (4, 3, 4) and torch.allclose(mh[:, 0], x)
    assert torch.allclose(mh[:, 1].sum(1), mh[:, 1].sum(1))             # finite
    e = generate_expander_edges(50, 3, seed=1)
    deg = torch.bincount(e[0], minlength=50)
    assert int(deg.min()) >= 4 and int(deg.max()) <= 6 and bool((e[0] != e[1]).all())


def test_even_quantile_labels_and_cli(tmp_path):
    vals = np.arange(100, dtype=np.float64)
    lab = even_quantile_labels(vals, 5)
    assert np.bincount(lab).tolist() == [20, 20, 20, 20, 20]
    path = tmp_path / "snap-patents"
    os.makedirs(path)
    torch.save(torch.arange(1970, 2070), path / "y.pt")
    assert prepare_labels(str(path))
    y = torch.load(path / "y.pt")
    assert y.unique().tolist() == [0, 1, 2, 3, 4] and (path / "y_raw_year.pt").exists()
    assert not prepare_labels(str(path))                                  # idempotent


def test_split_discovery_layouts(tmp_path):
    root = tmp_path / "ds"
    os.makedirs(root / "a")
    torch.save({"train": torch.tensor([0, 1]), "val": torch.tensor([2]), "test": torch.tensor([3])}, root / "a" / "split_idx.pt")
    s = load_default_split("a", str(root))
    assert s["valid"].tolist() == [2]
    os.makedirs(root / "b")
    m = torch.zeros(5, 2, dtype=torch.bool); m[1, 1] = True
    for n in ("train", "val", "test"):
        torch.save(m, root / "b" / f"{n}_mask.pt")
    assert load_default_split("b", str(root), split_id=1)["train"].tolist() == [1]
    assert load_default_split("missing", str(root)) is None
    sp = rand_train_test_idx(100, seed=3)
    assert sp["train"].numel() == 50 and sp["valid"].numel() == 25


def test_synthetic_dataset_cli(tmp_path):
    p = get_dataset("synthetic:sbm2k", str(tmp_path))
    assert torch.load(os.path.join(p, "x.pt")).shape == (2048, 128)


def test_edge_set_analytics_and_legacy_samplers():
    import torch
    from budgetformer_b200.graph import legacy_samplers as ls
    from budgetformer_b200.utils import analytics as an
    a = torch.tensor([[0, 1, 2, 3, 3], [1, 2, 3, 0, 0]])
    b = torch.tensor([[0, 1, 4], [1, 2, 0]])
    assert an.edge_ids(a, 5).numel() == 4                              # duplicate (3, 0) counted once
    assert abs(an.edge_index_jaccard(a, b, 5) - 2 / 5) < 1e-9
    assert abs(an.edge_index_new_edge_ratio(a, b, 5) - 1 / 3) < 1e-9
    assert an.slice_edge_index(a, 1, 4).tolist() == [[0, 1], [1, 2]]
    assert abs(an.calculate_sparsity(a, 5) - (1 - 4 / 25)) < 1e-9
    p2 = an.calc_power_edge_index(torch.tensor([[0, 1], [1, 2]]), 3, 2)
    assert sorted(map(tuple, p2.t().tolist())) == [(0, 1), (0, 2), (1, 2)]
    sc = an.make_strongly_connected(torch.tensor([[0], [2]]), 4)
    assert an.calc_power_edge_index(sc, 4, 4).size(1) == 12            # every ordered pair reachable
    hops = an.bfs_hop_matrix(torch.tensor([[1, 2], [0, 1]]), 3, torch.tensor([0]))
    assert hops.tolist() == [[0, 1, 2]]
    tr = an.HopMassTracker(mass=0.9, max_hop=4, max_batches=2)
    tr.add_sparse(torch.tensor([0, 0, 0]), torch.tensor([0, 1, 2]), torch.tensor([0.5, 0.4, 0.1]))
    s = tr.summary()
    assert s["calls"] == 1 and abs(s["hop_mass"][1] - 0.4) < 1e-6 and s["hops_for_target_max"] == 1
    # samplers / head views
    e = torch.stack([torch.arange(10), torch.arange(10).flip(0)])
    assert ls.IdentitySubgraphSampler().sample(e, None, 10) is e
    kept = ls.EdgeDropSubgraphSampler(0.5, torch.Generator().manual_seed(0)).sample(e, None, 10)
    assert 0 < kept.size(1) <= 10
    views = ls.GroupedHeadSubgraphProvider(2).build(e, 4)
    assert len(views) == 4 and views[0] is views[1] and views[2] is views[3]
    assert bool((views[0][0] % 2 == 0).all()) and bool((views[2][0] % 2 == 1).all())
    hop_views = ls.HopMappedHeadSubgraphProvider([0, 1], 2).build([e[:, :3], e[:, 3:]], 4)
    assert hop_views[0].size(1) == 3 and hop_views[3].size(1) == 7
    assert len(ls.SharedHeadSubgraphProvider().build([None, e], 3)) == 3


def test_hop_mass_tracking_on_core_attention():
    import torch
    from budgetformer_b200.models.common import SparseCoreAttention
    from tests.helpers import random_attn_graph
    torch.manual_seed(0)
    core = SparseCoreAttention(32, 0.0, 4)
    core.enable_hop_mass_tracking(mass=0.9, max_batches=3, max_hop=8)
    g = random_attn_graph(50, 300, seed=2)
    core.edge_hops = torch.randint(0, 4, (g.num_edges,))
    q, k, v = (torch.randn(1, 50, 4, 8) for _ in range(3))
    out = core(q, k, v, edge_index=g)
    assert out.shape == (1, 50, 32)
    stats = core.get_hop_mass_stats()
    assert stats is not None and abs(sum(stats["hop_mass"]) - 1.0) < 1e-5
    assert core.get_head_mass_stats().shape == (4,)
    core.disable_hop_mass_tracking()
    assert core.get_hop_mass_stats() is None


def test_memory_mapped_load_matches_plain_load(tmp_path):
    from budgetformer_b200.utils.split_utils import safe_torch_load
    p = str(tmp_path / "x.pt")
    x = torch.randn(64, 8)
    torch.save(x, p)
    mapped = safe_torch_load(p, mmap=True)
    assert torch.equal(mapped, x) and mapped.float() is mapped        # fp32 stays mapped, no second copy
    mapped[0, 0] = 123.0                                              # private mapping: the file is not written
    assert torch.equal(safe_torch_load(p), x)
    old = str(tmp_path / "old.pt")
    torch.save(x, old, _use_new_zipfile_serialization=False)          # cannot be mapped: falls back to a plain load
    assert torch.equal(safe_torch_load(old, mmap=True), x)


def test_locality_reordering_is_an_isomorphism(tmp_path):
    import types
    from budgetformer_b200.graph.partition import edge_cut
    from budgetformer_b200.graph.synthetic import sbm_graph, write_dataset
    from budgetformer_b200.train.data import load_data, reorder_for_locality
    n = 1200
    x, y, ei = sbm_graph(n, blocks=4, p_in=0.03, p_out=0.001, feat_dim=6, seed=2)
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(1))      # hide the block structure in the ids
    inv = torch.empty(n, dtype=torch.long)
    inv[perm] = torch.arange(n)
    write_dataset(str(tmp_path), "g", x[inv], y[inv], perm[ei])
    ns = lambda k: types.SimpleNamespace(dataset_dir=str(tmp_path), dataset="g", force_random_split=True, seed=3,
                                         locality_reorder_parts=k)
    plain, re = load_data(ns(0)), load_data(ns(4))
    assert plain.node_order is None and torch.equal(torch.sort(re.node_order).values, torch.arange(n))
    # features, labels and splits follow their nodes
    assert torch.equal(re.x, plain.x[re.node_order]) and torch.equal(re.y, plain.y[re.node_order])
    for k in plain.split_idx:
        assert torch.equal(torch.sort(re.node_order[re.split_idx[k]]).values, torch.sort(plain.split_idx[k]).values)
    # the same edge set in the old ids
    back = re.node_order[re.edge_index]
    assert torch.equal(torch.unique(back[0] * n + back[1]), torch.unique(plain.edge_index[0] * n + plain.edge_index[1]))
    # contiguous id ranges are now clusters: far fewer edges cross the four ranges
    ranges = lambda m: torch.arange(m) * 4 // m
    assert edge_cut(re.edge_index, ranges(n)) < 0.25 * edge_cut(plain.edge_index, ranges(n))
    # padded rows stay where they are
    padded = pad_to_sequence_parallel_world(plain, 7)
    again = reorder_for_locality(padded, 4)
    assert again.x.size(0) == padded.x.size(0) and float(again.x[n:].abs().sum()) == 0.0


# ---------------------------------------------------------------------------------------------- offline converters
def _tiny_raw(n=30, classes=4, seed=0):
    import numpy as np
    import scipy.sparse as sp
    rng = np.random.default_rng(seed)
    rows, cols = rng.integers(0, n, 120), rng.integers(0, n, 120)
    adj = sp.coo_matrix((np.ones(120, dtype=np.float32), (rows, cols)), shape=(n, n)).tocsr()   # duplicates get summed
    feat = rng.normal(size=(n, 6)).astype(np.float32)
    cls = rng.integers(0, classes, n)
    onehot = np.eye(classes, dtype=np.float32)[cls]
    return adj, feat, cls, onehot


def _check_written(path, adj, feat, cls):
    import numpy as np
    x, y, ei = (torch.load(os.path.join(path, f)) for f in ("x.pt", "y.pt", "edge_index.pt"))
    assert torch.allclose(x, torch.as_tensor(feat)) and y.tolist() == cls.tolist() and ei.dtype == torch.int64
    want = sorted(set(zip(*adj.nonzero())))
    assert sorted(zip(ei[0].tolist(), ei[1].tolist())) == [(int(a), int(b)) for a, b in want]     # coalesced


def test_offline_converters_from_raw_files(tmp_path):
    import json
    import pickle
    import numpy as np
    import scipy.io
    import scipy.sparse as sp
    from budgetformer_b200.utils.preprocess_data import get_dataset
    root = str(tmp_path)
    adj, feat, cls, onehot = _tiny_raw()
    # aminer: pickles next to the output
    d = tmp_path / "aminer"; d.mkdir()
    for name, obj in (("adj.sp", adj), ("features", feat), ("labels", onehot)):
        pickle.dump(obj, open(d / f"aminer.{name}.pkl", "wb"))
    _check_written(get_dataset("aminer", root), adj, feat, cls)
    # reddit / Amazon2M: npz + npy under raw/<name>
    for name in ("reddit", "Amazon2M"):
        d = tmp_path / "raw" / name; d.mkdir(parents=True)
        sp.save_npz(d / f"{name}_adj.npz", adj); np.save(d / f"{name}_feat.npy", feat); np.save(d / f"{name}_labels.npy", onehot)
        _check_written(get_dataset(name, root), adj, feat, cls)
    # GraphSAINT amazon with its role.json split
    d = tmp_path / "raw" / "amazon"; d.mkdir(parents=True)
    sp.save_npz(d / "adj_full.npz", adj); np.save(d / "feats.npy", feat); np.save(d / "labels.npy", onehot)
    role = {"tr": list(range(0, 24)), "va": [24, 25], "te": [26, 27, 28, 29]}
    json.dump(role, open(d / "role.json", "w"))
    path = get_dataset("amazon", root)
    _check_written(path, adj, feat, cls)
    split = torch.load(os.path.join(path, "split_idx.pt"))
    assert split["train"].tolist() == role["tr"] and split["valid"].tolist() == role["va"] and split["test"].tolist() == role["te"]
    assert json.load(open(os.path.join(path, "role.json"))) == role
    # LINKX .mat files: pokec as is, genius with five seeded splits over its labelled nodes
    coo = adj.tocoo()
    ei = np.stack([coo.row, coo.col]).astype(np.int64)
    lab = cls.copy(); lab[:5] = -1
    d = tmp_path / "raw"
    scipy.io.savemat(d / "pokec.mat", {"edge_index": ei, "node_feat": feat, "label": lab.reshape(1, -1)})
    scipy.io.savemat(d / "genius.mat", {"edge_index": ei, "node_feat": feat, "label": lab.reshape(1, -1)})
    p = get_dataset("pokec", root)
    assert torch.load(os.path.join(p, "y.pt")).tolist() == lab.tolist() and not os.path.exists(os.path.join(p, "split_idx.pt"))
    g = get_dataset("genius", root, split_id=3)
    all_splits = torch.load(os.path.join(g, "split_idx_all.pt"))
    assert len(all_splits) == 5
    chosen = torch.load(os.path.join(g, "split_idx.pt"))
    assert chosen["train"].tolist() == all_splits[3]["train"].tolist()
    for s in all_splits:
        ids = torch.cat([s["train"], s["valid"], s["test"]])
        assert sorted(ids.tolist()) == list(range(5, 30))                    # unlabelled nodes are in no part
        assert len(s["train"]) == 12 and len(s["valid"]) == 6                # 50 / 25 / 25 of the 25 labelled nodes
    assert all_splits[0]["train"].tolist() != all_splits[1]["train"].tolist()
    with pytest.raises(SystemExit):
        get_dataset("genius", root, split_id=7)
    with pytest.raises(SystemExit):
        get_dataset("aminer", str(tmp_path / "nowhere"))


def test_device_chung_lu_generator_gives_the_requested_graph():
    from budgetformer_b200.graph.synthetic import chung_lu_edges_device
    n, e = 5000, 40000
    ei = chung_lu_edges_device(n, e, 2.1, True, 7, "cpu")
    assert ei.shape == (2, e) and ei.dtype == torch.int64 and int((ei[0] == ei[1]).sum()) == 0
    assert torch.unique(ei[0] * n + ei[1]).numel() == e                       # distinct pairs, exactly the requested count
    assert torch.equal(ei, chung_lu_edges_device(n, e, 2.1, True, 7, "cpu"))   # deterministic in the seed
    assert int(torch.bincount(ei[1], minlength=n).max()) > 50 * e // n        # heavy tail: a hub far above the mean degree
    und = chung_lu_edges_device(n, e // 2, 2.1, False, 7, "cpu")
    assert und.shape == (2, e)
    fwd = set(zip(und[0].tolist(), und[1].tolist()))
    assert all((b, a) in fwd for a, b in fwd)                                 # both directions present
