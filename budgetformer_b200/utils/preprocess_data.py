"""Dataset preparation CLI: writes the on-disk contract ``<dataset_dir>/<name>/{x.pt, y.pt, edge_index.pt[, split_idx.pt]}``.

``python -m budgetformer_b200.utils.preprocess_data --dataset <name> [--dataset_dir ./dataset/] [--split_id 0]``

Sources (utils/preprocess_data.py:161-427 in the reference): Planetoid, CitationFull, Coauthor, Amazon Photo /
Computers, HeterophilousGraphDataset (PyG); ogbn-arxiv / products / papers100M (OGB); and, converted offline from raw
files that are already on disk (searched in ``<dataset_dir>/<name>/``, ``<dataset_dir>/raw/<name>/``,
``<dataset_dir>/raw/``): ``aminer`` (pickled scipy adjacency / features / one-hot labels), ``reddit`` and ``Amazon2M``
(``<name>_adj.npz``, ``<name>_feat.npy``, ``<name>_labels.npy``), ``amazon`` (GraphSAINT ``adj_full.npz`` / ``feats.npy``
/ ``labels.npy`` with the official ``role.json`` split), ``pokec`` / ``snap-patents`` / ``genius`` (LINKX ``.mat``
files; genius gets five seeded 50/25/25 splits over its labelled nodes, all of them in ``split_idx_all.pt``); and
``synthetic:<config>`` which generates the benchmark graphs of this repository without any download.
PyG / OGB are optional: when they are not importable the corresponding names fail with a clear message.

The legacy dense-bias sequence files are kept as well (utils/preprocess_data.py:25-50,431-555 in the reference):
``adj_normalize`` / ``column_normalize`` / ``eigenvector``, ``process_data`` (one sequence per node: the node plus
``k1`` neighbours drawn from its personalised-PageRank row, with the powers of the normalised adjacency as attention
bias) and ``rand_nodes_seq`` (disjoint random sequences of ``k1`` nodes); ``--sequences ppr|rand --k1 K``."""
from __future__ import annotations

import argparse
import os
from typing import Optional

import numpy as np
import torch

PYG_SETS = {
    "cora": ("Planetoid", "Cora"), "citeseer": ("Planetoid", "CiteSeer"), "pubmed": ("Planetoid", "PubMed"),
    "dblp": ("CitationFull", "DBLP"), "cora_full": ("CitationFull", "Cora"),
    "cs": ("Coauthor", "CS"), "physics": ("Coauthor", "Physics"),
    "photo": ("Amazon", "Photo"), "computers": ("Amazon", "Computers"),
    "roman-empire": ("HeterophilousGraphDataset", "Roman-empire"), "amazon-ratings": ("HeterophilousGraphDataset", "Amazon-ratings"),
    "minesweeper": ("HeterophilousGraphDataset", "Minesweeper"), "tolokers": ("HeterophilousGraphDataset", "Tolokers"),
    "questions": ("HeterophilousGraphDataset", "Questions"),
}


def rand_train_test_idx(n: int, train_prop: float = 0.5, valid_prop: float = 0.25, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n, generator=g)
    a, b = int(train_prop * n), int((train_prop + valid_prop) * n)
    return {"train": perm[:a], "valid": perm[a:b], "test": perm[b:]}


def save_dataset(root: str, name: str, x, y, edge_index, split=None, splits_all=None) -> str:
    path = os.path.join(root, name)
    os.makedirs(path, exist_ok=True)
    torch.save(torch.as_tensor(x).float(), os.path.join(path, "x.pt"))
    torch.save(torch.as_tensor(y), os.path.join(path, "y.pt"))
    torch.save(torch.as_tensor(edge_index).long(), os.path.join(path, "edge_index.pt"))
    if split is not None:
        torch.save(split, os.path.join(path, "split_idx.pt"))
    if splits_all is not None:
        torch.save(splits_all, os.path.join(path, "split_idx_all.pt"))
    return path


def _masks_to_split(data, split_id: int) -> Optional[dict]:
    if not all(hasattr(data, a) for a in ("train_mask", "val_mask", "test_mask")):
        return None
    pick = lambda m: (m[:, split_id] if m.dim() == 2 else m).nonzero().reshape(-1)
    return {"train": pick(data.train_mask), "valid": pick(data.val_mask), "test": pick(data.test_mask)}


def _from_pyg(name: str, root: str, split_id: int):
    try:
        import torch_geometric.datasets as D
    except ImportError as e:
        raise SystemExit(f"dataset {name!r} needs torch_geometric, which is not installed") from e
    cls, sub = PYG_SETS[name]
    ds = getattr(D, cls)(root=os.path.join(root, "raw", name)) if sub is None else getattr(D, cls)(root=os.path.join(root, "raw"), name=sub)
    data = ds[0]
    return data.x, data.y.reshape(-1), data.edge_index, _masks_to_split(data, split_id)


def _from_ogb(name: str, root: str):
    try:
        from ogb.nodeproppred import NodePropPredDataset
    except ImportError as e:
        raise SystemExit(f"dataset {name!r} needs the ogb package, which is not installed") from e
    ds = NodePropPredDataset(name=name, root=os.path.join(root, "raw"))
    graph, label = ds[0]
    split = {k: torch.as_tensor(v) for k, v in ds.get_idx_split().items()}
    return graph["node_feat"], torch.as_tensor(label).reshape(-1), graph["edge_index"], split


def find_raw(root: str, name: str, files) -> str:
    """Folder that holds every file of ``files`` for dataset ``name``; exits with the list of places searched."""
    places = [os.path.join(root, name), os.path.join(root, "raw", name), os.path.join(root, "raw")]
    for d in places:
        if all(os.path.exists(os.path.join(d, f)) for f in files):
            return d
    raise SystemExit(f"dataset {name!r}: put {', '.join(files)} into one of {places}")


def _edges_of(adj) -> torch.Tensor:
    """Sorted, duplicate-free ``[2, E]`` int64 edge list of a scipy sparse adjacency (row = source)."""
    coo = adj.tocoo()
    n = max(adj.shape)
    key = np.unique(coo.row.astype(np.int64) * n + coo.col.astype(np.int64))
    return torch.from_numpy(np.stack([key // n, key % n]))


def _class_ids(labels) -> torch.Tensor:
    """Class id per node from one-hot (or multi-hot: first set column wins, as ``argmax`` does) rows, or from ids."""
    y = torch.as_tensor(np.asarray(labels))
    return y.argmax(-1).long() if y.dim() == 2 and y.size(1) > 1 else y.reshape(-1).long()


def _from_pickles(name: str, root: str):
    """``aminer``: ``<name>.adj.sp.pkl`` (scipy sparse), ``<name>.features.pkl``, ``<name>.labels.pkl`` (one-hot)."""
    import pickle
    files = [f"{name}.adj.sp.pkl", f"{name}.features.pkl", f"{name}.labels.pkl"]
    d = find_raw(root, name, files)
    adj, feat, lab = (pickle.load(open(os.path.join(d, f), "rb")) for f in files)
    feat = feat.todense() if hasattr(feat, "todense") else feat
    return torch.as_tensor(np.asarray(feat), dtype=torch.float32), _class_ids(lab), _edges_of(adj), None


def _from_npz_triplet(name: str, root: str, files):
    """``reddit`` / ``Amazon2M`` / GraphSAINT ``amazon``: a scipy ``.npz`` adjacency plus feature and label ``.npy`` files."""
    import scipy.sparse as sp
    d = find_raw(root, name, files)
    adj = sp.load_npz(os.path.join(d, files[0]))
    x = torch.as_tensor(np.load(os.path.join(d, files[1])), dtype=torch.float32)
    return x, _class_ids(np.load(os.path.join(d, files[2]))), _edges_of(adj), d


def _graphsaint_split(raw_dir: str, out_dir: str) -> dict:
    """GraphSAINT's ``role.json`` (keys tr / va / te) is the official 80/5/15 split of AmazonProducts; it is also
    copied next to the converted tensors, where the split loader accepts it as well."""
    import json
    import shutil
    src = os.path.join(raw_dir, "role.json")
    if not os.path.exists(src):
        raise SystemExit(f"amazon: role.json (the official GraphSAINT split) is missing from {raw_dir}")
    with open(src, encoding="utf-8") as fh:
        role = json.load(fh)
    os.makedirs(out_dir, exist_ok=True)
    dst = os.path.join(out_dir, "role.json")
    if os.path.abspath(dst) != os.path.abspath(src):
        shutil.copyfile(src, dst)
    return {"train": torch.as_tensor(role["tr"]).long(), "valid": torch.as_tensor(role["va"]).long(),
            "test": torch.as_tensor(role["te"]).long()}


def _from_linkx_mat(name: str, root: str):
    import scipy.io
    fname = {"snap-patents": "snap_patents.mat"}.get(name, f"{name}.mat")
    alts = [fname, f"{name}.mat"]
    path = None
    for f in alts:
        for d in (os.path.join(root, name), os.path.join(root, "raw", name), os.path.join(root, "raw")):
            if os.path.exists(os.path.join(d, f)):
                path = os.path.join(d, f)
    if path is None:
        raise SystemExit(f"place the LINKX file {fname} for {name!r} under {os.path.join(root, 'raw')}")
    m = scipy.io.loadmat(path)
    y = np.asarray(m["label"] if "label" in m else m["years"]).reshape(-1)
    feat = m["node_feat"]
    feat = feat.todense() if hasattr(feat, "todense") else feat
    return torch.as_tensor(np.asarray(feat), dtype=torch.float32), torch.as_tensor(y).long(), m["edge_index"], None


def labelled_random_split(y: torch.Tensor, train_prop: float = 0.5, valid_prop: float = 0.25, seed: int = 0) -> dict:
    """LINKX-style random split: only labelled nodes (label != -1) are distributed."""
    labelled = torch.nonzero(torch.as_tensor(y).reshape(-1) != -1).reshape(-1)
    part = rand_train_test_idx(int(labelled.numel()), train_prop, valid_prop, seed)
    return {k: labelled[v] for k, v in part.items()}


def get_dataset(name: str, root: str = "./dataset/", split_id: int = 0, seed: int = 42) -> str:
    key = name.lower()
    if key.startswith("synthetic:"):
        from ..graph.synthetic import make_bench_graph
        cfg = key.split(":", 1)[1]
        x, y, ei, _ = make_bench_graph(cfg, seed=seed)
        return save_dataset(root, cfg, x, y, ei)
    if key in PYG_SETS:
        x, y, ei, split = _from_pyg(key, root, split_id)
        return save_dataset(root, name, x, y, ei, split)
    if key.startswith("ogbn-"):
        x, y, ei, split = _from_ogb(key, root)
        return save_dataset(root, name, x, y, ei, split)
    if key == "aminer":
        x, y, ei, _ = _from_pickles(key, root)
        return save_dataset(root, name, x, y, ei)
    if key in ("reddit", "amazon2m"):
        raw = name if key == "reddit" else "Amazon2M"
        x, y, ei, _ = _from_npz_triplet(raw, root, [f"{raw}_adj.npz", f"{raw}_feat.npy", f"{raw}_labels.npy"])
        return save_dataset(root, name, x, y, ei)
    if key == "amazon":
        x, y, ei, raw_dir = _from_npz_triplet(key, root, ["adj_full.npz", "feats.npy", "labels.npy"])
        return save_dataset(root, name, x, y, ei, _graphsaint_split(raw_dir, os.path.join(root, name)))
    if key in ("pokec", "snap-patents", "genius"):
        x, y, ei, _ = _from_linkx_mat(key, root)
        splits = None
        if key == "genius":
            if not 0 <= split_id < 5:
                raise SystemExit(f"split_id={split_id} out of range for the 5 genius splits")
            splits = [labelled_random_split(y, 0.5, 0.25, seed=s) for s in range(5)]
        path = save_dataset(root, name, x, y, ei, splits[split_id] if splits else None, splits)
        if key == "snap-patents":
            from .prepare_snap_patents import prepare_labels
            prepare_labels(path)
        return path
    raise SystemExit(f"unknown dataset {name!r}")


# ----------------------------------------------------------------------------------------------- legacy sequence files
def adjacency(edge_index, num_nodes: int):
    import scipy.sparse as sp
    ei = torch.as_tensor(edge_index).cpu().numpy()
    return sp.coo_matrix((np.ones(ei.shape[1], dtype=np.float32), (ei[0], ei[1])), shape=(num_nodes, num_nodes)).tocsr()


def adj_normalize(mx):
    """``(D + I)^-1/2 (A + I) (D + I)^-1/2``."""
    import scipy.sparse as sp
    mx = (mx + sp.eye(mx.shape[0], dtype=np.float32)).tocsr()
    deg = np.asarray(mx.sum(1)).reshape(-1)
    scale = np.where(deg > 0, 1.0 / np.sqrt(np.maximum(deg, 1e-30)), 0.0)
    return (sp.diags(scale) @ mx @ sp.diags(scale)).tocsr()


def column_normalize(mx):
    """``A D^-1`` with D the row sums."""
    import scipy.sparse as sp
    deg = np.asarray(mx.sum(1)).reshape(-1)
    return (mx @ sp.diags(np.where(deg > 0, 1.0 / np.maximum(deg, 1e-30), 0.0))).tocsr()


def eigenvector(lap, k: int = 10) -> torch.Tensor:
    """Eigenvectors 1..k of a (small, dense-able) Laplacian in increasing eigenvalue order."""
    val, vec = np.linalg.eig(np.asarray(lap.todense() if hasattr(lap, "todense") else lap))
    order = np.argsort(val.real)
    return torch.tensor(np.real(vec[:, order])[:, 1:k + 1], dtype=torch.float32)


def power_adjacency_list(normalized_adj, depth: int = 6):
    """``[A', A'^2, ..., A'^depth]``: the channels of the dense attention bias."""
    out = [normalized_adj.tocsr()]
    for _ in range(depth - 1):
        out.append((out[0] @ out[-1]).tocsr())
    return out


def _sequence_record(powers, ids: torch.Tensor, y: torch.Tensor):
    from ..train.legacy_utils import dense_bias_from_adjs
    return [dense_bias_from_adjs(powers, ids), ids, y[ids].long()]


def process_data(root: str, name: str, k1: int, restart: float = 0.15, seed: int = 0, bias_dim: int = 6) -> str:
    """``data_s<k1>.pt``: for every node the sequence [node, neighbours sampled without replacement in proportion to
    its personalised-PageRank row, topped up with the highest-ranked ones], its ``[k1+1, k1+1, bias_dim]`` bias and
    labels.  The PPR matrix is a dense inverse, so this is for small graphs only."""
    path = os.path.join(root, name)
    x, y = torch.load(os.path.join(path, "x.pt")), torch.load(os.path.join(path, "y.pt"))
    n = int(y.shape[0])
    norm = adj_normalize(adjacency(torch.load(os.path.join(path, "edge_index.pt")), n))
    powers = power_adjacency_list(norm, bias_dim)
    ppr = restart * np.linalg.inv(np.eye(n) - (1.0 - restart) * np.asarray(norm.todense(), dtype=np.float64))
    rng = np.random.default_rng(seed)
    records = []
    for v in range(n):
        row = ppr[v].copy()
        row[v] = -np.inf
        top = np.argsort(row)[-k1:]                       # ascending: weakest of the top k1 first, like the reference
        w = np.maximum(np.where(np.isfinite(row), row, 0.0), 0.0)
        m = int(min(k1, (w > 0).sum()))
        drawn = rng.choice(n, size=m, replace=False, p=w / w.sum()) if m > 0 else np.zeros(0, dtype=np.int64)
        ids = torch.from_numpy(np.concatenate([[v], drawn, top[: k1 - m]]).astype(np.int64))
        records.append([_sequence_record(powers, ids, y)])
    out = os.path.join(path, f"data_s{k1}.pt")
    torch.save(records, out)
    return out


def rand_nodes_seq(root: str, name: str, k1: int, seed: int = 0, bias_dim: int = 6) -> str:
    """``data_rand<k1>.pt``: the shuffled node set cut into disjoint sequences of ``k1`` nodes (the last one shorter)."""
    path = os.path.join(root, name)
    y = torch.load(os.path.join(path, "y.pt"))
    n = int(y.shape[0])
    powers = power_adjacency_list(adj_normalize(adjacency(torch.load(os.path.join(path, "edge_index.pt")), n)), bias_dim)
    order = torch.randperm(n, generator=torch.Generator().manual_seed(seed))
    records = [[_sequence_record(powers, ids, y)] for ids in torch.split(order, int(k1))]
    out = os.path.join(path, f"data_rand{k1}.pt")
    if not os.path.exists(out):
        torch.save(records, out)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--dataset_dir", default="./dataset/")
    ap.add_argument("--split_id", type=int, default=0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--sequences", choices=["none", "ppr", "rand"], default="none")
    ap.add_argument("--k1", type=int, default=100)
    a = ap.parse_args(argv)
    path = get_dataset(a.dataset, a.dataset_dir, a.split_id, a.seed)
    print("wrote", path)
    if a.sequences != "none":
        fn = process_data if a.sequences == "ppr" else rand_nodes_seq
        root, name = os.path.split(os.path.normpath(path))          # the folder written above (synthetic:<x> -> <x>)
        print("wrote", fn(root, name, a.k1, seed=a.seed))


if __name__ == "__main__":
    main()
