"""Dataset preparation CLI: writes the on-disk contract ``<dataset_dir>/<name>/{x.pt, y.pt, edge_index.pt[, split_idx.pt]}``.

``python -m budgetformer_b200.utils.preprocess_data --dataset <name> [--dataset_dir ./dataset/] [--split_id 0]``

Sources (utils/preprocess_data.py:161-427 in the reference): Planetoid, CitationFull, Coauthor, Amazon Photo /
Computers, Reddit, HeterophilousGraphDataset (PyG); ogbn-arxiv / products / papers100M (OGB); pokec, snap-patents,
genius (LINKX ``.mat`` / ``.npz`` files placed under ``<dataset_dir>/raw``; genius gets five seeded 50/25/25
splits); and ``synthetic:<config>`` which generates the benchmark graphs of this repository without any download.
PyG / OGB are optional: when they are not importable the corresponding names fail with a clear message."""
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
    "photo": ("Amazon", "Photo"), "computers": ("Amazon", "Computers"), "reddit": ("Reddit", None),
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


def _from_linkx_mat(name: str, root: str):
    import scipy.io
    path = os.path.join(root, "raw", f"{name}.mat")
    if not os.path.exists(path):
        raise SystemExit(f"place the LINKX file for {name!r} at {path}")
    m = scipy.io.loadmat(path)
    y = np.asarray(m["label"] if "label" in m else m["years"]).reshape(-1)
    return m["node_feat"], torch.as_tensor(y).long(), m["edge_index"], None


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
    if key in ("pokec", "snap-patents", "genius"):
        x, y, ei, _ = _from_linkx_mat(key, root)
        splits = [rand_train_test_idx(len(y), 0.5, 0.25, seed=s) for s in range(5)] if key == "genius" else None
        path = save_dataset(root, name, x, y, ei, splits[split_id] if splits else None, splits)
        if key == "snap-patents":
            from .prepare_snap_patents import prepare_labels
            prepare_labels(path)
        return path
    raise SystemExit(f"unknown dataset {name!r}")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--dataset_dir", default="./dataset/")
    ap.add_argument("--split_id", type=int, default=0)
    ap.add_argument("--seed", type=int, default=42)
    a = ap.parse_args(argv)
    print("wrote", get_dataset(a.dataset, a.dataset_dir, a.split_id, a.seed))


if __name__ == "__main__":
    main()
