"""Train/valid/test split discovery.

Looks for the same on-disk layouts as the reference (utils/split_utils.py:78-145): multi-split
containers, a single split dict, index triples, mask triples and GraphSAINT ``role.json``; then OGB
and PyG default splits when those packages are importable (:148-210).  Multi-rank callers use the
rank-0-first barrier protocol (:186-196) so that only one process touches a cold dataset folder."""
from __future__ import annotations

import json
import os
import pickle
from typing import Optional

import numpy as np
import torch

_MULTI = ("split_idx_all.pt", "official_splits.npy", "fixed_splits.npy", "snap-patents-splits.npy")
_SINGLE = ("split_idx.pt", "split.pt")
_INDEX_TRIPLES = (
    ("train_idx.pt", "valid_idx.pt", "test_idx.pt"), ("train_idx.pt", "val_idx.pt", "test_idx.pt"),
    ("split/train.pt", "split/valid.pt", "split/test.pt"), ("split/train_idx.pt", "split/valid_idx.pt", "split/test_idx.pt"),
)
_MASK_TRIPLES = (
    ("train_mask.pt", "valid_mask.pt", "test_mask.pt"), ("train_mask.pt", "val_mask.pt", "test_mask.pt"),
    ("split/train_mask.pt", "split/valid_mask.pt", "split/test_mask.pt"),
)


def safe_torch_load(path: str, mmap: bool = False):
    """CPU load that prefers the safe unpickler.  ``mmap=True`` first tries a memory-mapped load (the ranks of a node
    then share one page-cache copy of a large feature matrix instead of holding one each; files in the old
    non-zip format cannot be mapped and fall through), like the attempt ladder of the reference's loader
    (utils/fullgraph_sp_support.py:692-715)."""
    attempts = ([{"weights_only": True, "mmap": True}, {"weights_only": False, "mmap": True}] if mmap else []) + \
        [{"weights_only": True}, {"weights_only": False}]
    last = None
    for kw in attempts:
        try:
            return torch.load(path, map_location="cpu", **kw)
        except (TypeError, pickle.UnpicklingError, RuntimeError, ValueError) as exc:
            last = exc
    raise last


def _as_idx(value) -> torch.Tensor:
    t = value.detach().cpu() if isinstance(value, torch.Tensor) else torch.as_tensor(np.asarray(value))
    t = t.reshape(-1)
    if t.dtype == torch.bool:
        t = torch.nonzero(t, as_tuple=False).reshape(-1)
    return t.to(torch.long)


def _mask_to_idx(mask: torch.Tensor, split_id: int = 0) -> torch.Tensor:
    mask = mask.detach().cpu()
    if mask.dim() == 2:
        if not (0 <= split_id < mask.size(1)):
            raise ValueError(f"split_id={split_id} out of range for mask with {mask.size(1)} splits")
        mask = mask[:, split_id]
    return torch.nonzero(mask.to(torch.bool), as_tuple=False).reshape(-1).to(torch.long)


def _from_dict(obj) -> Optional[dict]:
    if not isinstance(obj, dict):
        return None
    tr, va, te = obj.get("train", obj.get("tr")), obj.get("valid", obj.get("val", obj.get("va"))), obj.get("test", obj.get("te"))
    if tr is None or va is None or te is None:
        return None
    return {"train": _as_idx(tr), "valid": _as_idx(va), "test": _as_idx(te)}


def _normalize(obj, split_id: int = 0) -> Optional[dict]:
    d = _from_dict(obj)
    if d is not None:
        return d
    if isinstance(obj, np.ndarray):
        seq = obj.tolist() if obj.dtype == object else list(obj)
    elif isinstance(obj, (list, tuple)):
        seq = list(obj)
    else:
        return None
    if not seq:
        return None
    if not (0 <= split_id < len(seq)):
        raise ValueError(f"split_id={split_id} out of range for {len(seq)} stored splits")
    return _from_dict(seq[split_id])


def load_split_from_dir(path: str, split_id: int = 0) -> Optional[dict]:
    for name in _MULTI + _SINGLE:
        f = os.path.join(path, name)
        if os.path.exists(f):
            obj = np.load(f, allow_pickle=True) if name.endswith(".npy") else safe_torch_load(f)
            d = _normalize(obj, split_id)
            if d is not None:
                return d
    for names, conv in ((_INDEX_TRIPLES, lambda t: _as_idx(t)), (_MASK_TRIPLES, lambda t: _mask_to_idx(t, split_id))):
        for triple in names:
            files = [os.path.join(path, n) for n in triple]
            if all(os.path.exists(f) for f in files):
                tr, va, te = (conv(safe_torch_load(f)) for f in files)
                return {"train": tr, "valid": va, "test": te}
    role = os.path.join(path, "role.json")
    if os.path.exists(role):
        with open(role, "r", encoding="utf-8") as fh:
            return _from_dict(json.load(fh))
    return None


def _library_split(name: str, root: str, split_id: int) -> Optional[dict]:
    key = name.lower()
    try:
        if key.startswith("ogbn-"):
            from ogb.nodeproppred import PygNodePropPredDataset
            return _from_dict(PygNodePropPredDataset(name=name, root=root).get_idx_split())
        data = None
        if key in {"cora", "citeseer", "pubmed"}:
            from torch_geometric.datasets import Planetoid
            data = Planetoid(root=root, name=key)[0]
        elif key in {"roman-empire", "amazon-ratings", "minesweeper", "tolokers", "questions"}:
            from torch_geometric.datasets import HeterophilousGraphDataset
            data = HeterophilousGraphDataset(root=root, name=name.capitalize())[0]
        elif key in {"photo", "computers", "amazon-photo", "amazon-computers"}:
            from torch_geometric.datasets import Amazon
            data = Amazon(root=root, name="Photo" if "photo" in key else "Computers")[0]
        if data is not None and all(hasattr(data, a) for a in ("train_mask", "val_mask", "test_mask")):
            return {"train": _mask_to_idx(data.train_mask, split_id), "valid": _mask_to_idx(data.val_mask, split_id),
                    "test": _mask_to_idx(data.test_mask, split_id)}
    except Exception:
        return None
    return None


def load_default_split(dataset_name: str, root_dir: str, dist_module=None, wait_for_rank0: bool = False,
                       split_id: int = 0) -> Optional[dict]:
    path = os.path.join(root_dir, dataset_name)
    wait = wait_for_rank0 and dist_module is not None and dist_module.is_initialized()
    rank0 = (not wait) or dist_module.get_rank() == 0
    if wait and not rank0:
        dist_module.barrier()
    try:
        out = load_split_from_dir(path, split_id)
        if out is None:
            out = _library_split(str(dataset_name), root_dir, split_id)
    finally:
        if wait and rank0:
            dist_module.barrier()
    return out
