"""snap-patents label / split preparation (LINKX benchmark format).

``python -m budgetformer_b200.utils.prepare_snap_patents --dataset_dir ./dataset --nclasses 5``

Converts raw grant years in ``y.pt`` into ``nclasses`` even-quantile classes (the LINKX rule: class k holds the
values in ``[q_k, q_{k+1})``, NaNs keep label -1; utils/prepare_snap-patents.py:14-31 in the reference), keeping the
raw years in ``y_raw_year.pt``, and normalises an official splits file into ``split_idx_all.pt``.  Downloading the
splits needs ``gdown`` and network access; without them point ``--splits_file`` at a local copy."""
from __future__ import annotations

import argparse
import os
from typing import Dict, List

import numpy as np
import torch

SPLITS_DRIVE_ID = "12xbBRqd8mtG_XkNLH8dRRNZJvVM4Pw-N"


def even_quantile_labels(vals: np.ndarray, nclasses: int = 5, verbose: bool = False) -> np.ndarray:
    vals = np.asarray(vals, dtype=np.float64)
    label = np.full(vals.shape[0], -1, dtype=np.int64)
    edges = [-np.inf] + [float(np.nanquantile(vals, (k + 1) / nclasses)) for k in range(nclasses - 1)] + [np.inf]
    for k in range(nclasses):
        lo, hi = edges[k], edges[k + 1]
        sel = (vals >= lo) & (vals < hi) if k < nclasses - 1 else (vals >= lo)
        label[sel] = k
        if verbose:
            print(f"  class {k}: [{lo}, {hi})")
    return label


def prepare_labels(path: str, label_file: str = "y.pt", nclasses: int = 5, force: bool = False) -> bool:
    raw_path = os.path.join(path, "y_raw_year.pt")
    y_path = os.path.join(path, label_file)
    src = raw_path if os.path.exists(raw_path) else y_path
    years = torch.load(src, map_location="cpu").reshape(-1).to(torch.long)
    cur = torch.load(y_path, map_location="cpu").reshape(-1).to(torch.long) if os.path.exists(y_path) else years
    already = cur.unique().numel() <= nclasses and int(cur.min()) >= 0 and int(cur.max()) < nclasses
    if already and not force:
        print(f"[labels] {y_path} already holds {nclasses}-class labels; nothing to do")
        return False
    if src != raw_path:
        torch.save(years.clone(), raw_path)
    y = torch.from_numpy(even_quantile_labels(years.numpy(), nclasses, verbose=True))
    torch.save(y, y_path)
    vals, cnts = torch.unique(y, return_counts=True)
    print("[labels] class counts: " + ", ".join(f"{int(v)}: {int(c)}" for v, c in zip(vals, cnts)))
    return True


def normalize_splits(obj) -> List[Dict[str, torch.Tensor]]:
    seq = obj.tolist() if isinstance(obj, np.ndarray) else list(obj) if isinstance(obj, (list, tuple)) else [obj]
    out = []
    for s in seq:
        va = s.get("valid", s.get("val"))
        if s.get("train") is None or va is None or s.get("test") is None:
            raise ValueError("split entry is missing train/valid/test")
        out.append({k: torch.as_tensor(np.asarray(v)).reshape(-1).long() for k, v in
                    (("train", s["train"]), ("valid", va), ("test", s["test"]))})
    return out


def prepare_splits(path: str, splits_file: str = "", force: bool = False) -> bool:
    raw = splits_file or os.path.join(path, "snap-patents-splits.npy")
    if not os.path.exists(raw):
        try:
            import gdown
            gdown.download(id=SPLITS_DRIVE_ID, output=raw, quiet=False)
        except Exception as e:
            print(f"[splits] cannot download the official splits ({type(e).__name__}); pass --splits_file")
            return False
    out = os.path.join(path, "split_idx_all.pt")
    if os.path.exists(out) and not force:
        return False
    torch.save(normalize_splits(np.load(raw, allow_pickle=True)), out)
    print(f"[splits] wrote {out}")
    return True


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset_dir", default="./dataset/")
    ap.add_argument("--dataset", default="snap-patents")
    ap.add_argument("--label_file", default="y.pt")
    ap.add_argument("--nclasses", type=int, default=5)
    ap.add_argument("--splits_file", default="")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--skip_splits", action="store_true")
    a = ap.parse_args(argv)
    path = os.path.join(a.dataset_dir, a.dataset)
    prepare_labels(path, a.label_file, a.nclasses, a.force)
    if not a.skip_splits:
        prepare_splits(path, a.splits_file, a.force)


if __name__ == "__main__":
    main()
