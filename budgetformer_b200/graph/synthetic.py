"""Synthetic graph generators for the benchmark configurations (no dataset download is possible in
the target environment): stochastic block model, Chung-Lu power law (directed / undirected) and a
citation-like DAG with power-law out-degree.  ``write_dataset`` stores a graph in the on-disk data
contract so that the command-line driver (and the reference) can train on it."""
from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np
import torch


def sbm_graph(num_nodes: int = 2048, blocks: int = 7, p_in: float = 0.02, p_out: float = 0.001, feat_dim: int = 128,
              seed: int = 42) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Symmetrised SBM with equal blocks; labels = block id; N(0,1) features plus a weak class signal."""
    rng = np.random.default_rng(seed)
    n = int(num_nodes)
    label = (np.arange(n) * blocks // n).astype(np.int64)
    iu, ju = np.triu_indices(n, k=1)
    p = np.where(label[iu] == label[ju], p_in, p_out)
    keep = rng.random(iu.size) < p
    s, d = iu[keep], ju[keep]
    ei = np.stack([np.concatenate([s, d]), np.concatenate([d, s])])
    x = rng.standard_normal((n, feat_dim)).astype(np.float32)
    centers = rng.standard_normal((blocks, feat_dim)).astype(np.float32)
    x += 0.5 * centers[label]
    return torch.from_numpy(x), torch.from_numpy(label), torch.from_numpy(ei.astype(np.int64))


def _power_law_weights(n: int, exponent: float, rng, w_min: float = 1.0) -> np.ndarray:
    u = rng.random(n)
    return w_min * (1.0 - u) ** (-1.0 / (exponent - 1.0))


def _unique_to_target(sample, target: int, rng) -> np.ndarray:
    """Distinct int64 keys drawn with ``sample(m)`` until exactly ``target`` of them exist (heavy-tailed samplers
    repeat hub pairs often, so one draw of ``target`` pairs falls well short after deduplication)."""
    keys = np.unique(sample(int(target)))
    for _ in range(64):
        need = int(target) - keys.size
        if need <= 0:
            break
        fresh = np.setdiff1d(np.unique(sample(int(need * 1.5) + 1024)), keys, assume_unique=True)
        if fresh.size > need:
            fresh = fresh[np.sort(rng.permutation(fresh.size)[:need])]
        keys = np.union1d(keys, fresh)
    return keys


def chung_lu_edges(num_nodes: int, num_edges: int, exponent: float = 2.1, directed: bool = True, seed: int = 0,
                   chunk: int = 1 << 24) -> torch.Tensor:
    """``num_edges`` distinct (src, dst) pairs (no self loops) with endpoint probabilities proportional to power-law
    weights: the Chung-Lu model in its fast form, topped up until the requested count is reached.  Undirected graphs
    take ``num_edges`` node pairs and return both directions (``2 * num_edges`` columns)."""
    rng = np.random.default_rng(seed)
    n = int(num_nodes)
    w_out = _power_law_weights(n, exponent, rng)
    w_in = _power_law_weights(n, exponent, rng) if directed else w_out
    cdf_out = np.cumsum(w_out / w_out.sum())
    cdf_in = np.cumsum(w_in / w_in.sum())

    def sample(m: int) -> np.ndarray:
        parts = []
        while m > 0:
            c = min(m, chunk)
            s = np.searchsorted(cdf_out, rng.random(c)).clip(0, n - 1).astype(np.int64)
            d = np.searchsorted(cdf_in, rng.random(c)).clip(0, n - 1).astype(np.int64)
            ok = s != d
            s, d = s[ok], d[ok]
            if not directed:
                s, d = np.minimum(s, d), np.maximum(s, d)
            parts.append(s * n + d)
            m -= c
        return np.concatenate(parts)

    key = _unique_to_target(sample, num_edges, rng)
    s, d = key // n, key % n
    if not directed:
        key = np.sort(np.concatenate([s * n + d, d * n + s]))
        s, d = key // n, key % n
    return torch.from_numpy(np.stack([s, d]).astype(np.int64))


def chung_lu_edges_device(num_nodes: int, num_edges: int, exponent: float = 2.1, directed: bool = True, seed: int = 0,
                          device="cuda", chunk: int = 1 << 26) -> torch.Tensor:
    """The same model as ``chung_lu_edges`` generated with torch on ``device`` (searchsorted / unique on a GPU take
    seconds where the NumPy form takes minutes at 10^8 edges).  Deterministic for a given seed and device type; it is
    a different random stream than the NumPy form, so the two give different graphs of the same distribution."""
    dev = torch.device(device)
    n = int(num_nodes)
    g = torch.Generator(device=dev).manual_seed(int(seed))

    def weights():
        u = torch.rand(n, generator=g, device=dev, dtype=torch.float64)
        w = (1.0 - u) ** (-1.0 / (exponent - 1.0))
        return torch.cumsum(w / w.sum(), 0)

    cdf_out = weights()
    cdf_in = weights() if directed else cdf_out

    def sample(m: int) -> torch.Tensor:
        parts = []
        while m > 0:
            c = min(m, chunk)
            s = torch.searchsorted(cdf_out, torch.rand(c, generator=g, device=dev, dtype=torch.float64)).clamp_(0, n - 1)
            d = torch.searchsorted(cdf_in, torch.rand(c, generator=g, device=dev, dtype=torch.float64)).clamp_(0, n - 1)
            ok = s != d
            s, d = s[ok], d[ok]
            if not directed:
                s, d = torch.minimum(s, d), torch.maximum(s, d)
            parts.append(s * n + d)
            m -= c
        return torch.cat(parts)

    keys = torch.unique(sample(int(num_edges)))
    for _ in range(64):
        need = int(num_edges) - keys.numel()
        if need <= 0:
            break
        fresh = torch.unique(sample(int(need * 1.5) + 1024))
        fresh = fresh[~torch.isin(fresh, keys, assume_unique=True)]
        if fresh.numel() > need:
            pick = torch.randperm(fresh.numel(), generator=g, device=dev)[:need]
            fresh = fresh[torch.sort(pick).values]
        keys = torch.unique(torch.cat([keys, fresh]))
    s, d = torch.div(keys, n, rounding_mode="floor"), keys % n
    if not directed:
        both = torch.sort(torch.cat([s * n + d, d * n + s])).values
        s, d = torch.div(both, n, rounding_mode="floor"), both % n
    return torch.stack([s, d]).cpu()


def citation_dag_edges(num_nodes: int, num_edges: int, exponent: float = 2.2, seed: int = 0) -> torch.Tensor:
    """Heterophilous citation-like DAG with exactly ``num_edges`` distinct edges: node i cites uniformly chosen
    earlier nodes j < i; the number of citations per node follows a power law."""
    rng = np.random.default_rng(seed)
    n = int(num_nodes)
    w = _power_law_weights(n, exponent, rng)
    w[0] = 0.0                                            # node 0 has no predecessor
    p = w / w.sum()
    cdf = np.cumsum(p)
    out_deg = np.floor(p * num_edges).astype(np.int64)
    out_deg = np.minimum(out_deg, np.arange(n))           # node i has only i predecessors
    src0 = np.repeat(np.arange(n, dtype=np.int64), out_deg)
    first = [src0 * n + (rng.random(src0.size) * src0).astype(np.int64)]

    def sample(m: int) -> np.ndarray:
        if first:
            return first.pop()
        src = np.searchsorted(cdf, rng.random(m)).clip(1, n - 1).astype(np.int64)
        return src * n + (rng.random(m) * src).astype(np.int64)

    key = _unique_to_target(sample, num_edges, rng)
    return torch.from_numpy(np.stack([key // n, key % n]).astype(np.int64))


def random_features(num_nodes: int, dim: int, seed: int = 0, dtype=torch.float32) -> torch.Tensor:
    g = torch.Generator().manual_seed(int(seed))
    return torch.randn(int(num_nodes), int(dim), generator=g, dtype=dtype)


def random_labels(num_nodes: int, num_classes: int, seed: int = 0, multilabel_p: Optional[float] = None) -> torch.Tensor:
    g = torch.Generator().manual_seed(int(seed) + 1)
    if multilabel_p is not None:
        return (torch.rand(int(num_nodes), int(num_classes), generator=g) < multilabel_p).to(torch.float32)
    return torch.randint(0, int(num_classes), (int(num_nodes),), generator=g)


BENCH_CONFIGS = {
    # name: model/graph shape of the five benchmark configurations
    "sbm2k": dict(model="gt", n_layers=2, hidden_dim=64, num_heads=4, nodes=2048, feat=128, classes=7,
                  budget=8, walk_length=4, walks_per_node=2, graph="sbm"),
    "arxiv_like": dict(model="graphormer", n_layers=4, hidden_dim=128, num_heads=8, nodes=169_343, edges=1_166_243,
                       feat=128, classes=40, budget=8, walk_length=4, walks_per_node=2, graph="chung_lu_directed"),
    "products_like": dict(model="graphgps", n_layers=4, hidden_dim=256, num_heads=8, nodes=2_449_029,
                          edges=61_859_140, feat=100, classes=47, budget=16, walk_length=6, walks_per_node=4,
                          graph="chung_lu_undirected"),
    "amazon_like": dict(model="exphormer", n_layers=3, hidden_dim=256, num_heads=8, nodes=1_569_960,
                        edges=264_339_468, feat=200, classes=107, budget=32, walk_length=4, walks_per_node=2,
                        graph="chung_lu_directed", multilabel=True),
    "patents_like": dict(model="gt", n_layers=4, hidden_dim=128, num_heads=8, nodes=2_923_922, edges=13_975_788,
                         feat=269, classes=5, budget=8, walk_length=4, walks_per_node=2, graph="dag"),
}


def make_bench_graph(name: str, seed: int = 42, scale: float = 1.0):
    """(x, y, edge_index, cfg) for a named configuration; ``scale`` < 1 shrinks nodes and edges for tests."""
    cfg = dict(BENCH_CONFIGS[name])
    n = max(64, int(cfg["nodes"] * scale))
    if cfg["graph"] == "sbm":
        x, y, ei = sbm_graph(n, feat_dim=cfg["feat"], seed=seed)
        return x, y, ei, cfg
    e = max(n, int(cfg["edges"] * scale))
    ei = _cached_edges(f"{name}_{cfg['graph']}_{n}_{e}_{int(seed)}", lambda: _make_edges(cfg["graph"], n, e, seed))
    x = random_features(n, cfg["feat"], seed)
    y = random_labels(n, cfg["classes"], seed, 0.05 if cfg.get("multilabel") else None)
    return x, y, ei, cfg


# Chung-Lu graphs at least this large are generated on the GPU when one is available (minutes -> seconds)
DEVICE_GENERATION_MIN_EDGES = 20_000_000


def _make_edges(kind: str, n: int, e: int, seed: int) -> torch.Tensor:
    if kind in ("chung_lu_directed", "chung_lu_undirected"):
        directed = kind == "chung_lu_directed"
        if e >= DEVICE_GENERATION_MIN_EDGES and torch.cuda.is_available():
            return chung_lu_edges_device(n, e, 2.1, directed, seed, torch.device("cuda", torch.cuda.current_device()))
        return chung_lu_edges(n, e, 2.1, directed, seed)
    return citation_dag_edges(n, e, 2.2, seed)


def _cached_edges(tag: str, make) -> torch.Tensor:
    """Edge lists of the large configurations take minutes of sorting to generate; consecutive benchmark runs on one
    machine (1/2/4/8 ranks, both arms) share them through ``$BF_BENCH_CACHE`` (default: ``.bench_cache`` beside the
    package; an empty value disables it).  Generation is deterministic, so concurrent writers produce identical files;
    the rename is atomic."""
    pkg_parent = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    root = os.environ.get("BF_BENCH_CACHE", os.path.join(pkg_parent, ".bench_cache"))
    path = os.path.join(root, tag + ".pt")
    if root and os.path.exists(path):
        try:
            return torch.load(path)
        except Exception:
            pass
    ei = make()
    if root and ei.numel() >= (1 << 20):
        try:
            os.makedirs(root, exist_ok=True)
            tmp = f"{path}.{os.getpid()}.tmp"
            torch.save(ei, tmp)
            os.replace(tmp, path)
        except OSError:
            pass
    return ei


def write_dataset(root: str, name: str, x: torch.Tensor, y: torch.Tensor, edge_index: torch.Tensor) -> str:
    path = os.path.join(root, name)
    os.makedirs(path, exist_ok=True)
    torch.save(x, os.path.join(path, "x.pt"))
    torch.save(y, os.path.join(path, "y.pt"))
    torch.save(edge_index, os.path.join(path, "edge_index.pt"))
    return path
