"""Does the fused layer path train like the portable one?

    python -m budgetformer_b200.utils.convergence --graph sbm --epochs 300
    python -m budgetformer_b200.utils.convergence --graph patents --scale 0.05 --epochs 300

Trains the same model twice on one GPU from the same seed - once on the fused B200 path (bf16 activations and residual
stream, fp32 statistics and accumulation) and once on the portable path (``torch.autocast`` like the reference: bf16
matmuls, fp32 residual stream) - and prints one JSON line with both loss curves (sampled), the best validation accuracy
and the test accuracy at that epoch.  The two runs see the same graphs (the builders are counter-based) but different
dropout masks, so the comparison is between two seeds' worth of noise, not bit for bit."""
from __future__ import annotations

import argparse
import json

import torch


def _data(kind: str, scale: float, seed: int):
    from ..graph.synthetic import make_bench_graph, sbm_graph
    from ..train.data import GraphData, random_split_idx
    if kind == "sbm":
        # the 2,048-node stochastic block model of the plumbing configuration: 7 blocks, labels = block id
        x, y, ei = sbm_graph(2048, feat_dim=128, seed=seed)
        return GraphData(x, y, ei, random_split_idx(2048, seed), 2048, 7), dict(hidden_dim=64, num_heads=4, n_layers=2)
    x, y, ei, cfg = make_bench_graph("patents_like", seed=seed, scale=scale)
    n = x.size(0)
    # the benchmark's labels are independent of everything (nothing to learn): plant a learnable signal so that accuracy
    # separates a path that trains from one that does not - the class is a linear function of the features
    w = torch.randn(x.size(1), int(cfg["classes"]), generator=torch.Generator().manual_seed(seed + 11))
    y = (x @ w).argmax(1)
    return (GraphData(x, y, ei, random_split_idx(n, seed), n, int(cfg["classes"])),
            dict(hidden_dim=cfg["hidden_dim"], num_heads=cfg["num_heads"], n_layers=cfg["n_layers"]))


def _run(kind: str, scale: float, seed: int, epochs: int, fused: bool, lr: float, device: str = "cuda:0"):
    from ..config import parse_fullgraph_args
    from ..train.engine import FullGraphTrainer
    data, shape = _data(kind, scale, seed)
    argv = ["--model", "gt", "--dataset", f"conv_{kind}", "--n_layers", str(shape["n_layers"]), "--hidden_dim", str(shape["hidden_dim"]),
            "--num_heads", str(shape["num_heads"]), "--ffn_dim", str(2 * shape["hidden_dim"]), "--amp_dtype", "bf16",
            "--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4", "--force_random_split",
            "--epochs", str(epochs), "--peak_lr", str(lr), "--warmup_updates", "10", "--seed", str(seed),
            "--fused_sp", "on" if fused else "off", "--device", device]
    torch.manual_seed(seed)
    t = FullGraphTrainer(parse_fullgraph_args(argv), data=data, log=lambda *a, **k: None)
    assert bool(t.fused_sp) == fused or not device.startswith("cuda")      # a CPU run has only the portable path
    keep = sorted({1, 2, 5, 10, 20, 50, 100, 150, 200, 250, epochs} & set(range(1, epochs + 1)))
    curve, best = {}, {"valid": -1.0, "test": -1.0, "epoch": 0}
    for epoch in range(1, epochs + 1):
        out = t.train_step(epoch)
        if epoch in keep:
            curve[epoch] = round(out["loss"], 5)
        if epoch % 25 == 0 or epoch == epochs:
            res = t.evaluate(epoch)
            if res["valid"] > best["valid"]:
                best = {"valid": round(res["valid"], 4), "test": round(res["test"], 4), "epoch": epoch}
    t.edge_engine.shutdown()
    return {"loss": curve, "best": best}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--graph", choices=["sbm", "patents"], default="sbm")
    ap.add_argument("--scale", type=float, default=0.05)
    ap.add_argument("--epochs", type=int, default=300)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--lr", type=float, default=2e-3)
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)
    rec = {"graph": a.graph, "scale": a.scale if a.graph == "patents" else 1.0, "epochs": a.epochs, "seed": a.seed,
           "fused": _run(a.graph, a.scale, a.seed, a.epochs, True, a.lr, a.device),
           "portable": _run(a.graph, a.scale, a.seed, a.epochs, False, a.lr, a.device)}
    rec["best_valid_gap"] = round(rec["fused"]["best"]["valid"] - rec["portable"]["best"]["valid"], 4)
    print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
