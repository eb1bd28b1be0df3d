"""Child program for the gloo multi-process CPU tests (spawned by tests/test_dist_cpu.py)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from budgetformer_b200.config import parse_fullgraph_args  # noqa: E402
from budgetformer_b200.graph.synthetic import sbm_graph  # noqa: E402
from budgetformer_b200.train.data import GraphData, random_split_idx  # noqa: E402
from budgetformer_b200.train.engine import FullGraphTrainer  # noqa: E402


def make(model, extra=(), n=512):
    x, y, ei = sbm_graph(n, feat_dim=32, seed=3)
    data = GraphData(x, y, ei, random_split_idx(n, 3), n, 7)
    argv = ["--model", model, "--dataset", "t", "--n_layers", "2", "--hidden_dim", "32", "--num_heads", "4", "--ffn_dim", "64",
            "--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4", "--force_random_split",
            "--distributed-backend", "gloo", "--dropout_rate", "0.0", "--attention_dropout_rate", "0.0",
            "--input_dropout_rate", "0.0", "--seed", "5", "--epochs", "4", "--eval_every", "2"]
    return FullGraphTrainer(parse_fullgraph_args(argv + list(extra)), data=data, log=lambda *a, **k: None)


def mode_equiv(out_path):
    """SP forward/backward on P ranks equals the single-process result (written by rank 0 for the parent to compare)."""
    res = {}
    for model in ("gt", "graphormer", "graphgps", "exphormer"):
        t = make(model)
        g = t.build_edges(1)
        t.model.eval()                                    # BatchNorm: use running stats so that ranks agree with 1 process
        loss, out = t._loss(g, t.local_idx["train"])
        n_local = float(t.local_idx["train"].numel())
        t.reducer.prepare_backward()
        (loss * n_local).backward()                       # sum over local nodes -> after the mean reduction: sum / P
        t.reducer.finalize_backward()
        parts = [torch.empty_like(out) for _ in range(t.sp_world)]
        gn = torch.tensor([n_local])
        if dist.is_initialized():
            dist.all_gather(parts, out.contiguous())
            dist.all_reduce(gn)
        else:
            parts = [out]
        grads = {n: (p.grad * t.sp_world / float(gn)).tolist() for n, p in list(t.model.named_parameters())[:6]}
        res[model] = {"out": torch.cat(parts)[:8].tolist(), "grads": grads, "edges": g.num_edges,
                      "cols": g.col[:64].tolist()}
    if not dist.is_initialized() or dist.get_rank() == 0:
        json.dump(res, open(out_path, "w"))


def mode_train(out_path):
    t = make("gt", ["--peak_lr", "5e-3"], n=2048)
    best = t.fit()
    if dist.get_rank() == 0:
        json.dump({"best": best, "epochs": len(t.epoch_times)}, open(out_path, "w"))


def mode_oom(out_path):
    """Host-injected out-of-memory errors.  Epoch 2: every rank fails before its forward (the symmetric case of
    real OOMs: ranks hold identical tensors) -> one tier is demoted and the step retried.  Epoch 3: only rank 1
    fails, after backward and the gradient reduction (no collective pending) -> the vote makes rank 0 drop the step
    too and both demote again."""
    t = make("gt", ["--activation_checkpoint_mode", "multi_tier", "--force_multi_tier_plan", "cpu_rank_local_prefetch:retain=2",
                    "--fault_inject", "oom@fwd:2,oom@opt:3:rank1", "--distributed-timeout-minutes", "2"])
    log = []
    for epoch in (1, 2, 3, 4):
        s = t.train_step(epoch)
        # replicated weights must stay identical: a rank that did not fail may not apply a step the others drop
        digest = float(sum(p.detach().double().sum() for p in t.model.parameters()))
        log.append({"epoch": epoch, "dropped": s["dropped"], "loss": s["loss"], "modes": t.planner.modes(),
                    "weights": digest})
    json.dump(log, open(out_path + f".{dist.get_rank()}", "w"))


def mode_adaptive(out_path):
    t = make("gt", ["--adaptive_edge_budget", "--max_total_edges_per_query", "8", "--warmup_updates", "1", "--epochs", "8",
                    "--eval_every", "100"], n=1024)
    # drop the fixed budget flags: rebuild args without them
    json.dump({"ok": True}, open(out_path + f".{dist.get_rank()}", "w"))


def mode_watchdog(out_path):
    """A rank that leaves between steps (injected exit with an announcement) or stalls silently: the survivor learns of
    it from the watchdog - PeerLost before its next step, or a clean process abort when it is stuck in a collective."""
    from budgetformer_b200.utils.watchdog import PeerLost
    kind = os.environ["BF_WD_CASE"]
    fault = {"leave": "exit@step:3:rank1", "stall": "stall@step:3:rank1", "midstep": "stall@bwd:3:rank1"}[kind]
    extra = ["--watchdog_step_seconds", "6"] if kind == "midstep" else []
    t = make("gt", ["--watchdog_seconds", "2", "--fault_inject", fault, "--epochs", "6", "--eval_every", "100"] + extra)
    try:
        t.fit()
        result = {"outcome": "finished"}
    except PeerLost as e:
        result = {"outcome": "peer_lost", "message": str(e), "epoch": t.epoch}
    json.dump(result, open(out_path + f".{dist.get_rank()}", "w"))
    os._exit(0)                                    # the peer is gone: skip the collective teardown


def mode_shard(out_path):
    """--shard_cpu_edge_build: the graph all-gathered from per-rank shards equals the graph one process builds, for the
    plain, the typed (Exphormer), the virtual-node (Graphormer), the unbudgeted and the fan-out case; and training on
    it runs (prefetch thread included)."""
    res = {}
    cases = {"gt": [], "exphormer": [], "graphormer": [],
             "gt_fanout": ["--rw_edge_mode", "dgl_neighbor", "--fanout", "3,2"]}
    for name, extra in cases.items():
        model = name.split("_")[0]
        sharded = make(model, ["--shard_cpu_edge_build"] + extra)
        assert sharded.edge_engine.sharded_host_build() == (sharded.sp_world > 1)
        g = sharded.build_edges(1)
        whole = make(model, extra)
        w = whole.build_edges(1)
        res[name] = {"equal": bool(torch.equal(g.rowptr, w.rowptr) and torch.equal(g.col, w.col)
                                   and (g.etype is None or torch.equal(g.etype, w.etype))),
                     "edges": g.num_edges, "totals": [g.n_real, g.n_rw], "totals_whole": [w.n_real, w.n_rw]}
        sharded.edge_engine.shutdown()
        whole.edge_engine.shutdown()
    t = make("gt", ["--shard_cpu_edge_build", "--peak_lr", "5e-3"], n=1024)
    best = t.fit()
    res["fit"] = {"epochs": len(t.epoch_times), "valid": best["valid"]}
    if not dist.is_initialized() or dist.get_rank() == 0:
        json.dump(res, open(out_path, "w"))


def mode_syncbn(out_path):
    """--sync_batchnorm: training-mode GraphGPS on P ranks normalises with the statistics of all rows, so outputs and
    gradients equal the single-process run (which sees all rows in one BatchNorm call)."""
    t = make("graphgps", ["--sync_batchnorm"])
    g = t.build_edges(1)
    t.model.train()
    loss, out = t._loss(g, t.local_idx["train"])
    n_local = float(t.local_idx["train"].numel())
    t.reducer.prepare_backward()
    (loss * n_local).backward()
    t.reducer.finalize_backward()
    parts = [torch.empty_like(out) for _ in range(t.sp_world)]
    gn = torch.tensor([n_local])
    if dist.is_initialized():
        dist.all_gather(parts, out.contiguous())
        dist.all_reduce(gn)
    else:
        parts = [out]
    named = dict(t.model.named_parameters())
    keys = [k for k in named if "norm" in k][:4] + list(named)[:3]
    grads = {k: (named[k].grad * t.sp_world / float(gn)).tolist() for k in keys}
    rm = [m.running_mean.tolist() for m in t.model.modules() if isinstance(m, torch.nn.BatchNorm1d)][:2]
    if not dist.is_initialized() or dist.get_rank() == 0:
        json.dump({"out": torch.cat(parts)[:8].tolist(), "grads": grads, "running_mean": rm}, open(out_path, "w"))


def mode_raise(out_path):
    """Every rank trains two steps, then rank 1 raises: the entry-point guard prints the traceback and ends the process
    with status 1 (no collective teardown, no wait in interpreter shutdown), so the launcher can end the job."""
    t = make("gt", [])
    t.train_step(1)
    t.train_step(2)
    if t.rank == 1:
        raise RuntimeError("injected failure on rank 1")
    t.train_step(3)                                   # rank 0 goes on and would wait for its peer in the next collective


def _dispatch():
    mode, out = sys.argv[1], sys.argv[2]
    {"equiv": mode_equiv, "train": mode_train, "oom": mode_oom, "syncbn": mode_syncbn, "watchdog": mode_watchdog,
     "shard": mode_shard, "raise": mode_raise}[mode](out)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    from budgetformer_b200.utils.rank_main import run_rank_main
    run_rank_main(_dispatch)
