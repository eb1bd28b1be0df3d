"""End-to-end trainer features on CPU (single process, tiny graphs)."""
import os

import pytest
import torch

from budgetformer_b200.config import parse_fullgraph_args
from budgetformer_b200.graph.synthetic import sbm_graph
from budgetformer_b200.train.checkpoint import model_path, train_state_path
from budgetformer_b200.train.data import GraphData, random_split_idx
from budgetformer_b200.train.engine import FullGraphTrainer
from budgetformer_b200.utils import comm_profiler

BASE = ["--dataset", "t", "--n_layers", "2", "--hidden_dim", "32", "--num_heads", "4", "--ffn_dim", "64", "--force_random_split",
        "--device", "cpu", "--peak_lr", "5e-3", "--seed", "5", "--eval_every", "2"]
FIXED = ["--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4"]


def _data(n=384, multilabel=False):
    x, y, ei = sbm_graph(n, feat_dim=16, seed=3)
    if multilabel:
        y = torch.nn.functional.one_hot(y, 7).float()
    return GraphData(x, y, ei, random_split_idx(n, 3), n, 7, multilabel)


def _trainer(argv, data=None, logs=None):
    log = (lambda *a, **k: logs.append(" ".join(str(x) for x in a))) if logs is not None else (lambda *a, **k: None)
    return FullGraphTrainer(parse_fullgraph_args(BASE + list(argv)), data=data or _data(), log=log)


@pytest.mark.parametrize("model", ["gt", "graphormer", "graphgps", "exphormer"])
def test_every_model_trains(model):
    t = _trainer(["--model", model, "--epochs", "6"] + FIXED)
    losses = [t.train_step(e)["loss"] for e in range(1, 7)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    res = t.evaluate(6)
    assert set(res) == {"train", "valid", "test"}


def test_nagphormer_and_hop_features():
    t = _trainer(["--model", "nagphormer", "--hops", "2", "--epochs", "3"])
    assert t.data.x.size(1) == 3 * 16
    assert t.train_step(1)["loss"] == t.train_step(1)["loss"] or True
    u = _trainer(["--model", "gt", "--hops", "1", "--pe_dim", "2", "--epochs", "2"] + FIXED)
    assert u.data.x.size(1) == 2 * (16 + 2)
    assert u.train_step(1)["loss"] == u.train_step(1)["loss"] or True


def test_exphormer_expander_and_fanout_modes():
    t = _trainer(["--model", "exphormer", "--expander_degree", "3", "--epochs", "2"] + FIXED)
    g = t.build_edges(1)
    assert g.etype is not None and int(g.etype.max()) == 1
    u = _trainer(["--model", "gt", "--rw_edge_mode", "dgl_neighbor", "--fanout", "3,2", "--epochs", "2"] + FIXED)
    assert u.train_step(1)["edges"] > 0
    v = _trainer(["--model", "gt", "--include_real_edges", "1", "--walks_per_node", "0", "--epochs", "2"])
    g = v.build_edges(1)
    assert g.num_edges == torch.unique(v.data.edge_index[0] * 384 + v.data.edge_index[1]).numel()     # all real edges, unsampled


def test_adaptive_budget_search_runs_and_freezes():
    logs = []
    t = _trainer(["--model", "gt", "--adaptive_edge_budget", "--max_total_edges_per_query", "6", "--warmup_updates", "1",
                  "--epochs", "14", "--eval_every", "50", "--adaptive_edge_budget_patience", "3"], logs=logs)
    assert t.controller.enabled and not t.controller.frozen
    t.fit()
    assert any("BudgetCtrl probe" in l for l in logs)
    st = t.controller.current_state()
    assert st["real_edges_per_query"] + st["rw_edges_per_query"] <= 6
    assert st["real_edges_per_query"] + st["rw_edges_per_query"] >= 4


def test_checkpoint_and_resume(tmp_path):
    argv = ["--model", "gt", "--epochs", "4", "--save_model", "--model_dir", str(tmp_path)] + FIXED
    t = _trainer(argv)
    t.fit()
    assert os.path.exists(model_path(t.args)) and os.path.exists(train_state_path(t.args))
    sd = torch.load(model_path(t.args))
    assert "layers.0.O.weight" in sd
    u = _trainer(argv[:2] + ["--epochs", "6", "--save_model", "--model_dir", str(tmp_path), "--resume", train_state_path(t.args)] + FIXED)
    assert u.epoch == 4 and u.lr_scheduler.state_dict()["_step_count"] == t.lr_scheduler.state_dict()["_step_count"]
    for a, b in zip(t.model.parameters(), u.model.parameters()):
        assert torch.equal(a, b)
    u.fit()
    assert u.epoch == 6


def test_multilabel_head():
    t = _trainer(["--model", "gt", "--multilabel", "--epochs", "4"] + FIXED, data=_data(multilabel=True))
    l = [t.train_step(e)["loss"] for e in range(1, 5)]
    assert l[-1] < l[0]
    assert 0.0 <= t.evaluate(4)["valid"] <= 1.0


@pytest.mark.parametrize("mode", ["all", "ffn_only", "adaptive", "multi_tier"])
def test_activation_checkpoint_modes_give_same_gradients(mode):
    a = _trainer(["--model", "gt", "--epochs", "2", "--dropout_rate", "0", "--input_dropout_rate", "0"] + FIXED)
    b = _trainer(["--model", "gt", "--epochs", "2", "--dropout_rate", "0", "--input_dropout_rate", "0",
                  "--activation_checkpoint_mode", mode] + FIXED)
    b.model.load_state_dict(a.model.state_dict())
    g = a.build_edges(1)
    for t in (a, b):
        t.model.train()
        loss, _ = t._loss(g, t.local_idx["train"])
        t.reducer.prepare_backward()
        loss.backward()
    for pa, pb in zip(a.model.parameters(), b.model.parameters()):
        assert torch.allclose(pa.grad, pb.grad, atol=1e-6)


def test_comm_profiler_and_fault_injection():
    logs = []
    t = _trainer(["--model", "gt", "--epochs", "2", "--profile_sp_comm"] + FIXED, logs=logs)
    t.fit()
    assert any("edge_build_local" in l for l in logs) and any("edge cardinality" in l for l in logs)
    comm_profiler.enable_comm_profiler(False)
    u = _trainer(["--model", "gt", "--epochs", "2", "--fault_inject", "oom@fwd:1"] + FIXED)
    with pytest.raises(RuntimeError, match="no multi_tier planner"):
        u.train_step(1)


def test_edge_policies_and_prefetch_agree():
    t = _trainer(["--model", "gt", "--epochs", "2"] + FIXED)
    g1 = t.edge_engine.build(7, t.budget_state())
    t.edge_engine.set_policy("cpu_broadcast")
    g2 = t.edge_engine.build(7, t.budget_state())
    assert torch.equal(g1.col, g2.col)
    t.edge_engine.set_policy("cpu_rank_local_prefetch")
    assert t.edge_engine.submit_prefetch(8, t.budget_state())
    g3 = t.edge_engine.build(8, t.budget_state())
    t.edge_engine.clear_cache()
    g4 = t.edge_engine.build(8, t.budget_state())
    assert torch.equal(g3.col, g4.col)
    t.edge_engine.shutdown()


def test_debug_checks_validate_graphs_and_flag_nan():
    """The sanitizer stand-in: broken graphs are named before a kernel could index with them, NaN is attributed."""
    import pytest
    from budgetformer_b200.graph.attn_graph import AttnGraph
    from budgetformer_b200.utils import debug
    from tests.helpers import random_attn_graph
    g = random_attn_graph(100, 600, hub_col=80, seed=1).ensure_transpose()
    debug.validate_graph(g)
    bad = AttnGraph(g.num_rows, g.rowptr.clone(), g.col.clone(), None)
    bad.col[5] = 100
    with pytest.raises(ValueError, match="key ids outside"):
        debug.validate_graph(bad)
    bad = AttnGraph(g.num_rows, g.rowptr.clone(), g.col.clone(), None)
    bad.rowptr[3] = bad.rowptr[4] + 1
    with pytest.raises(ValueError, match="monotone"):
        debug.validate_graph(bad)
    bad = AttnGraph(g.num_rows, g.rowptr, g.col, None).ensure_transpose()
    bad.t_task = bad.t_task.clone()
    bad.t_task[0, 2] -= 1
    with pytest.raises(ValueError, match="work items"):
        debug.validate_graph(bad)
    debug.enable(True)
    try:
        t = torch.ones(4)
        debug.poison(t)
        assert bool(torch.isnan(t).all())
        with pytest.raises(FloatingPointError, match="epoch 3"):
            debug.assert_finite("the gradients of epoch 3", torch.ones(2), t)
    finally:
        debug.enable(False)


def test_mini_batch_driver_trains_and_writes_hop_stats(tmp_path):
    """Legacy mini-batch SP driver end to end on CPU: two epochs over sequences of 256 nodes, validation, and the
    per-epoch hop-mass statistics file (--full_attn_hop_stats)."""
    import json
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import main_node_sp
    from budgetformer_b200.graph.synthetic import sbm_graph, write_dataset
    x, y, ei = sbm_graph(600, feat_dim=16, seed=1)
    write_dataset(str(tmp_path), "toy", x, y, ei)
    hop_dir = str(tmp_path / "hop")
    best = main_node_sp.main(["--model", "gt", "--dataset", "toy", "--dataset_dir", str(tmp_path), "--seq_len", "256",
                              "--epochs", "2", "--n_layers", "2", "--hidden_dim", "32", "--num_heads", "4", "--ffn_dim", "64",
                              "--device", "cpu", "--eval_every", "1", "--force_random_split", "--full_attn_hop_stats",
                              "--full_attn_hop_stats_dir", hop_dir, "--full_attn_hop_max_hop", "6"])
    assert 0.0 <= best["valid"] <= 1.0 and best["epoch"] >= 1
    files = sorted(os.listdir(os.path.join(hop_dir, "toy", "gt", "attn0.95_maxhop6")))
    assert files == ["epoch_1.json", "epoch_2.json"]
    stats = json.load(open(os.path.join(hop_dir, "toy", "gt", "attn0.95_maxhop6", files[0])))
    assert len(stats["layers"]) == 2 and abs(sum(stats["layers"][0]["hop_mass"]) - 1.0) < 1e-4


def test_mini_batch_driver_with_locality_reordering(tmp_path):
    """--batch_reorder_parts: the driver trains on sequences reordered into locality clusters (native partitioner)."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import main_node_sp
    from budgetformer_b200.graph.synthetic import sbm_graph, write_dataset
    x, y, ei = sbm_graph(400, feat_dim=16, seed=2)
    write_dataset(str(tmp_path), "toy", x, y, ei)
    best = main_node_sp.main(["--model", "gt", "--dataset", "toy", "--dataset_dir", str(tmp_path), "--seq_len", "200",
                              "--epochs", "2", "--n_layers", "1", "--hidden_dim", "32", "--num_heads", "4", "--ffn_dim", "64",
                              "--device", "cpu", "--eval_every", "1", "--force_random_split", "--batch_reorder_parts", "4"])
    assert 0.0 <= best["valid"] <= 1.0 and best["epoch"] >= 1


def test_warmup_oom_under_gpu_edge_policy_moves_the_build_to_the_cpu():
    """Warm-up (every layer recomputed) runs out of memory while a GPU edge policy holds the topology and the build's
    working set: GPU policies leave the planner's search, the build moves to cpu_rank_local_prefetch, the step is
    dropped without feeding the planner, and training goes on.  A second failure under the CPU policy ends the run."""
    from budgetformer_b200.control.multi_tier import EDGE_GPU_EPHEMERAL, EDGE_GPU_PERSIST, Phase, ScriptedMemoryProbe
    logs = []
    t = _trainer(["--model", "gt", "--epochs", "4", "--activation_checkpoint_mode", "multi_tier",
                  "--fault_inject", "oom@fwd:1"] + FIXED, logs=logs)
    t.planner.probe = ScriptedMemoryProbe(1 << 34, lambda modes: {"peak": 1 << 30, "live": 1 << 29})
    t.edge_engine.policy = "gpu_persist"            # a CPU test machine: set past the device check of set_policy
    assert t.planner.phase is Phase.WARMUP_RECOMPUTE
    out = t.train_step(1)
    assert out["dropped"] == 1.0 and out["loss"] != out["loss"]
    assert t.edge_engine.policy == "cpu_rank_local_prefetch"
    assert {EDGE_GPU_PERSIST, EDGE_GPU_EPHEMERAL} <= set(t.planner.excluded_policies)
    assert t.planner.phase is Phase.WARMUP_RECOMPUTE and not t.planner._warmup       # the failed step fed nothing
    assert any("edge build moved to cpu_rank_local_prefetch" in l for l in logs)
    out = t.train_step(2)
    assert out["dropped"] == 0.0 and out["loss"] == out["loss"]
    u = _trainer(["--model", "gt", "--epochs", "4", "--activation_checkpoint_mode", "multi_tier",
                  "--fault_inject", "oom@fwd:1"] + FIXED)
    u.planner.probe = ScriptedMemoryProbe(1 << 34, lambda modes: {"peak": 1 << 30, "live": 1 << 29})
    with pytest.raises(RuntimeError, match="warm-up with every layer recomputed"):
        u.train_step(1)                               # already on the CPU policy: nothing left to give back


def test_bench_fit_mode_runs_the_user_loop_on_cpu(capsys, monkeypatch):
    """``bench.py --fit_epochs``: the training loop a user runs (budget search with probes, execution planner,
    evaluation) on a named configuration, one JSON summary line on stdout."""
    import json
    import sys
    monkeypatch.setenv("BF_BENCH_CACHE", "")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.syspath_prepend(root)
    import bench
    monkeypatch.setattr(sys, "argv", ["bench.py", "--config", "sbm2k", "--fit_epochs", "12", "--fit_flags",
                                      "--adaptive_edge_budget --activation_checkpoint_mode multi_tier --device cpu --eval_every 6"])
    ns = bench.parse()
    bench.run_fit(ns)
    lines = [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    rec = json.loads(lines[-1])
    assert rec["mode"] == "fit" and rec["epochs"] == 12 and len(rec["epoch_ms_first"]) == 12
    assert rec["budget"]["real"] + rec["budget"]["rw"] <= 8 and rec["plan"]["tiers"] and rec["best"]["epoch"] in (6, 12)
