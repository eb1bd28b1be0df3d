"""Execution planner and budget controller end to end on a GPU (small graph)."""
import pytest
import torch

from budgetformer_b200.config import parse_fullgraph_args
from budgetformer_b200.graph.synthetic import sbm_graph
from budgetformer_b200.ops import gemm
from budgetformer_b200.train.data import GraphData, random_split_idx
from budgetformer_b200.train.engine import FullGraphTrainer

pytestmark = pytest.mark.gpu


def _trainer(extra, n=4096, logs=None):
    x, y, ei = sbm_graph(n, feat_dim=64, seed=3)
    data = GraphData(x, y, ei, random_split_idx(n, 3), n, 7)
    argv = ["--model", "gt", "--dataset", "t", "--n_layers", "3", "--hidden_dim", "128", "--num_heads", "8", "--ffn_dim", "256",
            "--amp_dtype", "bf16", "--force_random_split", "--device", "cuda:0", "--seed", "5", "--peak_lr", "3e-3",
            "--eval_every", "100", "--epochs", "14"] + list(extra)
    log = (lambda *a, **k: logs.append(" ".join(str(v) for v in a))) if logs is not None else (lambda *a, **k: None)
    return FullGraphTrainer(parse_fullgraph_args(argv), data=data, log=log)


def test_multi_tier_calibrates_and_activates_on_gpu():
    logs = []
    t = _trainer(["--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4",
                  "--activation_checkpoint_mode", "multi_tier"], logs=logs)
    assert t.planner is not None and t.planner.state_name() == "WARMUP_RECOMPUTE"
    t.profile_edge_policies()
    t.fit()
    gemm.check_status("cuda")
    assert t.planner.is_active()
    assert t.planner.edge_policy in ("gpu_persist", "gpu_ephemeral", "cpu_rank_local_prefetch")
    assert t.edge_engine.policy == t.planner.edge_policy and t.edge_engine.policy_locked
    assert t.planner.modes() == ["retain"] * 3            # a 4k-node graph fits: everything is retained
    assert any("edge policy gpu_persist: build=" in l for l in logs)


def test_forced_plan_and_cpu_policy_on_gpu():
    t = _trainer(["--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4",
                  "--activation_checkpoint_mode", "multi_tier",
                  "--force_multi_tier_plan", "cpu_rank_local_prefetch:keep_mha=1"])
    assert t.planner.is_active() and t.planner.modes() == ["recompute", "recompute", "keep_mha"]
    assert t.edge_engine.policy == "cpu_rank_local_prefetch"
    losses = [t.train_step(e)["loss"] for e in range(1, 6)]
    assert losses[-1] < losses[0]
    # the CPU-built graph equals the GPU-built one
    g_cpu = t.edge_engine.build(99, t.budget_state())
    t.edge_engine.set_policy("gpu_persist")
    g_gpu = t.edge_engine.build(99, t.budget_state())
    assert torch.equal(g_cpu.col, g_gpu.col) and torch.equal(g_cpu.rowptr, g_gpu.rowptr)
    t.edge_engine.shutdown()


def test_adaptive_budget_with_deferred_planner_on_gpu():
    logs = []
    t = _trainer(["--adaptive_edge_budget", "--max_total_edges_per_query", "6", "--warmup_updates", "1",
                  "--activation_checkpoint_mode", "multi_tier", "--epochs", "22"], logs=logs)
    assert t.planner.state_name() == "DEFERRED"
    t.fit()
    assert t.controller.frozen
    assert t.planner.state_name() != "DEFERRED"          # the frozen budget released the planner
    assert any("BudgetCtrl" in l for l in logs)


def test_device_lookahead_build_matches_synchronous_build():
    """The graph built one epoch ahead on the side stream is the graph a synchronous build of that epoch gives, and
    training with the look-ahead reproduces training without it."""
    losses = {}
    for mode in ("ahead", "sync"):
        extra = ["--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4"]
        if mode == "sync":
            extra.append("--disable_edge_prefetch")
        torch.manual_seed(11)
        t = _trainer(extra)
        assert t.edge_engine.uses_device_prefetch() == (mode == "ahead")
        vals = []
        for epoch in range(1, 5):
            out = t.train_step(epoch)
            vals.append(out["loss"])
            if mode == "ahead" and epoch >= 2:
                g = t.last_graph
                ref = t.edge_engine._finalize(t.edge_engine._build_device(t.edge_seed(epoch), t.budget_state()))
                assert torch.equal(g.rowptr, ref.rowptr) and torch.equal(g.col, ref.col)
                assert g.t_rowptr is not None                  # transposition came with the look-ahead build
        t.edge_engine.shutdown()
        losses[mode] = vals
    gemm.check_status("cuda")
    assert all(abs(a - b) < 2e-3 for a, b in zip(losses["ahead"], losses["sync"])), losses


def test_training_with_debug_checks_and_nvtx_runs_clean():
    """--debug_checks (graph validation, NaN-poisoned gradient buffers after use, finite checks) and --nvtx on the fused
    path: four steps without a complaint and with a falling loss."""
    from budgetformer_b200.utils import debug
    t = _trainer(["--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4", "--debug_checks", "--nvtx"])
    try:
        assert debug.enabled() and t.fused_sp
        losses = [t.train_step(e)["loss"] for e in range(1, 7)]
    finally:
        debug.enable(False)
        t.edge_engine.shutdown()
    gemm.check_status("cuda")
    assert all(l == l for l in losses) and losses[-1] < losses[0]
