"""Budget controller and execution planner decision logic (pure CPU)."""
import pytest

from budgetformer_b200.control.budget import (AdaptiveEdgeBudgetConfig, AdaptiveEdgeBudgetController, decide_budget_move,
                                              fixed_budget_controller, resolve_adaptive_edge_budget_config)
from budgetformer_b200.control.multi_tier import (EDGE_CPU_RANK_LOCAL_PREFETCH, EDGE_GPU_EPHEMERAL, EDGE_GPU_PERSIST,
                                                  ScriptedMemoryProbe, _MultiTierResourceManager, CommAwareCheckpointer,
                                                  parse_force_multi_tier_plan)

MIB = 2 ** 20


def _ctrl(max_total=8, rw_max=8, patience=3):
    return AdaptiveEdgeBudgetController(AdaptiveEdgeBudgetConfig(enabled=True, max_total_edges_per_query=max_total,
                                                                 rw_max_per_query=rw_max, patience=patience))


def test_controller_initial_state_and_candidates():
    c = _ctrl()
    assert c.current_state() == {"real_edges_per_query": 2, "rw_edges_per_query": 2}
    cands = c.candidate_states()
    assert set(cands) == {"real_up", "rw_up"}
    assert cands["real_up"]["real_edges_per_query"] == 4 and cands["rw_up"]["rw_edges_per_query"] == 4


def test_controller_confirmation_rounds_grow_with_updates():
    c = _ctrl()
    s = c.candidate_states()["real_up"]
    c.update("real_up", 0.1, s)                      # 1st move: 1 win suffices
    assert c.real_budget == 4 and c._n_budget_updates == 1
    s = c.candidate_states()["rw_up"]
    c.update("rw_up", 0.1, s)                        # 2nd move needs 2 consecutive wins
    assert c.rw_budget == 2 and c._pending_wins == 1
    c.update("real_up", 0.1, c.candidate_states()["real_up"])   # direction change restarts confirmation
    assert c._pending_kind == "real_up" and c._pending_wins == 1
    c.update("real_up", 0.1, c.candidate_states()["real_up"])
    assert c.real_budget == 6 and c._n_budget_updates == 2


def test_controller_ceiling_offers_shifts_and_rw_cap():
    c = _ctrl(max_total=8, rw_max=4)
    c.real_budget, c.rw_budget = 4, 4
    cands = c.candidate_states()
    assert set(cands) == {"shift_to_real"}            # rw is at its realisable cap (W*L = 4)
    c.rw_budget, c.real_budget = 2, 6
    assert set(c.candidate_states()) == {"shift_to_real", "shift_to_rw"}


def test_controller_patience_freezes():
    c = _ctrl(patience=3)
    for _ in range(3):
        assert not c.frozen
        c.update(None, -0.1, None)
    assert c.frozen


def test_controller_memory_gate_and_force_shrink():
    c = AdaptiveEdgeBudgetController(AdaptiveEdgeBudgetConfig(enabled=True, max_total_edges_per_query=16,
                                                             rw_max_per_query=16, gpu_limit_mib=1000))
    c.observe_peak(500)                               # B = 4
    c.real_budget = 4
    c.observe_peak(800)                               # B = 6: slope 150 MiB per edge
    assert "real_up" not in c.candidate_states()      # 800 + 2*150 = 1100 > 900
    c.observe_peak(950)
    assert c._over_budget
    st = c.force_shrink()
    assert st["real_edges_per_query"] + st["rw_edges_per_query"] == 4


def test_fixed_controller_is_frozen():
    c = fixed_budget_controller(4, 4, 6)
    assert c.frozen and c.current_state() == {"real_edges_per_query": 4, "rw_edges_per_query": 4, "walk_length": 6}


def test_decide_budget_move_growth_and_acc_tiebreak():
    c = _ctrl()
    rows = [{"kind": "current", "state": c.current_state(), "loss": 1.0, "acc": 0.5, "edges": 10},
            {"kind": "real_up", "state": c.candidate_states()["real_up"], "loss": 0.9, "acc": 0.5, "edges": 12},
            {"kind": "rw_up", "state": c.candidate_states()["rw_up"], "loss": 0.95, "acc": 0.6, "edges": 12}]
    assert decide_budget_move(c, rows, 6) == "grow"
    assert c.real_budget == 4 and c.auto_hold_released
    c.real_budget, c.rw_budget = 4, 4                # at the ceiling: |gain| < 1 % everywhere -> accuracy decides
    cands = c.candidate_states()
    rows = [{"kind": "current", "state": c.current_state(), "loss": 1.0, "acc": 0.5, "edges": 10},
            {"kind": "shift_to_real", "state": cands["shift_to_real"], "loss": 0.999, "acc": 0.50, "edges": 10},
            {"kind": "shift_to_rw", "state": cands["shift_to_rw"], "loss": 0.9995, "acc": 0.55, "edges": 10}]
    decide_budget_move(c, rows, 7)
    assert c._pending_kind == "shift_to_rw"


def test_config_resolution_defaults():
    class A:
        adaptive_edge_budget = True
        max_total_edges_per_query = 8
        walks_per_node, walk_length = 2, 4
    cfg = resolve_adaptive_edge_budget_config(A())
    assert cfg.block_size == 2 and cfg.patience == 3 and cfg.warmup_epochs is None and cfg.rw_max_per_query == 8


# ---------------------------------------------------------------------------------------------------- planner
def _scripted(total_mib, base=1000, mha=300, full=800, last_mha=50, last_full=120):
    def fn(modes):
        extra = 0
        n = len(modes)
        for i, m in enumerate(modes):
            last = i == n - 1
            if m == "keep_mha":
                extra += last_mha if last else mha
            elif m == "retain":
                extra += last_full if last else full
        live = 400 + sum({"keep_mha": mha, "retain": full}.get(m, 0) for m in modes)
        return {"peak": (base + extra) * MIB, "live": live * MIB}
    return ScriptedMemoryProbe(total_mib * MIB, fn)


def _calibrate(p, t_rec=(0.10, 0.30), t_mha=(0.10, 0.25), t_ret=(0.09, 0.20)):
    seq = []
    for _ in range(20):
        if p.is_active():
            break
        p.plan("cpu")
        p.record_post_forward_memory("cpu")
        seq.append(p.state_name())
        s = p.state_name()
        t = t_rec if "WARMUP" in s else t_mha if "MHA" in s else t_ret
        p.notify_step_end("cpu", t_bwd=t[1], t_fwd=t[0])
    return seq


def test_planner_state_machine_order_and_all_retain_when_memory_allows():
    p = _MultiTierResourceManager(4, probe=_scripted(100000), verbose=False)
    seq = _calibrate(p)
    assert seq == ["WARMUP_RECOMPUTE"] * 3 + ["CALIBRATE_MHA", "CALIBRATE_MHA_FRONT", "CALIBRATE_RETAIN", "CALIBRATE_RETAIN_FRONT"]
    assert p.is_active() and p.modes() == ["retain"] * 4


def test_planner_respects_memory_cap():
    # cap 2300 MiB * 0.9 = 2070: base 1000 + last retain 120 + one more retain 800 = 1920 fits; a third does not
    p = _MultiTierResourceManager(4, probe=_scripted(2300), verbose=False)
    _calibrate(p, t_mha=(0.10, 0.30))                 # keeping only the attention half buys no time here
    m = p.modes()
    assert m.count("retain") == 2 and m[-2:] == ["retain", "retain"]
    peak = _scripted(2300)._fn(m)["peak"]
    assert peak <= 2300 * MIB * 0.9


def test_planner_deferred_then_frozen():
    p = _MultiTierResourceManager(2, deferred=True, probe=_scripted(100000), verbose=False)
    p.plan("cpu"); p.record_post_forward_memory("cpu"); p.notify_step_end("cpu", 0.3, 0.1)
    assert p.state_name() == "DEFERRED" and p.modes() == ["recompute"] * 2
    p.notify_budget_frozen(reuse_deferred_baseline=True)
    assert p.state_name() == "CALIBRATE_MHA"


def test_planner_picks_cpu_policy_when_gpu_build_exceeds_cap():
    p = _MultiTierResourceManager(2, probe=_scripted(3000), verbose=False)
    p.set_edge_policy_profile(EDGE_GPU_PERSIST, 0.01, gpu_peak_bytes=5000 * MIB, cpu_delta_bytes=0, live_edge_bytes=900 * MIB)
    p.set_edge_policy_profile(EDGE_GPU_EPHEMERAL, 0.02, gpu_peak_bytes=5000 * MIB, cpu_delta_bytes=0)
    p.set_edge_policy_profile(EDGE_CPU_RANK_LOCAL_PREFETCH, 0.5, gpu_peak_bytes=1000 * MIB, cpu_delta_bytes=100 * MIB,
                              serial_time_s=0.0, overlap_time_s=0.5)
    _calibrate(p)
    assert p.edge_policy == EDGE_CPU_RANK_LOCAL_PREFETCH
    # uncapped: the GPU policy wins on time
    q = _MultiTierResourceManager(2, probe=_scripted(100000), verbose=False)
    for pol, args in ((EDGE_GPU_PERSIST, (0.01, 5000 * MIB, 0, 900 * MIB)), (EDGE_CPU_RANK_LOCAL_PREFETCH, (0.5, 1000 * MIB, 0, 0))):
        q.set_edge_policy_profile(pol, args[0], args[1], args[2], args[3], serial_time_s=args[0] if pol == EDGE_GPU_PERSIST else 0.9)
    _calibrate(q)
    assert q.edge_policy == EDGE_GPU_PERSIST and q.cache_edge


def test_planner_oom_fallback_and_calibration_infeasible():
    p = _MultiTierResourceManager(3, probe=_scripted(100000), verbose=False)
    _calibrate(p)
    assert p.modes() == ["retain"] * 3
    assert p.apply_oom_fallback("cpu")
    assert p.modes() == ["keep_mha", "retain", "retain"]
    q = _MultiTierResourceManager(3, probe=_scripted(100000), verbose=False)
    for _ in range(3):
        q.plan("cpu"); q.record_post_forward_memory("cpu"); q.notify_step_end("cpu", 0.3, 0.1)
    assert q.state_name() == "CALIBRATE_MHA"
    assert q.mark_current_calibration_infeasible("cpu") and q.state_name() == "CALIBRATE_RETAIN"
    _calibrate(q)
    assert "keep_mha" not in q.modes()


def test_planner_reconsider_and_gpu_infeasible():
    p = _MultiTierResourceManager(2, probe=_scripted(100000), verbose=False)
    p.set_edge_policy_profile(EDGE_GPU_EPHEMERAL, 0.3, 1000 * MIB, 0, serial_time_s=0.3)
    p.set_edge_policy_profile(EDGE_CPU_RANK_LOCAL_PREFETCH, 0.2, 1000 * MIB, 0, serial_time_s=0.0, overlap_time_s=0.2)
    _calibrate(p)
    assert p.edge_policy == EDGE_CPU_RANK_LOCAL_PREFETCH
    assert p.reconsider_with_actual_timing("cpu", 0.3, 0.2) is None          # wait not 0.5 s worse than the GPU build
    assert p.reconsider_with_actual_timing("cpu", 0.3, 1.5) == EDGE_GPU_EPHEMERAL
    assert p.report_runtime_edge_gpu_infeasible("cpu")
    assert p.edge_policy == EDGE_CPU_RANK_LOCAL_PREFETCH


def test_force_plan_parser():
    assert parse_force_multi_tier_plan("", 4) is None
    assert parse_force_multi_tier_plan("gpu_persist:recompute", 3) == ("gpu_persist", ["recompute"] * 3)
    pol, tiers = parse_force_multi_tier_plan("cpu_rank_local_prefetch:keep_mha=2", 4)
    assert pol == "cpu_rank_local_prefetch" and tiers == ["recompute", "recompute", "keep_mha", "keep_mha"]
    with pytest.raises(ValueError):
        parse_force_multi_tier_plan("nope:recompute", 4)
    with pytest.raises(ValueError):
        parse_force_multi_tier_plan("gpu_persist:retain=9", 4)


def test_comm_aware_checkpointer_greedy_from_the_back():
    probe = _scripted(1900, mha=300)
    c = CommAwareCheckpointer(4, probe=probe)
    for _ in range(2):
        c.plan("cpu"); c.record_post_forward_memory("cpu"); c.notify_step_end("cpu")
    assert c.is_active()
    assert [c.mode(i) for i in range(4)] == ["layer", "layer", "keep_mha", "keep_mha"]   # 1000 + 2*300 <= 1710 < 1000 + 3*300


def test_block_rounding_and_initial_candidates():
    from budgetformer_b200.control.budget import (AdaptiveEdgeBudgetConfig, auto_initial_budget_candidates,
                                                  floor_budget_to_block, round_budget_to_block)
    assert [round_budget_to_block(v, 4) for v in (0, 1, 4, 5)] == [0, 4, 4, 8]
    assert [floor_budget_to_block(v, 4) for v in (0, 1, 4, 7, 8)] == [0, 4, 4, 4, 8]
    cfg = AdaptiveEdgeBudgetConfig(max_total_edges_per_query=8, block_size=2)
    pairs = [(c["real_edges_per_query"], c["rw_edges_per_query"]) for c in auto_initial_budget_candidates(cfg)]
    assert pairs == [(2, 0), (4, 0), (2, 2), (4, 2), (2, 4), (8, 0), (4, 4)]
    assert all(r + w <= 8 for r, w in pairs)
    tiny = AdaptiveEdgeBudgetConfig(max_total_edges_per_query=1, block_size=2)
    assert auto_initial_budget_candidates(tiny) == [{"real_edges_per_query": 1, "rw_edges_per_query": 0}]
    assert auto_initial_budget_candidates(AdaptiveEdgeBudgetConfig(max_total_edges_per_query=0)) == []


def test_model_state_snapshot_and_dropout_scope():
    import torch
    from budgetformer_b200.utils.misc import clone_model_state_to_cpu, dropout_disabled
    m = torch.nn.Sequential(torch.nn.Linear(3, 3), torch.nn.Dropout(0.5), torch.nn.BatchNorm1d(3))
    snap = clone_model_state_to_cpu(m)
    with torch.no_grad():
        m[0].weight.add_(1.0)
    assert not torch.equal(snap["0.weight"], m[0].weight) and snap["0.weight"].device.type == "cpu"
    m.train()
    with dropout_disabled(m):
        assert not m[1].training and m[2].training and m.training
    assert m[1].training
    m[1].eval()
    with dropout_disabled(m):
        pass
    assert not m[1].training                                 # the previous mode comes back, whatever it was
