"""Budget controller and execution planner decision logic (pure CPU)."""
import pytest

from dataclasses import replace

from budgetformer_b200.control.budget import (AdaptiveEdgeBudgetConfig, BudgetSearch, Limits, SearchState, Split,
                                              after_round, decide_budget_move, fixed_budget_controller, initial_state,
                                              judge_round, offers, projected_peak_mib, resolve_adaptive_edge_budget_config,
                                              shrunk, wins_needed, with_peak)
from budgetformer_b200.control.multi_tier import (EDGE_CPU_RANK_LOCAL_PREFETCH, EDGE_GPU_EPHEMERAL, EDGE_GPU_PERSIST,
                                                  ScriptedMemoryProbe, ExecutionPlanner, CommAwareCheckpointer,
                                                  parse_force_multi_tier_plan)

MIB = 2 ** 20


def _ctrl(max_total=8, rw_max=8, patience=3):
    return BudgetSearch(AdaptiveEdgeBudgetConfig(enabled=True, max_total_edges_per_query=max_total,
                                                 rw_max_per_query=rw_max, patience=patience))


def _lim(ceiling=8, walk_cap=8, patience=3, hbm=0.0):
    return Limits(ceiling=ceiling, step=2, walk_cap=walk_cap, patience=patience, hbm_limit_mib=hbm)


def test_controller_initial_state_and_candidates():
    c = _ctrl()
    assert c.current_state() == {"real_edges_per_query": 2, "rw_edges_per_query": 2}
    cands = c.candidate_states()
    assert set(cands) == {"real_up", "rw_up"}
    assert cands["real_up"]["real_edges_per_query"] == 4 and cands["rw_up"]["rw_edges_per_query"] == 4


@pytest.mark.parametrize("split, ceiling, walk_cap, expected", [
    # below the ceiling: growth only
    ((2, 2), 8, 8, {"real_up": (4, 2), "rw_up": (2, 4)}),
    ((2, 2), 8, 2, {"real_up": (4, 2)}),                                  # walk side already at W*L
    ((4, 2), 8, 8, {"real_up": (6, 2), "rw_up": (4, 4)}),                 # one block of room: growth, no shifts yet
    # at the ceiling: shifts only
    ((4, 4), 8, 8, {"shift_to_real": (6, 2), "shift_to_rw": (2, 6)}),
    ((4, 4), 8, 4, {"shift_to_real": (6, 2)}),
    ((8, 0), 8, 8, {"shift_to_rw": (6, 2)}),                              # nothing to take from the walk side
    ((0, 8), 8, 8, {"shift_to_real": (2, 6)}),
    # an odd ceiling leaves one edge unused: neither a growth step nor "at the ceiling"
    ((4, 4), 9, 9, {}),
    ((0, 0), 0, 0, {}),
])
def test_offer_table(split, ceiling, walk_cap, expected):
    st = SearchState(Split(*split), frozen=False)
    got = {k: (v.real, v.walk) for k, v in offers(st, _lim(ceiling, walk_cap)).items()}
    assert got == expected


def test_initial_state_table():
    assert initial_state(_lim(8, 8), True).split == Split(2, 2)
    assert initial_state(_lim(8, 1), True).split == Split(2, 1)           # W*L = 1 caps the walk side
    assert initial_state(_lim(0, 0), True).split == Split(0, 0)
    off = initial_state(_lim(8, 8), False)
    assert off.frozen and off.split == Split(8, 0)


def test_confirm_rule_table():
    """The n-th committed move needs min(n, 3) consecutive wins of one kind."""
    st = SearchState(Split(2, 2), frozen=False)
    assert [wins_needed(replace(st, commits=n)) for n in range(5)] == [1, 2, 3, 3, 3]
    lim = _lim(32, 32)
    # first move: immediate
    st = after_round(st, lim, "real_up", 0.1, Split(4, 2))
    assert st.split == Split(4, 2) and st.commits == 1 and st.streak_len == 0
    # second move: win, interruption by another kind, then two in a row
    st = after_round(st, lim, "rw_up", 0.1, Split(4, 4))
    assert st.split == Split(4, 2) and (st.streak_kind, st.streak_len) == ("rw_up", 1)
    st = after_round(st, lim, "real_up", 0.1, Split(6, 2))
    assert (st.streak_kind, st.streak_len) == ("real_up", 1)
    st = after_round(st, lim, "real_up", 0.2, Split(6, 2))
    assert st.split == Split(6, 2) and st.commits == 2
    # a "stay" round voids the streak
    st = after_round(st, lim, "rw_up", 0.1, Split(6, 4))
    st = after_round(st, lim, None, 0.0, None)
    assert st.streak_kind is None and st.streak_len == 0 and st.dry_rounds == 1


def test_controller_confirmation_rounds_grow_with_updates():
    c = _ctrl()
    s = c.candidate_states()["real_up"]
    c.update("real_up", 0.1, s)                      # 1st move: 1 win suffices
    assert c.real_budget == 4 and c.state.commits == 1
    s = c.candidate_states()["rw_up"]
    c.update("rw_up", 0.1, s)                        # 2nd move needs 2 consecutive wins
    assert c.rw_budget == 2 and c.state.streak_len == 1
    c.update("real_up", 0.1, c.candidate_states()["real_up"])   # direction change restarts confirmation
    assert c.state.streak_kind == "real_up" and c.state.streak_len == 1
    c.update("real_up", 0.1, c.candidate_states()["real_up"])
    assert c.real_budget == 6 and c.state.commits == 2


def test_controller_ceiling_offers_shifts_and_rw_cap():
    c = _ctrl(max_total=8, rw_max=4)
    c.set_split(4, 4)
    cands = c.candidate_states()
    assert set(cands) == {"shift_to_real"}            # rw is at its realisable cap (W*L = 4)
    c.set_split(6, 2)
    assert set(c.candidate_states()) == {"shift_to_real", "shift_to_rw"}


def test_controller_patience_freezes():
    c = _ctrl(patience=3)
    for _ in range(3):
        assert not c.frozen
        c.update(None, -0.1, None)
    assert c.frozen


def test_patience_counts_only_non_positive_rounds_and_resets_on_commit():
    lim = _lim(32, 32, patience=3)
    st = SearchState(Split(2, 2), frozen=False, commits=1)
    st = after_round(st, lim, None, -0.1, None)
    st = after_round(st, lim, None, 0.0, None)
    assert st.dry_rounds == 2 and not st.frozen
    st = after_round(st, lim, "real_up", 0.3, Split(4, 2))        # pending (needs 2): the count stands
    assert st.dry_rounds == 2
    st = after_round(st, lim, "real_up", 0.3, Split(4, 2))        # committed: the count restarts
    assert st.dry_rounds == 0 and st.split == Split(4, 2)
    for _ in range(3):
        st = after_round(st, lim, None, -1.0, None)
    assert st.frozen


def test_memory_gate_table():
    assert projected_peak_mib((), 8) is None
    assert projected_peak_mib(((4, 500.0),), 8) is None                       # one reading: nothing to extend
    pts = ((4, 500.0), (6, 800.0), (8, 900.0))
    assert projected_peak_mib(pts, 6) == 900.0                                # at or below the top reading: that reading
    assert projected_peak_mib(pts, 10) == 900.0 + 150.0 * 2                   # steepest slope (4 -> 6), not the last one
    lim = _lim(16, 16, hbm=1000.0)
    st = SearchState(Split(2, 2), frozen=False)
    st = with_peak(st, lim, 500.0)
    st = with_peak(replace(st, split=Split(4, 2)), lim, 800.0)
    assert "real_up" not in offers(st, lim) and "rw_up" not in offers(st, lim)   # 800 + 2 * 150 > 900
    assert not st.over_limit
    st = with_peak(st, lim, 950.0)
    assert st.over_limit and dict(st.peaks)[6] == 950.0                       # highest reading per budget is kept
    assert with_peak(replace(st, frozen=True), lim, 2000.0) == replace(st, frozen=True)   # frozen: readings ignored


@pytest.mark.parametrize("split, expected", [((4, 4), (4, 2)), ((6, 2), (4, 2)), ((2, 6), (2, 4)), ((1, 0), (1, 0)),
                                             ((0, 1), (0, 1)), ((0, 0), (0, 0)), ((1, 6), (1, 4)), ((6, 1), (4, 1))])
def test_forced_shrink_table(split, expected):
    st = SearchState(Split(*split), frozen=False, over_limit=True, streak_kind="real_up", streak_len=1,
                     streak_target=Split(9, 9))
    out = shrunk(st, _lim(16, 16))
    assert (out.split.real, out.split.walk) == expected and not out.over_limit
    if sum(split) > 0:
        assert out.streak_kind is None and out.streak_len == 0


def test_controller_memory_gate_and_force_shrink():
    c = BudgetSearch(AdaptiveEdgeBudgetConfig(enabled=True, max_total_edges_per_query=16,
                                              rw_max_per_query=16, gpu_limit_mib=1000))
    c.observe_peak(500)                               # B = 4
    c.set_split(4, 2)
    c.observe_peak(800)                               # B = 6: slope 150 MiB per edge
    assert "real_up" not in c.candidate_states()      # 800 + 2*150 = 1100 > 900
    c.observe_peak(950)
    assert c.over_limit
    st = c.force_shrink()
    assert st["real_edges_per_query"] + st["rw_edges_per_query"] == 4


def test_fixed_controller_is_frozen():
    c = fixed_budget_controller(4, 4, 6)
    assert c.frozen and c.current_state() == {"real_edges_per_query": 4, "rw_edges_per_query": 4, "walk_length": 6}


def _row(kind, state, loss, acc=0.5, edges=10):
    return {"kind": kind, "state": state, "loss": loss, "acc": acc, "edges": edges}


def test_decide_budget_move_growth_and_acc_tiebreak():
    c = _ctrl()
    rows = [_row("current", c.current_state(), 1.0), _row("real_up", c.candidate_states()["real_up"], 0.9, edges=12),
            _row("rw_up", c.candidate_states()["rw_up"], 0.95, acc=0.6, edges=12)]
    assert decide_budget_move(c, rows, 6) == "grow"
    assert c.real_budget == 4 and c.state.hold_open
    c.set_split(4, 4)                                 # at the ceiling: |gain| < 1 % everywhere -> accuracy decides
    cands = c.candidate_states()
    rows = [_row("current", c.current_state(), 1.0), _row("shift_to_real", cands["shift_to_real"], 0.999, acc=0.50),
            _row("shift_to_rw", cands["shift_to_rw"], 0.9995, acc=0.55)]
    decide_budget_move(c, rows, 7)
    assert c.state.streak_kind == "shift_to_rw"


def test_round_table_hold_and_blank_rounds():
    lim = _lim(8, 8)
    st = SearchState(Split(4, 4), frozen=False)                   # at the ceiling, nothing gained yet: held
    cur = st.split.as_dict()
    cands = {k: v.as_dict() for k, v in offers(st, lim).items()}

    def table(loss_real, loss_rw):
        return [_row("current", cur, 1.0), _row("shift_to_real", cands["shift_to_real"], loss_real),
                _row("shift_to_rw", cands["shift_to_rw"], loss_rw)]

    out = judge_round(st, lim, table(1.2, 1.1))                   # both worse: stay, one dry round
    assert out.tag == "auto_hold" and out.state.dry_rounds == 1 and out.state.split == Split(4, 4)
    out = judge_round(st, lim, table(0.8, 1.1))                   # a gain opens the hold and (first move) commits
    assert out.tag == "update" and out.state.hold_open and out.state.split == Split(6, 2)
    blank = st
    for i in range(5):                                            # every candidate failed, five rounds running
        out = judge_round(blank, lim, table(float("inf"), float("nan")))
        blank = out.state
        assert out.tag == ("auto_hold_frozen" if i == 4 else "auto_hold")
    assert blank.frozen
    opened = replace(st, hold_open=True)
    out = judge_round(opened, lim, table(float("inf"), float("inf")))
    assert out.tag == "update" and out.state.dry_rounds == 1      # after the hold, failures are ordinary dry rounds
    rows = table(0.5, 2.0)
    judge_round(opened, lim, rows)
    assert rows[0]["gain"] == 0.0 and rows[1]["gain"] == 0.5 and rows[2]["gain"] == -1.0


def test_round_table_growth_below_ceiling_uses_best_growing_row_even_when_negative():
    lim = _lim(8, 8, patience=3)
    st = SearchState(Split(2, 2), frozen=False, commits=1)
    cands = {k: v.as_dict() for k, v in offers(st, lim).items()}
    rows = [_row("current", st.split.as_dict(), 1.0), _row("real_up", cands["real_up"], 1.05),
            _row("rw_up", cands["rw_up"], 1.02)]
    out = judge_round(st, lim, rows)
    assert out.tag == "grow" and not out.state.hold_open
    assert (out.state.streak_kind, out.state.streak_len) == ("rw_up", 1)     # least bad growth row still accumulates wins


def test_search_state_round_trips_through_state_dict():
    c = _ctrl()
    c.update("real_up", 0.1, c.candidate_states()["real_up"])
    c.update("rw_up", 0.1, c.candidate_states()["rw_up"])
    c.observe_peak(123.0)
    d = _ctrl()
    d.load_state_dict(c.state_dict())
    assert d.state == c.state


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
    p = ExecutionPlanner(4, probe=_scripted(100000), verbose=False)
    seq = _calibrate(p)
    assert seq == ["WARMUP_RECOMPUTE"] * 3 + ["CALIBRATE_MHA", "CALIBRATE_MHA_FRONT", "CALIBRATE_RETAIN", "CALIBRATE_RETAIN_FRONT"]
    assert p.is_active() and p.modes() == ["retain"] * 4


def test_planner_respects_memory_cap():
    # cap 2300 MiB * 0.9 = 2070: base 1000 + last retain 120 + one more retain 800 = 1920 fits; a third does not
    p = ExecutionPlanner(4, probe=_scripted(2300), verbose=False)
    _calibrate(p, t_mha=(0.10, 0.30))                 # keeping only the attention half buys no time here
    m = p.modes()
    assert m.count("retain") == 2 and m[-2:] == ["retain", "retain"]
    peak = _scripted(2300)._fn(m)["peak"]
    assert peak <= 2300 * MIB * 0.9


def test_planner_deferred_then_frozen():
    p = ExecutionPlanner(2, deferred=True, probe=_scripted(100000), verbose=False)
    p.plan("cpu"); p.record_post_forward_memory("cpu"); p.notify_step_end("cpu", 0.3, 0.1)
    assert p.state_name() == "DEFERRED" and p.modes() == ["recompute"] * 2
    p.notify_budget_frozen(reuse_deferred_baseline=True)
    assert p.state_name() == "CALIBRATE_MHA"


def test_planner_picks_cpu_policy_when_gpu_build_exceeds_cap():
    p = ExecutionPlanner(2, probe=_scripted(3000), verbose=False)
    p.set_edge_policy_profile(EDGE_GPU_PERSIST, 0.01, gpu_peak_bytes=5000 * MIB, cpu_delta_bytes=0, live_edge_bytes=900 * MIB)
    p.set_edge_policy_profile(EDGE_GPU_EPHEMERAL, 0.02, gpu_peak_bytes=5000 * MIB, cpu_delta_bytes=0)
    p.set_edge_policy_profile(EDGE_CPU_RANK_LOCAL_PREFETCH, 0.5, gpu_peak_bytes=1000 * MIB, cpu_delta_bytes=100 * MIB,
                              serial_time_s=0.0, overlap_time_s=0.5)
    _calibrate(p)
    assert p.edge_policy == EDGE_CPU_RANK_LOCAL_PREFETCH
    # uncapped: the GPU policy wins on time
    q = ExecutionPlanner(2, probe=_scripted(100000), verbose=False)
    for pol, args in ((EDGE_GPU_PERSIST, (0.01, 5000 * MIB, 0, 900 * MIB)), (EDGE_CPU_RANK_LOCAL_PREFETCH, (0.5, 1000 * MIB, 0, 0))):
        q.set_edge_policy_profile(pol, args[0], args[1], args[2], args[3], serial_time_s=args[0] if pol == EDGE_GPU_PERSIST else 0.9)
    _calibrate(q)
    assert q.edge_policy == EDGE_GPU_PERSIST and q.cache_edge


def test_planner_oom_fallback_and_calibration_infeasible():
    p = ExecutionPlanner(3, probe=_scripted(100000), verbose=False)
    _calibrate(p)
    assert p.modes() == ["retain"] * 3
    assert p.apply_oom_fallback("cpu")
    assert p.modes() == ["keep_mha", "retain", "retain"]
    q = ExecutionPlanner(3, probe=_scripted(100000), verbose=False)
    for _ in range(3):
        q.plan("cpu"); q.record_post_forward_memory("cpu"); q.notify_step_end("cpu", 0.3, 0.1)
    assert q.state_name() == "CALIBRATE_MHA"
    assert q.mark_current_calibration_infeasible("cpu") and q.state_name() == "CALIBRATE_RETAIN"
    _calibrate(q)
    assert "keep_mha" not in q.modes()


def test_planner_reconsider_and_gpu_infeasible():
    p = ExecutionPlanner(2, probe=_scripted(100000), verbose=False)
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


# ---------------------------------------------------------------------------------------------------- planner tables
def _cal(n=4, base=(1000, 400, 0.10, 0.30), keep_last=(1050, 700, 0.10, 0.25), keep_front=None,
         ret_last=(1120, 1200, 0.09, 0.20), ret_front=None, **flags):
    from budgetformer_b200.control.multi_tier import Calibration, StepReading, TierProbe
    rd = lambda t: None if t is None else StepReading(t[0] * MIB, t[1] * MIB, t[2], t[3])
    keep = TierProbe(rd(keep_last), rd(keep_front), flags.get("keep_impossible", False), flags.get("keep_last_only", False))
    ret = TierProbe(rd(ret_last), rd(ret_front), flags.get("ret_impossible", False), flags.get("ret_last_only", False))
    return Calibration(n, rd(base), keep, ret)


def test_phase_table_and_probe_layouts():
    from budgetformer_b200.control.multi_tier import Phase, StepReading, advance, after_failed_probe, probe_layout
    assert probe_layout(Phase.WARMUP_RECOMPUTE, 3) == ["recompute"] * 3
    assert probe_layout(Phase.CALIBRATE_MHA, 3) == ["recompute", "recompute", "keep_mha"]
    assert probe_layout(Phase.CALIBRATE_MHA_FRONT, 3) == ["keep_mha", "recompute", "recompute"]
    assert probe_layout(Phase.CALIBRATE_RETAIN, 3) == ["recompute", "recompute", "retain"]
    assert probe_layout(Phase.CALIBRATE_RETAIN_FRONT, 3) == ["retain", "recompute", "recompute"]
    cal = _cal(keep_last=None, ret_last=None)
    fits = StepReading(1050 * MIB, 700 * MIB, 0.1, 0.25)            # +300 MiB alive: a second layer fits under 2000
    nxt, c2 = advance(Phase.CALIBRATE_MHA, cal, fits, 2000 * MIB)
    assert nxt is Phase.CALIBRATE_MHA_FRONT and c2.keep.last == fits and not c2.keep.last_layer_only
    nxt, c2 = advance(Phase.CALIBRATE_MHA, cal, fits, 1200 * MIB)   # 1000 + 300 > 1200: front probe skipped
    assert nxt is Phase.CALIBRATE_RETAIN and c2.keep.last_layer_only
    nxt, c2 = advance(Phase.CALIBRATE_MHA_FRONT, c2, fits, 2000 * MIB)
    assert nxt is Phase.CALIBRATE_RETAIN and c2.keep.front == fits
    nxt, _ = advance(Phase.CALIBRATE_RETAIN, cal, fits, 2000 * MIB)
    assert nxt is Phase.CALIBRATE_RETAIN_FRONT
    nxt, _ = advance(Phase.CALIBRATE_RETAIN_FRONT, cal, fits, 2000 * MIB)
    assert nxt is Phase.ACTIVE
    one = _cal(n=1, keep_last=None, ret_last=None)                  # a single layer has no "front"
    assert advance(Phase.CALIBRATE_MHA, one, fits, 2000 * MIB)[0] is Phase.CALIBRATE_RETAIN
    assert advance(Phase.CALIBRATE_RETAIN, one, fits, 2000 * MIB)[0] is Phase.ACTIVE
    # out of memory during a probe
    assert after_failed_probe(Phase.WARMUP_RECOMPUTE, cal) is None
    nxt, c3 = after_failed_probe(Phase.CALIBRATE_MHA, cal)
    assert nxt is Phase.CALIBRATE_RETAIN and c3.keep.impossible
    nxt, c3 = after_failed_probe(Phase.CALIBRATE_RETAIN_FRONT, cal)
    assert nxt is Phase.ACTIVE and c3.retain.last_layer_only and not c3.retain.impossible


def test_warmup_baseline_drops_first_sample():
    from budgetformer_b200.control.multi_tier import StepReading, warmup_baseline
    s = [StepReading(900, 10, 1.0, 3.0), StepReading(500, 20, 0.1, 0.3), StepReading(700, 30, 0.3, 0.5)]
    b = warmup_baseline(s)
    assert (b.peak, b.live) == (700, 30) and abs(b.t_fwd - 0.2) < 1e-12 and abs(b.t_bwd - 0.4) < 1e-12
    assert warmup_baseline(s[:1]) == s[0]


def test_tier_cost_table():
    from budgetformer_b200.control.multi_tier import tier_costs
    c = tier_costs(_cal())
    rec, keep, ret = c["recompute"], c["keep_mha"], c["retain"]
    assert abs(rec.t_fwd - 0.025) < 1e-12 and abs(rec.t_bwd - 0.075) < 1e-12
    assert abs(keep.t_bwd - (0.075 - 0.05)) < 1e-12 and abs(ret.t_bwd - 0.0) < 1e-12      # 0.075 - 0.10 clamps at 0
    assert (keep.bytes_deepest, keep.bytes_each) == (50 * MIB, 300 * MIB)
    assert (ret.bytes_deepest, ret.bytes_each) == (120 * MIB, 800 * MIB)
    # a probe slower than the baseline never makes a tier cost more than the one below it
    slow = tier_costs(_cal(keep_last=(1050, 700, 0.12, 0.35), ret_last=(1120, 1200, 0.11, 0.31)))
    assert slow["keep_mha"].t_bwd == slow["recompute"].t_bwd and slow["retain"].t_bwd <= slow["keep_mha"].t_bwd
    # the front probe counts when it is the worse one
    worse = tier_costs(_cal(keep_front=(1040, 800, 0.10, 0.27)))
    assert worse["keep_mha"].bytes_each == 400 * MIB and abs(worse["keep_mha"].t_bwd - 0.045) < 1e-12
    assert worse["keep_mha"].bytes_deepest == 50 * MIB                                     # always from the last-layer probe


def test_layout_memory_table():
    from budgetformer_b200.control.multi_tier import Layout, layout_bytes, stacked_bytes, tier_costs
    assert [stacked_bytes(n, 100) for n in range(4)] == [0, 100, 2 * 105, 3 * 110]
    c = tier_costs(_cal())
    mb = lambda lay: layout_bytes(lay, c) / MIB
    assert mb(Layout(4, 0, 0)) == 0
    assert mb(Layout(3, 1, 0)) == 50                         # only the last layer keeps its attention half
    assert mb(Layout(2, 2, 0)) == 50 + 300
    assert mb(Layout(3, 0, 1)) == 120
    assert mb(Layout(1, 0, 3)) == 120 + 2 * 800 * 1.05
    assert mb(Layout(1, 2, 1)) == 120 + 2 * 300 * 1.05       # with a retained last layer every keep_mha layer is a full one


def test_admissible_layout_table():
    from budgetformer_b200.control.multi_tier import admissible_layouts
    trip = lambda cal: sorted((l.n_recompute, l.n_keep, l.n_retain) for l in admissible_layouts(cal))
    assert len(trip(_cal(n=3))) == 10                                            # all compositions of 3 into 3 parts
    assert trip(_cal(n=2, keep_impossible=True)) == [(0, 0, 2), (1, 0, 1), (2, 0, 0)]
    assert trip(_cal(n=2, ret_impossible=True)) == [(0, 2, 0), (1, 1, 0), (2, 0, 0)]
    assert trip(_cal(n=3, keep_last_only=True)) == [(0, 0, 3), (1, 0, 2), (2, 0, 1), (2, 1, 0), (3, 0, 0)]
    assert trip(_cal(n=3, ret_last_only=True)) == [(0, 2, 1), (0, 3, 0), (1, 1, 1), (1, 2, 0), (2, 0, 1), (2, 1, 0), (3, 0, 0)]


def test_plan_search_ordering_table():
    from budgetformer_b200.control.multi_tier import EdgeCost, search_plans
    cal = _cal()
    big = 10 ** 15
    # time first: a prefetched CPU build hidden behind the model step beats a serial GPU build
    gpu = EdgeCost("gpu_ephemeral", serial_s=0.05, build_peak=500 * MIB)
    cpu = EdgeCost("cpu_rank_local_prefetch", serial_s=0.0, overlap_s=0.05, build_peak=100 * MIB, host_bytes=MIB)
    best, free, rep = search_plans(cal, [gpu, cpu], 10 ** 6 * MIB, big)
    assert best.policy == "cpu_rank_local_prefetch" and best.layout.n_retain == 4 and rep["gpu_ephemeral"][0] == "ok"
    assert abs(best.t_edge) < 1e-12 and free.policy == best.policy
    # an overlapped build longer than the model step shows its excess
    slowcpu = EdgeCost("cpu_rank_local_prefetch", overlap_s=1.0)
    best, _, _ = search_plans(cal, [slowcpu], 10 ** 6 * MIB, big)
    assert abs(best.t_edge - (1.0 - best.t_model)) < 1e-9
    # equal time: the policy without a resident topology wins; host budget and exclusions are reported
    a = EdgeCost("gpu_persist", serial_s=0.01, resident_bytes=10 * MIB)
    b = EdgeCost("gpu_ephemeral", serial_s=0.01)
    best, free, _ = search_plans(cal, [a, b], 10 ** 6 * MIB, big)
    assert best.policy == "gpu_ephemeral" and free.policy == "gpu_ephemeral"
    _, _, rep = search_plans(cal, [a, cpu], 10 ** 6 * MIB, 0, excluded=("gpu_persist",))
    assert rep == {"gpu_persist": ("skip:gpu_infeasible", None), "cpu_rank_local_prefetch": ("skip:cpu_budget", None)}
    # the build peak alone can rule a policy out; the resident topology counts against the activation layout
    tight = 1000 * MIB + 120 * MIB + 800 * MIB
    best, _, rep = search_plans(cal, [EdgeCost("gpu_ephemeral", build_peak=5000 * MIB), EdgeCost("cpu_broadcast_prefetch")],
                                tight, big)
    assert rep["gpu_ephemeral"] == ("skip:no_feasible_tier", None) and best.policy == "cpu_broadcast_prefetch"
    assert (best.layout.n_keep, best.layout.n_retain) == (2, 1)       # 120 + 2 * 300 * 1.05 MiB fits and is faster than (0, 2)
    best, _, _ = search_plans(cal, [EdgeCost("gpu_persist", resident_bytes=700 * MIB)], tight, big)
    assert (best.layout.n_keep, best.layout.n_retain) == (0, 1)       # 700 MiB of topology leave room for 220 MiB of activations
    # walks forced onto the GPU: a variant of gpu_persist with no overlap and no host memory
    p = EdgeCost("gpu_persist", serial_s=0.0, overlap_s=5.0, resident_bytes=10 * MIB, walk_gpu_extra=20 * MIB, host_bytes=MIB)
    best, _, _ = search_plans(cal, [p], 10 ** 6 * MIB, big)
    assert best.walks_on_gpu and best.t_edge == 0.0


def test_plan_search_takes_the_warmup_policys_topology_out_of_the_baseline():
    """The warm-up ran under gpu_persist, so its peak holds the resident topology: a policy without one gets that memory
    back, gpu_persist is charged it once (not twice), and under a limit between the two the CPU-offloaded build wins."""
    from dataclasses import replace
    from budgetformer_b200.control.multi_tier import EdgeCost, search_plans
    cal = replace(_cal(), resident_in_baseline=200 * MIB)            # baseline peak 1000 MiB, of which 200 MiB topology
    big = 10 ** 15
    persist = EdgeCost("gpu_persist", serial_s=0.001, resident_bytes=200 * MIB, build_peak=300 * MIB)
    cpu = EdgeCost("cpu_rank_local_prefetch", overlap_s=0.001, build_peak=100 * MIB, host_bytes=MIB)
    # 950 MiB: the model alone (800) fits, the model with the topology (1000) does not
    best, _, rep = search_plans(cal, [persist, cpu], 950 * MIB, big)
    assert rep["gpu_persist"] == ("skip:no_feasible_tier", None) and best.policy == "cpu_rank_local_prefetch"
    assert best.peak <= 950 * MIB and best.layout.n_keep + best.layout.n_retain >= 1      # 150 MiB left for activations
    # 1000 MiB: gpu_persist fits exactly as measured (800 + 200), with every layer recomputed
    best, _, rep = search_plans(cal, [persist], 1000 * MIB, big)
    assert rep["gpu_persist"][0] == "ok" and best.peak == 1000 * MIB and best.layout.n_recompute == 4
    # without the correction the same limit would have ruled it out (1000 + 200)
    best, _, rep = search_plans(_cal(), [persist], 1000 * MIB, big)
    assert best is None and rep["gpu_persist"] == ("skip:no_feasible_tier", None)


def test_planner_falls_back_inside_the_policies_left_in_the_search():
    planner = ExecutionPlanner(2, probe=ScriptedMemoryProbe(1000 * MIB, lambda modes: {"peak": 990 * MIB, "live": 10 * MIB}),
                               verbose=False)
    planner.set_edge_policy_profile(EDGE_GPU_PERSIST, 0.01, 100 * MIB, 0, live_edge_bytes=50 * MIB)
    planner.set_edge_policy_profile(EDGE_CPU_RANK_LOCAL_PREFETCH, 0.2, 10 * MIB, MIB, serial_time_s=0.0, overlap_time_s=0.2)
    planner.active_edge_policy_fn = lambda: EDGE_GPU_PERSIST
    dev = "cpu"
    for _ in range(8):
        if planner.is_active():
            break
        planner.plan(dev)
        planner.record_post_forward_memory(dev)
        planner.notify_step_end(dev, t_bwd=0.02, t_fwd=0.01)
    assert planner.is_active() and planner.calibration.resident_in_baseline == 50 * MIB
    planner.report_runtime_edge_gpu_infeasible(dev)                  # nothing fits 900 MiB: the fallback must not name a GPU policy
    assert planner.edge_policy == EDGE_CPU_RANK_LOCAL_PREFETCH and planner.modes() == ["recompute", "recompute"]


def test_demotion_table():
    from budgetformer_b200.control.multi_tier import demoted
    assert demoted(["retain", "retain"]) == ["keep_mha", "retain"]
    assert demoted(["recompute", "keep_mha", "retain"]) == ["recompute", "recompute", "retain"]
    assert demoted(["recompute", "recompute"]) is None
