"""Adaptive Budget Selection: online greedy split of the per-query edge budget between real
in-edges (``b_r``) and random-walk edges (``b_w``).

``AdaptiveEdgeBudgetController`` restates ``_AdaptiveEdgeBudgetController``
(utils/fullgraph_sp_support.py:1942-2178): start at ``(2, min(2, W*L))``; offer ``real_up`` / ``rw_up``
below the ceiling and ``shift_to_real`` / ``shift_to_rw`` at it; the n-th committed move needs
``min(n, 3)`` consecutive wins of the same kind; ``patience`` rounds without a positive gain freeze
the budget; a linear peak-memory extrapolation gates growth.  ``decide_budget_move`` restates the
decision half of ``_maybe_update_edge_budget`` (:2772-2928) as a pure function of the probe table,
so it can be unit-tested without a model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

LOSS_BAND = 0.01


@dataclass
class AdaptiveEdgeBudgetConfig:
    enabled: bool = False
    max_total_edges_per_query: int = 0
    block_size: int = 2
    warmup_epochs: Optional[int] = None      # None = no cap
    patience: int = 3
    probe_size: int = 0
    static_seed_epochs: int = 0
    rw_max_per_query: int = 0                # W * L
    gpu_limit_mib: float = 0.0
    gpu_safety_margin: float = 0.1


def resolve_adaptive_edge_budget_config(args) -> AdaptiveEdgeBudgetConfig:
    """Flag -> config resolution (utils/fullgraph_sp_support.py:918-967)."""
    enabled = bool(getattr(args, "adaptive_edge_budget", False))
    block = int(getattr(args, "adaptive_edge_budget_block_size", 0) or 0)
    patience = int(getattr(args, "adaptive_edge_budget_patience", 0) or 0)
    warm = int(getattr(args, "adaptive_edge_budget_warmup_epochs", -1))
    wl = int(getattr(args, "fixed_walk_length", None) or getattr(args, "walk_length", 0) or 0)
    return AdaptiveEdgeBudgetConfig(
        enabled=enabled,
        max_total_edges_per_query=max(0, int(getattr(args, "max_total_edges_per_query", 0) or 0)),
        block_size=block if block > 0 else 2,
        warmup_epochs=None if warm < 0 else warm,
        patience=max(3, patience) if patience > 0 else 3,
        probe_size=int(getattr(args, "adaptive_edge_budget_probe_size", 0) or 0),
        static_seed_epochs=int(getattr(args, "adaptive_edge_budget_static_seed_epochs", 0) or 0),
        rw_max_per_query=max(0, int(getattr(args, "walks_per_node", 0)) * wl),
        gpu_limit_mib=float(getattr(args, "multi_tier_gpu_memory_limit_mib", 0) or 0),
        gpu_safety_margin=0.1,
    )


class AdaptiveEdgeBudgetController:
    def __init__(self, config: AdaptiveEdgeBudgetConfig) -> None:
        self.enabled = bool(config.enabled)
        self.block_size = int(config.block_size)
        self.max_total = int(config.max_total_edges_per_query)
        self.warmup_epochs = config.warmup_epochs
        self.patience = int(config.patience)
        self.bad_rounds = 0
        self.seen_positive_gain = False
        self._gpu_limit_mib = float(config.gpu_limit_mib or 0.0)
        self._gpu_safety_margin = float(config.gpu_safety_margin or 0.0)
        self._peak_hist: List[tuple] = []
        self._over_budget = False
        self.auto_hold_released = False
        self.auto_hold_neg_inf_streak = 0
        self.auto_hold_neg_inf_freeze_after = 5
        self.baseline_acc = -1.0
        self.walk_length: Optional[int] = None
        self._n_budget_updates = 0
        self._max_confirm_rounds = 3
        self._pending_kind: Optional[str] = None
        self._pending_state: Optional[dict] = None
        self._pending_wins = 0
        self.frozen = not self.enabled
        pl = int(config.rw_max_per_query or 0)
        self.rw_max = min(self.max_total, pl) if pl > 0 else self.max_total
        if not self.enabled:
            self.real_budget, self.rw_budget = self.max_total, 0
            return
        self.real_budget = 2 if self.max_total > 0 else 0
        self.rw_budget = min(2, self.rw_max) if self.max_total > 0 else 0

    # -- state ----------------------------------------------------------------------------
    def current_state(self) -> dict:
        s = {"real_edges_per_query": int(self.real_budget), "rw_edges_per_query": int(self.rw_budget)}
        if self.walk_length is not None:
            s["walk_length"] = int(self.walk_length)
        return s

    def set_state(self, state) -> None:
        if state is None:
            return
        self.real_budget = int(state.get("real_edges_per_query", self.real_budget))
        self.rw_budget = int(state.get("rw_edges_per_query", self.rw_budget))
        if "walk_length" in state:
            self.walk_length = int(state["walk_length"])

    def state_dict(self) -> dict:
        keys = ("real_budget", "rw_budget", "walk_length", "frozen", "bad_rounds", "seen_positive_gain",
                "_n_budget_updates", "_pending_kind", "_pending_state", "_pending_wins", "_peak_hist",
                "auto_hold_released", "auto_hold_neg_inf_streak", "baseline_acc", "_over_budget")
        return {k: getattr(self, k) for k in keys}

    def load_state_dict(self, sd: dict) -> None:
        for k, v in sd.items():
            setattr(self, k, v)

    def _mk(self, real: int, rw: int) -> dict:
        s = {"real_edges_per_query": int(real), "rw_edges_per_query": int(rw)}
        if self.walk_length is not None:
            s["walk_length"] = int(self.walk_length)
        return s

    def candidate_states(self) -> Dict[str, dict]:
        out: Dict[str, dict] = {}
        rw_can_grow = self.rw_budget + self.block_size <= self.rw_max
        if self.real_budget + self.rw_budget + self.block_size <= self.max_total:
            out["real_up"] = self._mk(self.real_budget + self.block_size, self.rw_budget)
            if rw_can_grow:
                out["rw_up"] = self._mk(self.real_budget, self.rw_budget + self.block_size)
        if self.real_budget + self.rw_budget >= self.max_total:
            if self.rw_budget >= self.block_size:
                out["shift_to_real"] = self._mk(self.real_budget + self.block_size, self.rw_budget - self.block_size)
            if self.real_budget >= self.block_size and rw_can_grow:
                out["shift_to_rw"] = self._mk(self.real_budget - self.block_size, self.rw_budget + self.block_size)
        return {k: v for k, v in out.items() if self._growth_fits(v)}

    # -- memory gate ------------------------------------------------------------------------
    def observe_peak(self, peak_mib) -> None:
        if (not self.enabled) or self.frozen or self._gpu_limit_mib <= 0 or not peak_mib or peak_mib <= 0:
            return
        self._over_budget = peak_mib > self._gpu_limit_mib * (1.0 - self._gpu_safety_margin)
        total = int(self.real_budget + self.rw_budget)
        for i, (b, p) in enumerate(self._peak_hist):
            if b == total:
                if peak_mib > p:
                    self._peak_hist[i] = (total, float(peak_mib))
                return
        self._peak_hist.append((total, float(peak_mib)))

    def _predict_peak(self, target_total: int):
        pts = sorted(self._peak_hist)
        if len(pts) < 2:
            return None
        b_hi, p_hi = pts[-1]
        if target_total <= b_hi:
            return p_hi
        slope = 0.0
        for (b0, p0), (b1, p1) in zip(pts, pts[1:]):
            if b1 > b0:
                slope = max(slope, (p1 - p0) / (b1 - b0))
        return p_hi + slope * (target_total - b_hi)

    def _growth_fits(self, cand) -> bool:
        if self._gpu_limit_mib <= 0:
            return True
        total = int(cand.get("real_edges_per_query", 0) + cand.get("rw_edges_per_query", 0))
        if total <= int(self.real_budget + self.rw_budget):
            return True
        pred = self._predict_peak(total)
        return True if pred is None else pred <= self._gpu_limit_mib * (1.0 - self._gpu_safety_margin)

    def force_shrink(self):
        self._over_budget = False
        if self.real_budget + self.rw_budget <= 0:
            return None
        if self.rw_budget >= self.real_budget:
            if self.rw_budget >= self.block_size:
                self.rw_budget -= self.block_size
            else:
                self.real_budget = max(0, self.real_budget - self.block_size)
        else:
            if self.real_budget >= self.block_size:
                self.real_budget -= self.block_size
            else:
                self.rw_budget = max(0, self.rw_budget - self.block_size)
        self._pending_kind, self._pending_state, self._pending_wins = None, None, 0
        return self.current_state()

    # -- commit logic -----------------------------------------------------------------------
    def required_confirm_rounds(self) -> int:
        return min(self._n_budget_updates + 1, self._max_confirm_rounds)

    def update(self, choice, best_gain, next_state=None) -> None:
        if best_gain > 0.0:
            self.seen_positive_gain = True
        if next_state is not None and choice is not None:
            if choice == self._pending_kind:
                self._pending_wins += 1
            else:
                self._pending_kind, self._pending_state, self._pending_wins = choice, next_state, 1
            if self._pending_wins >= self.required_confirm_rounds():
                self.set_state(self._pending_state)
                self._n_budget_updates += 1
                self._pending_kind, self._pending_state, self._pending_wins = None, None, 0
                self.bad_rounds = 0
            return
        self._pending_kind, self._pending_state, self._pending_wins = None, None, 0
        if best_gain <= 0.0:
            self.bad_rounds += 1
            if self.bad_rounds >= self.patience:
                self.frozen = True


def fixed_budget_controller(real: int, rw: int, walk_length: Optional[int] = None) -> AdaptiveEdgeBudgetController:
    """Frozen controller carrying a manual split (``--fixed_real_edges_per_query`` /
    ``--fixed_rw_edges_per_query``; main_node_fullgraph_sp.py:265-270)."""
    c = AdaptiveEdgeBudgetController(AdaptiveEdgeBudgetConfig(enabled=False, max_total_edges_per_query=real + rw))
    c.real_budget, c.rw_budget, c.walk_length, c.frozen = int(real), int(rw), walk_length, True
    return c


def round_budget_to_block(value: int, block_size: int) -> int:
    """``value`` rounded up to a multiple of the block (at least one block; 0 stays 0)."""
    b = max(1, int(block_size))
    return 0 if value <= 0 else max(b, -(-int(value) // b) * b)


def floor_budget_to_block(value: int, block_size: int) -> int:
    """``value`` rounded down to a multiple of the block (at least one block; 0 stays 0)."""
    b = max(1, int(block_size))
    return 0 if value <= 0 else max(b, (int(value) // b) * b)


def auto_initial_budget_candidates(config: AdaptiveEdgeBudgetConfig) -> List[dict]:
    """Start points for a budget search (utils/fullgraph_sp_support.py:2194-2235): (real, rw) pairs on block
    multiples - 1, 2 and 4 blocks of real edges with none, as many or twice as many walk edges - that fit under the
    ceiling, ordered by total and then by walk share."""
    ceiling, b = int(config.max_total_edges_per_query), max(1, int(config.block_size))
    if ceiling <= 0:
        return []
    grid = [(1, 0), (1, 1), (1, 2), (2, 0), (2, 1), (2, 2), (4, 0), (4, 2)]
    pairs = sorted({(r * b, w * b) for r, w in grid if (r + w) * b <= ceiling}, key=lambda p: (p[0] + p[1], p[1]))
    if not pairs:
        pairs = [(min(ceiling, b), 0)]
    return [{"real_edges_per_query": r, "rw_edges_per_query": w} for r, w in pairs]


def _pair(state) -> tuple:
    return int(state.get("real_edges_per_query", 0)), int(state.get("rw_edges_per_query", 0))


def decide_budget_move(controller: AdaptiveEdgeBudgetController, probe_rows: List[dict], epoch: int = 0,
                       log: Optional[Callable[[str], None]] = None) -> str:
    """Apply one probe round.  ``probe_rows``: ``{"kind", "state", "loss", "acc", "edges"}`` with the
    current state first (``kind == "current"``).  Fills in ``gain = (base - loss) / base`` and calls
    ``controller.update``.  Returns a tag describing the branch taken."""
    log = log or (lambda _m: None)
    base = probe_rows[0]
    base_loss = float(base["loss"])
    for r in probe_rows:
        if r["kind"] == "current":
            r["gain"] = 0.0
        elif not (r["loss"] == r["loss"]) or r["loss"] == float("inf"):
            r["gain"] = float("-inf")
        else:
            r["gain"] = (base_loss - float(r["loss"])) / base_loss if base_loss != 0 else 0.0
    cands = [r for r in probe_rows if r["kind"] != "current"]
    if cands:
        best = max(cands, key=lambda r: r["gain"])
        best_kind, best_gain, best_state = best["kind"], best["gain"], best["state"]
    else:
        best_kind, best_gain, best_state = None, float("-inf"), None
    at_ceiling = controller.real_budget + controller.rw_budget >= controller.max_total
    if at_ceiling and cands and all(abs(r["gain"]) < LOSS_BAND for r in cands):
        acc_win = max(cands, key=lambda r: r["acc"])
        if acc_win["kind"] != best_kind:
            log(f"  ↳ BudgetCtrl acc-driven epoch={epoch}: all |gain|<{LOSS_BAND:.0%}; acc picks {acc_win['kind']}")
            best_kind, best_gain, best_state = acc_win["kind"], acc_win["gain"], acc_win["state"]
    commit_ok = best_gain > 0.0
    cur = _pair(base["state"])
    log(f"  ↳ BudgetCtrl probe epoch={epoch} current=({cur[0]},{cur[1]})")
    for r in probe_rows:
        rb, wb = _pair(r["state"])
        gain_text = "base" if r["kind"] == "current" else f"{r['gain']:.8e}"
        log(f"     - {r['kind']:<13} budget=({rb},{wb}) loss={r['loss']:.6f} acc={r['acc']:.6f} "
            f"gain={gain_text} probe_edges={r['edges']}")

    def _tag():
        return (f" [confirm {controller._pending_wins}/{controller.required_confirm_rounds()}]"
                if controller._pending_wins > 0 else "")

    if not at_ceiling:
        base_total = sum(cur)
        growth = [r for r in cands if sum(_pair(r["state"])) > base_total]
        if growth:
            win = max(growth, key=lambda r: r["gain"])
            if win["gain"] > 0.0:
                controller.auto_hold_released = True
                controller.auto_hold_neg_inf_streak = 0
            controller.update(win["kind"], win["gain"], win["state"])
            nb = controller.current_state()
            log(f"  ↳ BudgetCtrl grow-below-ceiling epoch={epoch}: move={win['kind']}{_tag()} "
                f"rel_gain={win['gain']:.8e} new_budget=({nb['real_edges_per_query']},{nb['rw_edges_per_query']})")
            return "grow"
    if not controller.auto_hold_released:
        controller.auto_hold_neg_inf_streak = controller.auto_hold_neg_inf_streak + 1 if best_gain == float("-inf") else 0
        if controller.auto_hold_neg_inf_streak >= controller.auto_hold_neg_inf_freeze_after:
            controller.frozen = True
            log(f"  ↳ BudgetCtrl [AutoHoldFrozen] epoch={epoch}; freezing budget.")
            return "auto_hold_frozen"
        if commit_ok:
            controller.auto_hold_released = True
            controller.auto_hold_neg_inf_streak = 0
        else:
            controller.update(None, best_gain, None)
            log(f"  ↳ BudgetCtrl [AutoHold] epoch={epoch} STAY best_rel_gain_found={best_gain:.8e} "
                f"bad_rounds={controller.bad_rounds}/{controller.patience}"
                f"{' freezing budget.' if controller.frozen else ''}")
            return "auto_hold"
    controller.update(best_kind if commit_ok else None, best_gain, best_state if commit_ok else None)
    nb = controller.current_state()
    log(f"  ↳ BudgetCtrl update epoch={epoch} move={best_kind if commit_ok else 'STAY'}{_tag()} "
        f"rel_gain={best_gain:.8e} new_budget=({nb['real_edges_per_query']},{nb['rw_edges_per_query']})")
    return "update"
