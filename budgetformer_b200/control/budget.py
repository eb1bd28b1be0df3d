"""Adaptive Budget Selection: an online greedy search for the split of the per-query edge budget between
real in-edges and random-walk edges.

Behaviour (what ``_AdaptiveEdgeBudgetController`` and the decision half of ``_maybe_update_edge_budget`` do,
utils/fullgraph_sp_support.py:1942-2178 and :2772-2928), restated here as data + pure functions:

* the search is a value, ``SearchState`` (frozen dataclass); every event - a probe round, a memory reading, a
  forced shrink - is a function ``(state, limits, observation) -> state``.  ``BudgetSearch`` is the thin mutable
  holder the trainer talks to; it only swaps the value;
* start at ``(2, min(2, W*L))``; below the ceiling the offers are ``real_up`` / ``rw_up``, at the ceiling
  ``shift_to_real`` / ``shift_to_rw``; the walk side never exceeds ``W*L`` (more cannot be realised per query);
* the n-th committed move needs ``min(n, 3)`` consecutive rounds won by the same kind of move; a round whose best
  gain is not positive counts towards ``patience``, which freezes the search;
* growth offers pass a memory gate: a straight line through the observed (total budget, peak MiB) points with
  the steepest slope seen must stay under ``limit * (1 - margin)``;
* until the first positive gain the search is "held": five rounds in a row in which every candidate failed
  (gain = -inf) freeze it.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Callable, Dict, List, Optional, Tuple

LOSS_BAND = 0.01            # at the ceiling, gains inside this band are a tie that accuracy breaks
CONFIRM_CAP = 3             # no move ever needs more consecutive wins than this
BLANK_ROUNDS_TO_FREEZE = 5  # all-candidates-failed rounds in a row, before any gain was ever seen

GROW_KINDS = ("real_up", "rw_up")
SHIFT_KINDS = ("shift_to_real", "shift_to_rw")


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
    """Flags -> configuration (utils/fullgraph_sp_support.py:918-967): block 2 unless given, patience at least 3,
    no warm-up cap unless given, walk ceiling ``walks_per_node * walk_length``."""
    def flag(name, default=0):
        v = getattr(args, name, default)
        return default if v is None else v

    block, patience = int(flag("adaptive_edge_budget_block_size")), int(flag("adaptive_edge_budget_patience"))
    warm = int(flag("adaptive_edge_budget_warmup_epochs", -1))
    walk_len = int(getattr(args, "fixed_walk_length", None) or flag("walk_length"))
    return AdaptiveEdgeBudgetConfig(
        enabled=bool(flag("adaptive_edge_budget", False)),
        max_total_edges_per_query=max(0, int(flag("max_total_edges_per_query"))),
        block_size=block if block > 0 else 2,
        warmup_epochs=warm if warm >= 0 else None,
        patience=max(3, patience),
        probe_size=int(flag("adaptive_edge_budget_probe_size")),
        static_seed_epochs=int(flag("adaptive_edge_budget_static_seed_epochs")),
        rw_max_per_query=max(0, int(flag("walks_per_node")) * walk_len),
        gpu_limit_mib=float(flag("multi_tier_gpu_memory_limit_mib")),
    )


# ---------------------------------------------------------------------------------------------------------
# values
# ---------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Split:
    """One point of the search space."""
    real: int
    walk: int
    walk_length: Optional[int] = None

    @property
    def total(self) -> int:
        return self.real + self.walk

    def as_dict(self) -> dict:
        d = {"real_edges_per_query": int(self.real), "rw_edges_per_query": int(self.walk)}
        if self.walk_length is not None:
            d["walk_length"] = int(self.walk_length)
        return d

    @staticmethod
    def from_dict(d: dict, like: Optional["Split"] = None) -> "Split":
        base = like or Split(0, 0)
        wl = d.get("walk_length", base.walk_length)
        return Split(int(d.get("real_edges_per_query", base.real)), int(d.get("rw_edges_per_query", base.walk)),
                     None if wl is None else int(wl))


@dataclass(frozen=True)
class Limits:
    """What bounds the search; fixed for a run."""
    ceiling: int                 # B: real + walk never exceeds it
    step: int                    # moves change a side by this many edges
    walk_cap: int                # W * L (or the ceiling when unknown)
    patience: int
    hbm_limit_mib: float = 0.0   # 0 = no memory gate
    hbm_margin: float = 0.1

    @property
    def hbm_ceiling_mib(self) -> float:
        return self.hbm_limit_mib * (1.0 - self.hbm_margin)

    @staticmethod
    def from_config(cfg: AdaptiveEdgeBudgetConfig) -> "Limits":
        ceiling = int(cfg.max_total_edges_per_query)
        realisable = int(cfg.rw_max_per_query or 0)
        return Limits(ceiling=ceiling, step=int(cfg.block_size), walk_cap=min(ceiling, realisable) if realisable > 0 else ceiling,
                      patience=int(cfg.patience), hbm_limit_mib=float(cfg.gpu_limit_mib or 0.0),
                      hbm_margin=float(cfg.gpu_safety_margin or 0.0))


@dataclass(frozen=True)
class SearchState:
    split: Split
    frozen: bool
    commits: int = 0                               # moves applied so far
    streak_kind: Optional[str] = None              # move kind that won the most recent round(s) ...
    streak_target: Optional[Split] = None          # ... the split it proposed when the streak began ...
    streak_len: int = 0                            # ... and for how many rounds in a row
    dry_rounds: int = 0                            # rounds without a positive gain since the last commit
    improved_once: bool = False
    hold_open: bool = False                        # a positive gain has been seen: the initial hold is over
    blank_rounds: int = 0                          # consecutive all-failed rounds while held
    peaks: Tuple[Tuple[int, float], ...] = ()      # (total budget, highest peak MiB seen at it)
    over_limit: bool = False                       # the last reading was above the memory ceiling
    reference_acc: float = -1.0


def initial_state(limits: Limits, enabled: bool) -> SearchState:
    if not enabled:
        return SearchState(Split(limits.ceiling, 0), frozen=True)
    if limits.ceiling <= 0:
        return SearchState(Split(0, 0), frozen=False)
    return SearchState(Split(2, min(2, limits.walk_cap)), frozen=False)


# ---------------------------------------------------------------------------------------------------------
# memory gate
# ---------------------------------------------------------------------------------------------------------
def projected_peak_mib(peaks, total: int) -> Optional[float]:
    """Peak expected at ``total`` edges per query: the highest-budget reading, extended with the steepest slope
    between neighbouring readings.  ``None`` with fewer than two readings (nothing to extrapolate from)."""
    pts = sorted(peaks)
    if len(pts) < 2:
        return None
    top_budget, top_peak = pts[-1]
    if total <= top_budget:
        return top_peak
    slopes = [(p1 - p0) / (b1 - b0) for (b0, p0), (b1, p1) in zip(pts, pts[1:]) if b1 > b0]
    return top_peak + max([0.0] + slopes) * (total - top_budget)


def fits_memory(state: SearchState, limits: Limits, target: Split) -> bool:
    if limits.hbm_limit_mib <= 0 or target.total <= state.split.total:
        return True
    expected = projected_peak_mib(state.peaks, target.total)
    return expected is None or expected <= limits.hbm_ceiling_mib


def with_peak(state: SearchState, limits: Limits, peak_mib: Optional[float]) -> SearchState:
    """A peak-memory reading taken while training at ``state.split``."""
    if state.frozen or limits.hbm_limit_mib <= 0 or not peak_mib or peak_mib <= 0:
        return state
    seen = dict(state.peaks)
    seen[state.split.total] = max(float(peak_mib), seen.get(state.split.total, 0.0))
    return replace(state, peaks=tuple(sorted(seen.items())), over_limit=peak_mib > limits.hbm_ceiling_mib)


def shrunk(state: SearchState, limits: Limits) -> SearchState:
    """One step down after a reading above the ceiling: the larger side gives (walk on a tie), the other one if the
    larger side has less than a step left.  Any confirmation streak is void."""
    s, step = state.split, limits.step
    cleared = replace(state, over_limit=False)
    if s.total <= 0:
        return cleared
    first, second = ("walk", "real") if s.walk >= s.real else ("real", "walk")
    side = first if getattr(s, first) >= step else second
    new_split = replace(s, **{side: max(0, getattr(s, side) - step)})
    return replace(cleared, split=new_split, streak_kind=None, streak_target=None, streak_len=0)


# ---------------------------------------------------------------------------------------------------------
# offers and transitions
# ---------------------------------------------------------------------------------------------------------
def offers(state: SearchState, limits: Limits) -> Dict[str, Split]:
    """Moves open from ``state.split`` (insertion order = probe order)."""
    s, step = state.split, limits.step
    walk_room = s.walk + step <= limits.walk_cap
    table: List[Tuple[str, bool, Split]] = [
        ("real_up", s.total + step <= limits.ceiling, replace(s, real=s.real + step)),
        ("rw_up", s.total + step <= limits.ceiling and walk_room, replace(s, walk=s.walk + step)),
        ("shift_to_real", s.total >= limits.ceiling and s.walk >= step, replace(s, real=s.real + step, walk=s.walk - step)),
        ("shift_to_rw", s.total >= limits.ceiling and s.real >= step and walk_room,
         replace(s, real=s.real - step, walk=s.walk + step)),
    ]
    return {kind: target for kind, open_, target in table if open_ and fits_memory(state, limits, target)}


def wins_needed(state: SearchState) -> int:
    return min(state.commits + 1, CONFIRM_CAP)


def after_round(state: SearchState, limits: Limits, kind: Optional[str], gain: float,
                target: Optional[Split]) -> SearchState:
    """Outcome of one probe round.  ``kind``/``target`` name the winning move, or are ``None`` for "stay"."""
    state = replace(state, improved_once=state.improved_once or gain > 0.0)
    if kind is None or target is None:
        dry = state.dry_rounds + (1 if gain <= 0.0 else 0)
        return replace(state, streak_kind=None, streak_target=None, streak_len=0, dry_rounds=dry,
                       frozen=state.frozen or (gain <= 0.0 and dry >= limits.patience))
    if kind == state.streak_kind:
        state = replace(state, streak_len=state.streak_len + 1)
    else:
        state = replace(state, streak_kind=kind, streak_target=target, streak_len=1)
    if state.streak_len < wins_needed(state):
        return state
    return replace(state, split=state.streak_target, commits=state.commits + 1, dry_rounds=0,
                   streak_kind=None, streak_target=None, streak_len=0)


@dataclass
class RoundOutcome:
    tag: str                      # "grow" | "auto_hold" | "auto_hold_frozen" | "update"
    state: SearchState
    lines: List[str] = field(default_factory=list)


def _gain(base_loss: float, loss: float) -> float:
    if loss != loss or loss == float("inf"):
        return float("-inf")
    return (base_loss - loss) / base_loss if base_loss != 0 else 0.0


def judge_round(state: SearchState, limits: Limits, rows: List[dict], epoch: int = 0) -> RoundOutcome:
    """One probe table -> next state.  ``rows``: dicts with ``kind, state, loss, acc, edges``; the first row is the
    current split (``kind == "current"``).  Adds ``gain`` to every row."""
    base_loss = float(rows[0]["loss"])
    for r in rows:
        r["gain"] = 0.0 if r["kind"] == "current" else _gain(base_loss, float(r["loss"]))
    cands = rows[1:]
    lines = [f"  ↳ BudgetCtrl probe epoch={epoch} current=({state.split.real},{state.split.walk})"]
    for r in rows:
        sp = Split.from_dict(r["state"])
        shown = "base" if r["kind"] == "current" else f"{r['gain']:.8e}"
        lines.append(f"     - {r['kind']:<13} budget=({sp.real},{sp.walk}) loss={r['loss']:.6f} acc={r['acc']:.6f} "
                     f"gain={shown} probe_edges={r['edges']}")

    def target_of(row) -> Split:
        return Split.from_dict(row["state"], like=state.split)

    def confirm_note(st: SearchState) -> str:
        return f" [confirm {st.streak_len}/{wins_needed(st)}]" if st.streak_len > 0 else ""

    def budget_note(st: SearchState) -> str:
        return f"new_budget=({st.split.real},{st.split.walk})"

    at_ceiling = state.split.total >= limits.ceiling
    # ---- below the ceiling: the best *growing* row drives the round, whatever its sign -------------------
    if not at_ceiling:
        growing = [r for r in cands if target_of(r).total > state.split.total]
        if growing:
            top = max(growing, key=lambda r: r["gain"])
            if top["gain"] > 0.0:
                state = replace(state, hold_open=True, blank_rounds=0)
            state = after_round(state, limits, top["kind"], top["gain"], target_of(top))
            lines.append(f"  ↳ BudgetCtrl grow-below-ceiling epoch={epoch}: move={top['kind']}{confirm_note(state)} "
                         f"rel_gain={top['gain']:.8e} {budget_note(state)}")
            return RoundOutcome("grow", state, lines)
    # ---- overall winner; inside the loss band at the ceiling, accuracy decides -----------------------------
    winner = max(cands, key=lambda r: r["gain"]) if cands else None
    if at_ceiling and cands and all(abs(r["gain"]) < LOSS_BAND for r in cands):
        by_acc = max(cands, key=lambda r: r["acc"])
        if by_acc["kind"] != winner["kind"]:
            lines.insert(0, f"  ↳ BudgetCtrl acc-driven epoch={epoch}: all |gain|<{LOSS_BAND:.0%}; acc picks {by_acc['kind']}")
            winner = by_acc
    top_gain = winner["gain"] if winner is not None else float("-inf")
    positive = top_gain > 0.0
    # ---- initial hold ---------------------------------------------------------------------------------------
    if not state.hold_open:
        blanks = state.blank_rounds + 1 if top_gain == float("-inf") else 0
        state = replace(state, blank_rounds=blanks)
        if blanks >= BLANK_ROUNDS_TO_FREEZE:
            lines.append(f"  ↳ BudgetCtrl [AutoHoldFrozen] epoch={epoch}; freezing budget.")
            return RoundOutcome("auto_hold_frozen", replace(state, frozen=True), lines)
        if positive:
            state = replace(state, hold_open=True, blank_rounds=0)
        else:
            state = after_round(state, limits, None, top_gain, None)
            lines.append(f"  ↳ BudgetCtrl [AutoHold] epoch={epoch} STAY best_rel_gain_found={top_gain:.8e} "
                         f"bad_rounds={state.dry_rounds}/{limits.patience}{' freezing budget.' if state.frozen else ''}")
            return RoundOutcome("auto_hold", state, lines)
    # ---- ordinary round --------------------------------------------------------------------------------------
    if positive:
        state = after_round(state, limits, winner["kind"], top_gain, target_of(winner))
    else:
        state = after_round(state, limits, None, top_gain, None)
    lines.append(f"  ↳ BudgetCtrl update epoch={epoch} move={winner['kind'] if positive else 'STAY'}{confirm_note(state)} "
                 f"rel_gain={top_gain:.8e} {budget_note(state)}")
    return RoundOutcome("update", state, lines)


# ---------------------------------------------------------------------------------------------------------
# the holder the trainer uses
# ---------------------------------------------------------------------------------------------------------
class BudgetSearch:
    """Mutable handle on a ``SearchState``; every method swaps the value for the one the pure function returns."""

    def __init__(self, config: AdaptiveEdgeBudgetConfig) -> None:
        self.enabled = bool(config.enabled)
        self.warmup_epochs = config.warmup_epochs
        self.limits = Limits.from_config(config)
        self.state = initial_state(self.limits, self.enabled)

    # read-only views
    @property
    def frozen(self) -> bool:
        return self.state.frozen

    @frozen.setter
    def frozen(self, value: bool) -> None:
        self.state = replace(self.state, frozen=bool(value))

    @property
    def split(self) -> Split:
        return self.state.split

    @property
    def real_budget(self) -> int:
        return self.state.split.real

    @property
    def rw_budget(self) -> int:
        return self.state.split.walk

    @property
    def max_total(self) -> int:
        return self.limits.ceiling

    @property
    def patience(self) -> int:
        return self.limits.patience

    @property
    def over_limit(self) -> bool:
        return self.state.over_limit

    def current_state(self) -> dict:
        return self.state.split.as_dict()

    def candidate_states(self) -> Dict[str, dict]:
        return {k: s.as_dict() for k, s in offers(self.state, self.limits).items()}

    def required_confirm_rounds(self) -> int:
        return wins_needed(self.state)

    # events
    def set_split(self, real: int, walk: int, walk_length: Optional[int] = None) -> None:
        wl = self.state.split.walk_length if walk_length is None else walk_length
        self.state = replace(self.state, split=Split(int(real), int(walk), wl))

    def update(self, choice: Optional[str], best_gain: float, next_state: Optional[dict] = None) -> None:
        target = None if next_state is None else Split.from_dict(next_state, like=self.state.split)
        self.state = after_round(self.state, self.limits, choice, float(best_gain), target)

    def observe_peak(self, peak_mib) -> None:
        if self.enabled:
            self.state = with_peak(self.state, self.limits, peak_mib)

    def force_shrink(self) -> Optional[dict]:
        had_budget = self.state.split.total > 0
        self.state = shrunk(self.state, self.limits)
        return self.current_state() if had_budget else None

    def apply_round(self, rows: List[dict], epoch: int = 0) -> RoundOutcome:
        out = judge_round(self.state, self.limits, rows, epoch)
        self.state = out.state
        return out

    # persistence (sidecar training state)
    def state_dict(self) -> dict:
        d = asdict(self.state)
        d["peaks"] = [list(p) for p in self.state.peaks]
        return d

    def load_state_dict(self, sd: dict) -> None:
        sd = dict(sd)
        split = sd.pop("split")
        target = sd.pop("streak_target", None)
        peaks = tuple((int(b), float(p)) for b, p in sd.pop("peaks", ()))
        self.state = SearchState(split=Split(**split), streak_target=None if target is None else Split(**target),
                                 peaks=peaks, **sd)


def fixed_budget_controller(real: int, rw: int, walk_length: Optional[int] = None) -> BudgetSearch:
    """A frozen search carrying a manual split (``--fixed_real_edges_per_query`` / ``--fixed_rw_edges_per_query``;
    main_node_fullgraph_sp.py:265-270)."""
    c = BudgetSearch(AdaptiveEdgeBudgetConfig(enabled=False, max_total_edges_per_query=int(real) + int(rw)))
    c.set_split(real, rw, walk_length)
    c.state = replace(c.state, split=Split(int(real), int(rw), walk_length), frozen=True)
    return c


def decide_budget_move(controller: BudgetSearch, probe_rows: List[dict], epoch: int = 0,
                       log: Optional[Callable[[str], None]] = None) -> str:
    """Feed one probe table to the search and log what it decided; returns the branch tag."""
    out = controller.apply_round(probe_rows, epoch)
    if log is not None:
        for line in out.lines:
            log(line)
    return out.tag


# ---------------------------------------------------------------------------------------------------------
# block arithmetic and start points
# ---------------------------------------------------------------------------------------------------------
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
    return [Split(r, w).as_dict() for r, w in pairs]
