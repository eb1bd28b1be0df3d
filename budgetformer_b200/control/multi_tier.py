"""Multi-Tier Execution Planner: profile -> plan -> execute under an HBM cap.

Jointly chooses (a) where the per-epoch attention graph is built (``gpu_persist`` | ``gpu_ephemeral`` |
``cpu_rank_local_prefetch`` | ``cpu_broadcast_prefetch``) and (b) a per-layer activation layout
``[recompute]*a + [keep_mha]*b + [retain]*c``.  It behaves like the reference's planner
(gt_sp/multi_tier.py:60-1562): phases DEFERRED -> WARMUP_RECOMPUTE -> CALIBRATE_MHA [-> MHA_FRONT] ->
CALIBRATE_RETAIN [-> RETAIN_FRONT] -> ACTIVE, one probed layer per calibration step, then a search over
(policy, layout) for the fastest estimated step that fits.

Structure.  Measurements are immutable records (``StepReading``, ``TierProbe``, ``Calibration``, ``EdgeCost``);
the phase order is a table (``_PHASE_PROBE``) read by ``advance``; the cost model is a set of pure functions
(``tier_costs``, ``layout_bytes``, ``layout_times``, ``search_plans``) that take those records as data, so the
decision tables can be tested without a device.  ``ExecutionPlanner`` is the object the model and the trainer
talk to: it reads memory through a ``MemoryProbe`` (which adds peer-mapped symmetric buffers that live outside
PyTorch's caching allocator, and can be scripted on a CPU box), MAX-reduces each step's readings over the ranks
in one packed collective, and installs what ``search_plans`` returns.
"""
from __future__ import annotations

import os
import enum
from dataclasses import dataclass, replace
from typing import Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

T0_RECOMPUTE = "recompute"
T1_KEEP_MHA = "keep_mha"
T2_OFFLOAD = "offload"      # defined for completeness; excluded from the search as in the reference (:82-101)
T4_RETAIN = "retain"

EDGE_GPU_PERSIST = "gpu_persist"
EDGE_GPU_EPHEMERAL = "gpu_ephemeral"
EDGE_CPU_BROADCAST = "cpu_broadcast"
EDGE_CPU_RANK_LOCAL_PREFETCH = "cpu_rank_local_prefetch"
EDGE_CPU_BROADCAST_PREFETCH = "cpu_broadcast_prefetch"
EDGE_POLICY_ORDER = (EDGE_GPU_PERSIST, EDGE_GPU_EPHEMERAL, EDGE_CPU_RANK_LOCAL_PREFETCH,
                     EDGE_CPU_BROADCAST_PREFETCH, EDGE_CPU_BROADCAST)
TIER_IDS = {T0_RECOMPUTE: 0, T1_KEEP_MHA: 1, T4_RETAIN: 2}
TIER_FROM_ID = {v: k for k, v in TIER_IDS.items()}

FRAGMENTATION_PER_EXTRA_LAYER = 0.05   # each kept layer beyond the first inflates the per-layer bytes by this much
SWITCH_TO_GPU_AFTER_WAIT_S = 0.5       # a CPU policy is reconsidered when its wait exceeds a GPU build by this
HEADROOM = 0.1                         # fraction of the (capped) device memory the plan must leave free


class MemoryProbe:
    """Device-memory readings used by the planner."""

    extra_bytes_fn: Optional[Callable[[], int]] = None   # e.g. symmetric buffers outside the allocator

    def available(self) -> bool:
        return torch.cuda.is_available()

    def _extra(self) -> int:
        return int(self.extra_bytes_fn()) if self.extra_bytes_fn is not None else 0

    def reset_peak(self, device) -> None:
        torch.cuda.reset_peak_memory_stats(device)

    def peak(self, device) -> int:
        return int(torch.cuda.max_memory_allocated(device)) + self._extra()

    def live(self, device) -> int:
        return int(torch.cuda.memory_allocated(device)) + self._extra()

    def total(self, device) -> int:
        return int(torch.cuda.get_device_properties(device).total_memory)

    def cpu_available(self) -> int:
        try:
            import psutil
            return int(psutil.virtual_memory().available)
        except Exception:
            return 1 << 62

    def rss(self) -> int:
        try:
            with open("/proc/self/statm") as fh:
                return int(fh.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")
        except Exception:
            return 0


class ScriptedMemoryProbe(MemoryProbe):
    """Probe for tests and dry runs: peak/live come from a function of the current tier layout."""

    def __init__(self, total_bytes: int, fn: Callable[[Sequence[str]], Dict[str, int]]):
        self._total, self._fn, self.modes = int(total_bytes), fn, []

    def available(self) -> bool:
        return True

    def reset_peak(self, device) -> None:
        pass

    def peak(self, device) -> int:
        return int(self._fn(self.modes)["peak"])

    def live(self, device) -> int:
        return int(self._fn(self.modes)["live"])

    def total(self, device) -> int:
        return self._total

    def cpu_available(self) -> int:
        return 1 << 50


def _is_rank0() -> bool:
    return (not dist.is_initialized()) or dist.get_rank() == 0


def _sync_max(values: Sequence[float], device) -> List[float]:
    """MAX over ranks of several scalars in one collective."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return [float(v) for v in values]
    dev = torch.device(device) if dist.get_backend() == "nccl" else torch.device("cpu")
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.tolist()]


# ---------------------------------------------------------------------------------------------------------
# records
# ---------------------------------------------------------------------------------------------------------
class Phase(enum.Enum):
    DEFERRED = "DEFERRED"
    WARMUP_RECOMPUTE = "WARMUP_RECOMPUTE"
    CALIBRATE_MHA = "CALIBRATE_MHA"
    CALIBRATE_MHA_FRONT = "CALIBRATE_MHA_FRONT"
    CALIBRATE_RETAIN = "CALIBRATE_RETAIN"
    CALIBRATE_RETAIN_FRONT = "CALIBRATE_RETAIN_FRONT"
    ACTIVE = "ACTIVE"


# calibration phase -> (tier under test, probed layer: -1 last / 0 first, phase after it, phase when the probe of the
# first layer is skipped or this was it)
_PHASE_PROBE = {
    Phase.CALIBRATE_MHA: (T1_KEEP_MHA, -1, Phase.CALIBRATE_MHA_FRONT, Phase.CALIBRATE_RETAIN),
    Phase.CALIBRATE_MHA_FRONT: (T1_KEEP_MHA, 0, None, Phase.CALIBRATE_RETAIN),
    Phase.CALIBRATE_RETAIN: (T4_RETAIN, -1, Phase.CALIBRATE_RETAIN_FRONT, Phase.ACTIVE),
    Phase.CALIBRATE_RETAIN_FRONT: (T4_RETAIN, 0, None, Phase.ACTIVE),
}


@dataclass(frozen=True)
class StepReading:
    """One training step as the planner sees it (already MAX-reduced over ranks)."""
    peak: int = 0               # allocator peak of the step (+ symmetric buffers)
    live: int = 0               # bytes alive right after the forward pass
    t_fwd: float = 0.0
    t_bwd: float = 0.0


@dataclass(frozen=True)
class TierProbe:
    """What one tier costs, from probing a single layer at the back and (optionally) at the front of the stack."""
    last: Optional[StepReading] = None
    front: Optional[StepReading] = None
    impossible: bool = False        # the tier ran out of memory even on one layer
    last_layer_only: bool = False   # a second layer of this tier cannot fit (front probe skipped or failed)

    def worst(self) -> StepReading:
        rs = [r for r in (self.last, self.front) if r is not None]
        if not rs:
            return StepReading()
        return StepReading(max(r.peak for r in rs), max(r.live for r in rs), max(r.t_fwd for r in rs),
                           max(r.t_bwd for r in rs))


@dataclass(frozen=True)
class Calibration:
    n_layers: int
    baseline: StepReading = StepReading()       # every layer recomputed
    keep: TierProbe = TierProbe()
    retain: TierProbe = TierProbe()
    # device bytes of a resident topology that were alive while the baseline was measured (the warm-up runs under
    # whatever edge policy is active then): taken out of the baseline before a policy's own residency is added
    resident_in_baseline: int = 0

    def probe(self, tier: str) -> TierProbe:
        return self.keep if tier == T1_KEEP_MHA else self.retain

    def with_probe(self, tier: str, p: TierProbe) -> "Calibration":
        return replace(self, keep=p) if tier == T1_KEEP_MHA else replace(self, retain=p)


@dataclass(frozen=True)
class EdgeCost:
    """Measured cost of one graph-placement policy."""
    policy: str
    prep_s: float = 0.0
    serial_s: float = 0.0           # part of the build the step has to wait for
    overlap_s: float = 0.0          # part hidden behind the model step (prefetch)
    build_peak: int = 0             # device peak during the build
    host_bytes: int = 0             # resident-set growth on the host
    resident_bytes: int = 0         # device bytes that stay alive between epochs (persistent topology)
    walk_gpu_extra: int = 0         # extra device bytes if the walks are forced onto the GPU


@dataclass(frozen=True)
class TierCost:
    t_fwd: float                    # per layer
    t_bwd: float
    bytes_deepest: int              # charged to the deepest layer of the tier when it is the last layer of the model
    bytes_each: int                 # charged to every further layer of the tier


@dataclass(frozen=True)
class Layout:
    n_recompute: int
    n_keep: int
    n_retain: int

    def tiers(self) -> List[str]:
        return [T0_RECOMPUTE] * self.n_recompute + [T1_KEEP_MHA] * self.n_keep + [T4_RETAIN] * self.n_retain

    @property
    def kept_score(self) -> int:    # tie-break: more retained state first
        return 2 * self.n_retain + self.n_keep


@dataclass(frozen=True)
class PlanChoice:
    policy: str
    layout: Layout
    walks_on_gpu: bool
    t_step: float
    t_model: float
    t_edge: float
    peak: int


# ---------------------------------------------------------------------------------------------------------
# phase transitions
# ---------------------------------------------------------------------------------------------------------
def probe_layout(phase: Phase, n_layers: int) -> List[str]:
    """Tier of every layer while ``phase`` runs: all recomputed, except the one layer a calibration phase tests."""
    modes = [T0_RECOMPUTE] * n_layers
    if phase in _PHASE_PROBE and n_layers > 0:
        tier, where, _nxt, _skip = _PHASE_PROBE[phase]
        modes[where] = tier
    return modes


def warmup_baseline(samples: Sequence[StepReading]) -> StepReading:
    """Baseline from the warm-up steps: the first one is discarded when there are several (allocator warm-up); peak is
    the maximum, times are means."""
    used = list(samples[1:]) if len(samples) > 1 else list(samples)
    n = float(len(used))
    return StepReading(max(r.peak for r in used), max(r.live for r in used), sum(r.t_fwd for r in used) / n,
                       sum(r.t_bwd for r in used) / n)


def advance(phase: Phase, cal: Calibration, reading: StepReading, peak_limit: int) -> Tuple[Phase, Calibration]:
    """Record a calibration step and name the next phase.  The first-layer probe of a tier is skipped when a second
    layer of it cannot fit on top of the baseline (the tier is then usable on the last layer only)."""
    tier, where, nxt, skip_to = _PHASE_PROBE[phase]
    p = cal.probe(tier)
    if where == -1:
        p = replace(p, last=reading)
        per_layer = max(0, reading.live - cal.baseline.live)
        second_fits = cal.baseline.peak + per_layer <= peak_limit
        if cal.n_layers <= 1:
            return skip_to, cal.with_probe(tier, p)
        if not second_fits:
            return skip_to, cal.with_probe(tier, replace(p, last_layer_only=True))
        return nxt, cal.with_probe(tier, p)
    return skip_to, cal.with_probe(tier, replace(p, front=reading))


def after_failed_probe(phase: Phase, cal: Calibration) -> Optional[Tuple[Phase, Calibration]]:
    """A calibration step ran out of memory: a failed last-layer probe rules the tier out, a failed first-layer probe
    restricts it to the last layer.  ``None`` outside calibration."""
    if phase not in _PHASE_PROBE:
        return None
    tier, where, _nxt, skip_to = _PHASE_PROBE[phase]
    p = cal.probe(tier)
    p = replace(p, impossible=True) if where == -1 else replace(p, last_layer_only=True)
    return skip_to, cal.with_probe(tier, p)


# ---------------------------------------------------------------------------------------------------------
# cost model
# ---------------------------------------------------------------------------------------------------------
def tier_costs(cal: Calibration) -> Dict[str, TierCost]:
    """Per-layer time and memory of each tier.  A probe changes one layer, so its step time differs from the
    baseline's by (tier layer - recomputed layer): ``t_tier = T_base / L + (T_probe - T_base)``, then forced into the
    physical order retain <= keep_mha <= recompute.  Memory: the deepest kept layer costs what the last-layer probe
    added to the step peak; any further layer costs the bytes the probe left alive after the forward pass."""
    n = max(1, cal.n_layers)
    base = cal.baseline
    rec = TierCost(base.t_fwd / n, base.t_bwd / n, 0, 0)
    out = {T0_RECOMPUTE: rec}
    ceiling = rec
    for tier in (T1_KEEP_MHA, T4_RETAIN):
        pr = cal.probe(tier)
        w = pr.worst()
        t_f = min(max(rec.t_fwd + (w.t_fwd - base.t_fwd), 0.0), ceiling.t_fwd)
        t_b = min(max(rec.t_bwd + (w.t_bwd - base.t_bwd), 0.0), ceiling.t_bwd)
        deepest = max(0, (pr.last.peak if pr.last is not None else 0) - base.peak)
        each = max(0, w.live - base.live) if pr.last is not None else 0
        out[tier] = ceiling = TierCost(t_f, t_b, deepest, each)
    return out


def stacked_bytes(n_layers: int, bytes_each: int) -> int:
    """``n_layers`` further layers of one tier; every layer beyond the first adds 5 % for fragmentation."""
    return n_layers * int(bytes_each * (1.0 + FRAGMENTATION_PER_EXTRA_LAYER * max(0, n_layers - 1)))


def layout_bytes(layout: Layout, costs: Dict[str, TierCost]) -> int:
    """Activation bytes a layout adds to the all-recompute peak.  The model's last layer is the deepest kept one and
    is charged the measured last-layer delta of its tier; the others are stacked per tier."""
    keep, ret = costs[T1_KEEP_MHA], costs[T4_RETAIN]
    if layout.n_retain > 0:
        return ret.bytes_deepest + stacked_bytes(layout.n_retain - 1, ret.bytes_each) + stacked_bytes(layout.n_keep, keep.bytes_each)
    if layout.n_keep > 0:
        return keep.bytes_deepest + stacked_bytes(layout.n_keep - 1, keep.bytes_each)
    return 0


def layout_times(layout: Layout, costs: Dict[str, TierCost]) -> Tuple[float, float]:
    counts = ((T0_RECOMPUTE, layout.n_recompute), (T1_KEEP_MHA, layout.n_keep), (T4_RETAIN, layout.n_retain))
    return (sum(k * costs[t].t_fwd for t, k in counts), sum(k * costs[t].t_bwd for t, k in counts))


def admissible_layouts(cal: Calibration) -> Iterator[Layout]:
    """Every ``[recompute]*a + [keep_mha]*b + [retain]*c`` the probes did not rule out."""
    n = cal.n_layers
    for n_keep in range(n + 1):
        for n_ret in range(n - n_keep + 1):
            if n_keep and cal.keep.impossible:
                continue
            if n_ret and cal.retain.impossible:
                continue
            if cal.keep.last_layer_only and n_keep and (n_keep > 1 or n_ret > 0):
                continue                                   # keep_mha only as the model's last layer
            if cal.retain.last_layer_only and n_ret > 1:
                continue
            yield Layout(n - n_keep - n_ret, n_keep, n_ret)


def search_plans(cal: Calibration, edge_costs: Sequence[EdgeCost], peak_limit: int, host_budget: int,
                 excluded: Sequence[str] = ()):
    """Fastest feasible (policy, layout).  Returns ``(best, best_without_resident_topology, report)``; ``report`` maps
    each policy to ``("ok", best ms)`` or ``("skip:<why>", None)``.

    feasible:  max(build peak, baseline peak without the topology that was resident while it was measured
                                + this policy's resident topology + layout bytes) <= peak_limit
    step time: model + serial build + the part of the overlapped build the model step does not hide
    order:     time, then more kept activations, then no resident topology, then less host memory, then lower build peak"""
    costs = tier_costs(cal)
    layouts = [(lay, layout_bytes(lay, costs), layout_times(lay, costs)) for lay in admissible_layouts(cal)] \
        if cal.baseline.t_bwd > 0 else []
    best = best_free = None
    best_key = best_free_key = None
    report: Dict[str, tuple] = {}
    model_peak = max(0, cal.baseline.peak - cal.resident_in_baseline)
    for ec in edge_costs:
        if ec.policy in excluded:
            report[ec.policy] = ("skip:gpu_infeasible", None)
            continue
        if ec.host_bytes > host_budget:
            report[ec.policy] = ("skip:cpu_budget", None)
            continue
        variants = [(ec.build_peak, ec.overlap_s, False, ec.host_bytes)]
        if ec.policy == EDGE_GPU_PERSIST and ec.walk_gpu_extra > 0:
            # walks forced onto the GPU: nothing left to overlap, no host memory, a larger build peak
            variants.append((max(ec.build_peak, ec.resident_bytes + ec.walk_gpu_extra), 0.0, True, 0))
        fastest = float("inf")
        for build_peak, overlap, walks_gpu, host in variants:
            for lay, extra, (t_f, t_b) in layouts:
                peak = max(int(build_peak), model_peak + ec.resident_bytes + extra)
                if peak > peak_limit:
                    continue
                t_model = t_f + t_b
                t_edge = ec.serial_s + max(0.0, overlap - t_model)
                t_step = t_model + t_edge
                fastest = min(fastest, t_step)
                key = (t_step, -lay.kept_score, int(ec.resident_bytes > 0), host, build_peak)
                choice = PlanChoice(ec.policy, lay, walks_gpu, t_step, t_model, t_edge, peak)
                if best_key is None or key < best_key:
                    best_key, best = key, choice
                if ec.resident_bytes == 0 and (best_free_key is None or key < best_free_key):
                    best_free_key, best_free = key, choice
        report[ec.policy] = ("ok", fastest * 1e3) if fastest < float("inf") else ("skip:no_feasible_tier", None)
    return best, best_free, report


def demoted(modes: Sequence[str]) -> Optional[List[str]]:
    """One tier down on the shallowest layer that still keeps anything (retain -> keep_mha -> recompute); ``None``
    when every layer is already recomputed."""
    ids = [TIER_IDS[m] for m in modes]
    for i, t in enumerate(ids):
        if t > 0:
            ids[i] = t - 1
            return [TIER_FROM_ID[j] for j in ids]
    return None


def _count(tiers) -> dict:
    out: Dict[str, int] = {}
    for t in tiers:
        out[t] = out.get(t, 0) + 1
    return out


# ---------------------------------------------------------------------------------------------------------
# the planner object
# ---------------------------------------------------------------------------------------------------------
_NEUTRAL_EDGE_COST = EdgeCost(EDGE_GPU_EPHEMERAL)      # no profile yet: tiers can still be planned


class ExecutionPlanner:
    def __init__(self, n_layers: int, safety_margin: float = HEADROOM, deferred: bool = False,
                 probe: Optional[MemoryProbe] = None, verbose: bool = True):
        self.n_layers = int(n_layers)
        self.headroom = float(safety_margin)
        self.probe = probe if probe is not None else MemoryProbe()
        self.verbose = verbose
        self.phase = Phase.DEFERRED if deferred else Phase.WARMUP_RECOMPUTE
        self.calibration = Calibration(self.n_layers)
        self.edge_costs: Dict[str, EdgeCost] = {}
        self.excluded_policies: set = set()
        self.memory_cap_bytes = 0
        self.last_plan_log: Dict[str, tuple] = {}
        self._warmup_steps_wanted = 1 if deferred else 3
        self._warmup: List[StepReading] = []
        self._deferred_reading: Optional[StepReading] = None
        self._live_after_forward = 0
        self._modes: List[str] = [T0_RECOMPUTE] * self.n_layers
        self._choice = PlanChoice(EDGE_GPU_EPHEMERAL, Layout(self.n_layers, 0, 0), False, float("inf"), 0.0, 0.0, 0)
        self._fallback = (EDGE_GPU_EPHEMERAL, [T0_RECOMPUTE] * self.n_layers)   # best plan without a resident topology
        self._topology_bytes, self._topology_h2d_s = 0, 0.0
        # set by the trainer: names the edge policy the steps currently run under (None: unknown)
        self.active_edge_policy_fn: Optional[Callable[[], str]] = None

    # ------------------------------------------------------------------ small helpers
    def _log(self, msg: str) -> None:
        if self.verbose and _is_rank0():
            print(f"[MultiTierManager] {msg}")

    def _install(self, modes: Sequence[str]) -> None:
        self._modes = list(modes)
        if isinstance(self.probe, ScriptedMemoryProbe):
            self.probe.modes = self._modes

    def _device_bytes(self, device) -> int:
        total = int(self.probe.total(device))
        return min(total, self.memory_cap_bytes) if self.memory_cap_bytes > 0 else total

    def _peak_limit(self, device) -> int:
        return int(self._device_bytes(device) * (1.0 - self.headroom))

    # ------------------------------------------------------------------ inputs
    def set_gpu_memory_limit_bytes(self, limit_bytes: int) -> None:
        self.memory_cap_bytes = max(0, int(limit_bytes))

    def set_edge_info(self, edge_bytes: int, t_h2d: float) -> None:
        self._topology_bytes, self._topology_h2d_s = int(edge_bytes), float(t_h2d)

    def set_edge_policy_profile(self, policy: str, prep_time_s: float, gpu_peak_bytes: int, cpu_delta_bytes: int,
                                live_edge_bytes: int = 0, serial_time_s=None, overlap_time_s: float = 0.0,
                                rw_gpu_extra_bytes: int = 0, enabled: bool = True) -> None:
        if policy not in EDGE_POLICY_ORDER:
            raise ValueError(f"Unsupported edge policy profile: {policy!r}")
        if not enabled:
            self.edge_costs.pop(policy, None)
            return
        nn = lambda v: max(0, int(v))
        self.edge_costs[policy] = EdgeCost(
            policy, prep_s=max(0.0, float(prep_time_s)),
            serial_s=max(0.0, float(prep_time_s if serial_time_s is None else serial_time_s)),
            overlap_s=max(0.0, float(overlap_time_s)), build_peak=nn(gpu_peak_bytes), host_bytes=nn(cpu_delta_bytes),
            resident_bytes=nn(live_edge_bytes), walk_gpu_extra=nn(rw_gpu_extra_bytes))

    def _ordered_edge_costs(self) -> List[EdgeCost]:
        if not self.edge_costs:
            return [_NEUTRAL_EDGE_COST]
        return [self.edge_costs[p] for p in EDGE_POLICY_ORDER if p in self.edge_costs]

    # ------------------------------------------------------------------ per-step protocol
    def notify_budget_frozen(self, reuse_deferred_baseline: bool = False) -> None:
        """The edge budget stopped moving: leave DEFERRED.  The last deferred step (all layers recomputed) can serve as
        the warm-up sample, so calibration starts at once."""
        if self.phase is not Phase.DEFERRED:
            return
        self.phase, self._warmup = Phase.WARMUP_RECOMPUTE, []
        if reuse_deferred_baseline and self._deferred_reading is not None:
            self._warmup = [self._deferred_reading]
            self._close_warmup()
        self._log(f"edge budget frozen -> {self.state_name()}")

    def plan(self, device) -> None:
        """Called at the top of every forward pass: sets the layer tiers of this step."""
        if not self.probe.available() or self.phase is Phase.ACTIVE:
            return
        self._install(probe_layout(self.phase, self.n_layers))
        self.probe.reset_peak(device)
        if self.phase is not Phase.DEFERRED:
            self._log(f"{self.state_name()}: tiers={_count(self._modes)}")

    def record_post_forward_memory(self, device) -> None:
        if self.probe.available() and self.phase is not Phase.ACTIVE:
            self._live_after_forward = int(self.probe.live(device))

    def notify_step_end(self, device, t_bwd: float = None, t_fwd: float = None) -> None:
        if not self.probe.available() or self.phase is Phase.ACTIVE:
            return
        peak, live, t_f, t_b = _sync_max([self.probe.peak(device), self._live_after_forward, t_fwd or 0.0, t_bwd or 0.0],
                                         device)
        reading = StepReading(int(peak), int(live), t_f, t_b)
        if self.phase is Phase.DEFERRED:
            self._deferred_reading = reading
        elif self.phase is Phase.WARMUP_RECOMPUTE:
            self._warmup.append(reading)
            if len(self._warmup) >= self._warmup_steps_wanted:
                self._close_warmup()
        else:
            self.phase, self.calibration = advance(self.phase, self.calibration, reading, self._peak_limit(device))
            if self.phase is Phase.ACTIVE:
                self._choose(device)

    def _close_warmup(self) -> None:
        base = warmup_baseline(self._warmup)
        under = self.active_edge_policy_fn() if self.active_edge_policy_fn is not None else None
        resident = self.edge_costs[under].resident_bytes if under in self.edge_costs else 0
        self.calibration = replace(self.calibration, baseline=base, resident_in_baseline=int(resident))
        self.phase = Phase.CALIBRATE_MHA
        self._log(f"warm-up done: peak={base.peak / 2**20:.0f} MiB t_fwd={base.t_fwd * 1e3:.1f} ms "
                  f"t_bwd={base.t_bwd * 1e3:.1f} ms")

    # ------------------------------------------------------------------ planning
    def _choose(self, device) -> None:
        limit = self._peak_limit(device) if self.probe.available() else 0
        best, best_free, report = search_plans(self.calibration, self._ordered_edge_costs(), limit,
                                               self.probe.cpu_available(), tuple(self.excluded_policies))
        self.last_plan_log = report
        if best is None:
            # nothing fits the model's estimate: every layer recomputed under the cheapest policy still in the search
            left = [p for p in (EDGE_GPU_EPHEMERAL, EDGE_CPU_RANK_LOCAL_PREFETCH, EDGE_CPU_BROADCAST_PREFETCH, EDGE_GPU_PERSIST)
                    if p not in self.excluded_policies]
            best = PlanChoice(left[0] if left else EDGE_CPU_RANK_LOCAL_PREFETCH, Layout(self.n_layers, 0, 0), False,
                              float("inf"), 0.0, 0.0, 0)
        self._choice = best
        self._fallback = (best_free.policy, best_free.layout.tiers()) if best_free is not None else \
            (EDGE_GPU_EPHEMERAL, [T0_RECOMPUTE] * self.n_layers)
        self._install(best.layout.tiers())
        self.phase = Phase.ACTIVE
        shown = [f"{p}:{v[1]:.0f}ms{' [SELECTED]' if p == best.policy else ''}" if v[0] == "ok" else f"{p}:{v[0]}"
                 for p, v in report.items()]
        t_ms = best.t_step * 1e3 if best.t_step < float("inf") else 0.0
        self._log(f"ACTIVE plan: edge_policy={best.policy} rw_device={'GPU' if best.walks_on_gpu else 'auto'} "
                  f"tiers={_count(self._modes)} peak_limit={limit / 2**20:.0f} MiB est_T_step={t_ms:.0f} ms "
                  f"(model={best.t_model * 1e3:.0f} ms edge_prep={best.t_edge * 1e3:.0f} ms)")
        self._log("  policy candidates: " + " | ".join(shown))

    # ------------------------------------------------------------------ accessors
    def mode(self, layer_idx: int) -> str:
        return self._modes[layer_idx]

    def modes(self) -> List[str]:
        return list(self._modes)

    def is_active(self) -> bool:
        return self.phase is Phase.ACTIVE

    def state_name(self) -> str:
        return self.phase.value

    def needs_precise_timing(self) -> bool:
        return self.phase not in (Phase.ACTIVE, Phase.DEFERRED)

    @property
    def edge_policy(self) -> str:
        return self._choice.policy

    @property
    def cache_edge(self) -> bool:
        return self._choice.policy == EDGE_GPU_PERSIST

    @property
    def rw_on_gpu(self) -> bool:
        return self._choice.walks_on_gpu

    @property
    def best_nonpersistent_edge_policy(self) -> str:
        return self._fallback[0]

    @property
    def best_nonpersistent_tiers(self) -> list:
        return list(self._fallback[1])

    def override_cache_decision(self, cache: bool) -> None:
        """Giving up the resident topology moves the plan to the best one that never needed it."""
        if not cache and self.cache_edge:
            policy, tiers = self._fallback
            self._choice = replace(self._choice, policy=policy, walks_on_gpu=False)
            self._install(tiers)

    def override_active_plan(self, edge_policy: str, modes: List[str]) -> None:
        """Install an externally agreed plan (cross-rank consensus or ``--force_multi_tier_plan``)."""
        if len(modes) != self.n_layers:
            raise ValueError(f"plan has {len(modes)} tiers for {self.n_layers} layers")
        unknown = [m for m in modes if m not in TIER_IDS]
        if unknown:
            raise ValueError(f"unknown tier {unknown[0]!r}")
        self._choice = replace(self._choice, policy=str(edge_policy),
                               walks_on_gpu=self._choice.walks_on_gpu and edge_policy == EDGE_GPU_PERSIST)
        self._install(modes)
        self.phase = Phase.ACTIVE
        self._log(f"ACTIVE plan (override): edge_policy={edge_policy} tiers={_count(modes)}")

    # ------------------------------------------------------------------ run-time feedback
    def reconsider_with_actual_timing(self, device, t_model_actual: float, t_edge_wait_actual: float,
                                      gpu_policy_serial_s: Optional[float] = None) -> Optional[str]:
        """One-way CPU -> GPU switch.  Under a CPU prefetch policy, when the step waited for its graph more than
        0.5 s longer than the cheapest admissible GPU build would take, the policy's overlap figure is replaced by what
        was measured (model + wait) and the search runs again.  Returns the new policy when it changed."""
        current = self.edge_costs.get(self.edge_policy)
        if (not self.is_active() or current is None
                or self.edge_policy not in (EDGE_CPU_RANK_LOCAL_PREFETCH, EDGE_CPU_BROADCAST_PREFETCH)):
            return None
        gpu = [self.edge_costs[p] for p in (EDGE_GPU_PERSIST, EDGE_GPU_EPHEMERAL)
               if p in self.edge_costs and p not in self.excluded_policies]
        if not gpu:
            return None
        gpu_build_s = min(c.serial_s for c in gpu) if gpu_policy_serial_s is None else float(gpu_policy_serial_s)
        if t_edge_wait_actual - gpu_build_s <= SWITCH_TO_GPU_AFTER_WAIT_S:
            return None
        self.edge_costs[current.policy] = replace(current, overlap_s=float(t_model_actual + t_edge_wait_actual))
        before = self.edge_policy
        self._choose(device)
        if self.edge_policy == before:
            return None
        self._log(f"timing feedback: {before} waited {t_edge_wait_actual:.2f}s -> switched to {self.edge_policy}")
        return self.edge_policy

    def report_runtime_edge_gpu_infeasible(self, device) -> bool:
        """A GPU graph build fell back to the CPU at run time: GPU policies leave the search for good."""
        gpu = {EDGE_GPU_EPHEMERAL, EDGE_GPU_PERSIST}
        if gpu <= self.excluded_policies:
            return False
        self.excluded_policies |= gpu
        if self.is_active():
            self._choose(device)
        return True

    def mark_current_calibration_infeasible(self, device) -> bool:
        """The calibration step in flight ran out of memory."""
        moved = after_failed_probe(self.phase, self.calibration)
        if moved is None:
            return False
        self.phase, self.calibration = moved
        if self.phase is Phase.ACTIVE:
            self._choose(device)
        self._log(f"calibration step ran out of memory -> {self.state_name()}")
        return True

    def apply_oom_fallback(self, device, sp_group=None, sp_world_size: int = 1) -> bool:
        """An ACTIVE step ran out of memory: demote one layer by one tier and agree on the element-wise minimum over
        the ranks; with nothing left to demote, give up the resident topology; else report failure."""
        lower = demoted(self._modes)
        if lower is None:
            if self.cache_edge:
                self.override_cache_decision(False)
                return True
            return False
        if sp_world_size > 1 and dist.is_initialized():
            dev = torch.device(device) if dist.get_backend(sp_group) == "nccl" else torch.device("cpu")
            ids = torch.tensor([TIER_IDS[m] for m in lower], dtype=torch.int64, device=dev)
            dist.all_reduce(ids, op=dist.ReduceOp.MIN, group=sp_group)
            lower = [TIER_FROM_ID[int(i)] for i in ids.tolist()]
        self._install(lower)
        self._log(f"OOM fallback -> tiers={_count(self._modes)}")
        return True


class CommAwareCheckpointer:
    """``--activation_checkpoint_mode adaptive``: warm up with every layer recomputed, measure the
    per-layer cost of keeping the attention half, then keep ``keep_mha`` greedily from the last layer
    inward while the measured peak plus the kept layers stays under 90 % of the device
    (models/graphormer_dist_node_level.py:743-1105)."""

    _WARMUP, _CALIBRATE, _ACTIVE = 0, 1, 2

    def __init__(self, n_layers: int, safety_margin: float = 0.1, probe: Optional[MemoryProbe] = None):
        self.n_layers = int(n_layers)
        self.safety_margin = safety_margin
        self.probe = probe if probe is not None else MemoryProbe()
        self._state = self._WARMUP
        self._modes = ["layer"] * self.n_layers
        self._peak_warmup = 0
        self._live = {}
        self.cache_edge = False

    def plan(self, device) -> None:
        if not self.probe.available() or self._state == self._ACTIVE:
            return
        self._modes = ["layer"] * self.n_layers
        if self._state == self._CALIBRATE:
            self._modes[-1] = "keep_mha"
        if isinstance(self.probe, ScriptedMemoryProbe):
            self.probe.modes = ["recompute" if m == "layer" else m for m in self._modes]
        self.probe.reset_peak(device)

    def record_post_forward_memory(self, device) -> None:
        if self.probe.available() and self._state != self._ACTIVE:
            self._live[self._state] = self.probe.live(device)

    def notify_step_end(self, device, t_bwd=None, t_fwd=None) -> None:
        if not self.probe.available() or self._state == self._ACTIVE:
            return
        peak, live = _sync_max([self.probe.peak(device), self._live.get(self._state, 0)], device)
        if self._state == self._WARMUP:
            self._peak_warmup, self._live[self._WARMUP] = int(peak), int(live)
            self._state = self._CALIBRATE
            return
        m_layer = max(0, int(live) - int(self._live.get(self._WARMUP, 0)))
        limit = int(self.probe.total(device) * (1.0 - self.safety_margin))
        k = 0
        while k < self.n_layers and self._peak_warmup + (k + 1) * m_layer <= limit:
            k += 1
        self._modes = ["layer"] * (self.n_layers - k) + ["keep_mha"] * k
        self._state = self._ACTIVE

    def mode(self, i: int) -> str:
        return self._modes[i]

    def is_active(self) -> bool:
        return self._state == self._ACTIVE

    def needs_precise_timing(self) -> bool:
        return False


def parse_force_multi_tier_plan(spec: str, n_layers: int):
    """``"<edge_policy>:<recompute|keep_mha=N|retain=N>"`` -> (policy, tiers); N counts layers from the back
    (main_node_fullgraph_sp.py:114-156)."""
    spec = (spec or "").strip()
    if not spec:
        return None
    if ":" not in spec:
        raise ValueError(f"--force_multi_tier_plan expects '<edge_policy>:<tier_config>', got {spec!r}")
    policy, cfg = (s.strip() for s in spec.split(":", 1))
    if policy not in (EDGE_GPU_PERSIST, EDGE_GPU_EPHEMERAL, EDGE_CPU_RANK_LOCAL_PREFETCH, EDGE_CPU_BROADCAST_PREFETCH):
        raise ValueError(f"unknown edge policy {policy!r} in --force_multi_tier_plan")
    tiers = [T0_RECOMPUTE] * n_layers
    if cfg == "recompute":
        return policy, tiers
    if "=" not in cfg:
        raise ValueError(f"unknown tier config {cfg!r} in --force_multi_tier_plan")
    name, val = (s.strip() for s in cfg.split("=", 1))
    k = int(val)
    if name not in (T1_KEEP_MHA, T4_RETAIN) or not (0 <= k <= n_layers):
        raise ValueError(f"bad tier config {cfg!r} for {n_layers} layers")
    for i in range(n_layers - k, n_layers):
        tiers[i] = name
    return policy, tiers
