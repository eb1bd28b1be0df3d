"""Multi-Tier Execution Planner: profile -> plan -> execute under an HBM cap.

Jointly chooses (a) where the per-epoch attention graph is built (``gpu_persist`` |
``gpu_ephemeral`` | ``cpu_rank_local_prefetch`` | ``cpu_broadcast_prefetch``) and (b) a per-layer
activation layout ``[recompute]*a + [keep_mha]*b + [retain]*c``.  The state machine, the cost /
memory model and the public methods follow the reference's ``gt_sp/multi_tier.py``
(``_MultiTierResourceManager`` :60-1562): DEFERRED -> WARMUP_RECOMPUTE -> CALIBRATE_MHA
[-> MHA_FRONT] -> CALIBRATE_RETAIN [-> RETAIN_FRONT] -> ACTIVE.

Re-grounding for B200: memory is read through a ``MemoryProbe`` so that (1) bytes held in
symmetric (peer-mapped) buffers, which live outside PyTorch's caching allocator, are charged to the
plan, and (2) the whole state machine runs on a CPU box against a scripted probe.  Cross-rank
agreement uses one packed MAX all-reduce per step instead of one blocking call per scalar.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Sequence

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

_FRAG_FACTOR = 0.05          # per additional kept layer (reference :1064)
_RECONSIDER_THRESHOLD_S = 0.5


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


class _MultiTierResourceManager:
    T0_RECOMPUTE, T1_KEEP_MHA, T2_OFFLOAD, T4_RETAIN = T0_RECOMPUTE, T1_KEEP_MHA, T2_OFFLOAD, T4_RETAIN
    EDGE_GPU_PERSIST, EDGE_GPU_EPHEMERAL, EDGE_CPU_BROADCAST = EDGE_GPU_PERSIST, EDGE_GPU_EPHEMERAL, EDGE_CPU_BROADCAST
    EDGE_CPU_RANK_LOCAL_PREFETCH = EDGE_CPU_RANK_LOCAL_PREFETCH
    EDGE_CPU_BROADCAST_PREFETCH = EDGE_CPU_BROADCAST_PREFETCH

    _DEFERRED, _WARMUP_RECOMPUTE, _CALIBRATE_MHA, _CALIBRATE_MHA_FRONT = -1, 0, 1, 2
    _CALIBRATE_RETAIN, _CALIBRATE_RETAIN_FRONT, _ACTIVE = 3, 4, 5
    _STATE_NAMES = {-1: "DEFERRED", 0: "WARMUP_RECOMPUTE", 1: "CALIBRATE_MHA", 2: "CALIBRATE_MHA_FRONT",
                    3: "CALIBRATE_RETAIN", 4: "CALIBRATE_RETAIN_FRONT", 5: "ACTIVE"}

    def __init__(self, n_layers: int, safety_margin: float = 0.1, deferred: bool = False,
                 probe: Optional[MemoryProbe] = None, verbose: bool = True):
        self.n_layers = int(n_layers)
        self.safety_margin = float(safety_margin)
        self.probe = probe if probe is not None else MemoryProbe()
        self.verbose = verbose
        self._state = self._DEFERRED if deferred else self._WARMUP_RECOMPUTE
        self._modes: List[str] = [T0_RECOMPUTE] * self.n_layers
        self._warmup_target = 1 if deferred else 3
        self._warmup_samples: List[tuple] = []            # (peak, t_fwd, t_bwd)
        self._deferred_baseline = None                    # (peak, fwd_live, t_fwd, t_bwd)
        self._fwd_live: Dict[int, int] = {}
        self._peak: Dict[int, int] = {}
        self._t_fwd: Dict[int, float] = {}
        self._t_bwd: Dict[int, float] = {}
        self._peak_warmup = 0
        self._peak_mha_last = self._peak_mha = 0
        self._peak_retain_last = self._peak_retain = 0
        self._m_layer_mha = self._m_layer_full = 0
        self._t_fwd_recompute = self._t_bwd_recompute = 0.0
        self._t_fwd_mha = self._t_bwd_mha = 0.0
        self._t_fwd_retain = self._t_bwd_retain = 0.0
        self._edge_bytes, self._t_h2d_edge = 0, 0.0
        self._edge_profiles: Dict[str, dict] = {}
        self._gpu_memory_limit_bytes = 0
        self._t1_infeasible = self._t4_infeasible = False
        self._t1_nonlast_infeasible = self._t4_nonlast_infeasible = False
        self._gpu_infeasible_policies: set = set()
        self._active_peak_limit = 0
        self._cache_edge = False
        self._rw_on_gpu = False
        self._edge_policy = EDGE_GPU_EPHEMERAL
        self._best_nonpersistent_edge_policy = EDGE_GPU_EPHEMERAL
        self._best_nonpersistent_tiers: List[str] = [T0_RECOMPUTE] * self.n_layers
        self.last_plan_log: Dict[str, tuple] = {}

    # ------------------------------------------------------------------ utilities
    def _log(self, msg: str) -> None:
        if self.verbose and _is_rank0():
            print(f"[MultiTierManager] {msg}")

    def set_gpu_memory_limit_bytes(self, limit_bytes: int) -> None:
        self._gpu_memory_limit_bytes = max(0, int(limit_bytes))

    def _effective_total_gpu_bytes(self, real_total: int) -> int:
        if self._gpu_memory_limit_bytes > 0:
            return min(int(real_total), self._gpu_memory_limit_bytes)
        return int(real_total)

    def _model_peak_limit_bytes(self, total_gpu: int) -> int:
        return int(total_gpu * (1.0 - self.safety_margin))

    def set_edge_info(self, edge_bytes: int, t_h2d: float) -> None:
        self._edge_bytes, self._t_h2d_edge = int(edge_bytes), float(t_h2d)

    def set_edge_policy_profile(self, policy: str, prep_time_s: float, gpu_peak_bytes: int, cpu_delta_bytes: int,
                                live_edge_bytes: int = 0, serial_time_s=None, overlap_time_s: float = 0.0,
                                rw_gpu_extra_bytes: int = 0, enabled: bool = True) -> None:
        policy = str(policy)
        if policy not in EDGE_POLICY_ORDER:
            raise ValueError(f"Unsupported edge policy profile: {policy!r}")
        if not enabled:
            self._edge_profiles.pop(policy, None)
            return
        self._edge_profiles[policy] = {
            "prep_time_s": max(0.0, float(prep_time_s)),
            "serial_time_s": max(0.0, float(serial_time_s if serial_time_s is not None else prep_time_s)),
            "overlap_time_s": max(0.0, float(overlap_time_s)),
            "gpu_peak_bytes": max(0, int(gpu_peak_bytes)),
            "cpu_delta_bytes": max(0, int(cpu_delta_bytes)),
            "live_edge_bytes": max(0, int(live_edge_bytes)),
            "rw_gpu_extra_bytes": max(0, int(rw_gpu_extra_bytes)),
        }

    def _edge_policy_profiles(self):
        if not self._edge_profiles:
            # no profile: a neutral ephemeral-GPU entry so that tiers can still be planned
            return [(EDGE_GPU_EPHEMERAL, {"prep_time_s": 0.0, "serial_time_s": 0.0, "overlap_time_s": 0.0,
                                          "gpu_peak_bytes": 0, "cpu_delta_bytes": 0, "live_edge_bytes": 0,
                                          "rw_gpu_extra_bytes": 0})]
        return [(p, self._edge_profiles[p]) for p in EDGE_POLICY_ORDER if p in self._edge_profiles]

    # ------------------------------------------------------------------ state machine
    def notify_budget_frozen(self, reuse_deferred_baseline: bool = False) -> None:
        if self._state != self._DEFERRED:
            return
        self._state = self._WARMUP_RECOMPUTE
        self._warmup_samples = []
        if reuse_deferred_baseline and self._deferred_baseline is not None:
            peak, live, t_f, t_b = self._deferred_baseline
            self._warmup_samples.append((peak, t_f, t_b))
            self._fwd_live[self._WARMUP_RECOMPUTE] = live
            self._warmup_target = 1
            self._finish_warmup()
        self._log(f"edge budget frozen -> {self.state_name()}")

    def _set_modes(self, modes: List[str]) -> None:
        self._modes = list(modes)
        if isinstance(self.probe, ScriptedMemoryProbe):
            self.probe.modes = self._modes

    def plan(self, device) -> None:
        if not self.probe.available():
            return
        s = self._state
        if s == self._ACTIVE:
            return
        modes = [T0_RECOMPUTE] * self.n_layers
        if s == self._CALIBRATE_MHA:
            modes[-1] = T1_KEEP_MHA
        elif s == self._CALIBRATE_MHA_FRONT:
            modes[0] = T1_KEEP_MHA
        elif s == self._CALIBRATE_RETAIN:
            modes[-1] = T4_RETAIN
        elif s == self._CALIBRATE_RETAIN_FRONT:
            modes[0] = T4_RETAIN
        self._set_modes(modes)
        self.probe.reset_peak(device)
        if s != self._DEFERRED:
            self._log(f"{self.state_name()}: tiers={self._tier_counts(modes)}")

    def record_post_forward_memory(self, device) -> None:
        if not self.probe.available() or self._state == self._ACTIVE:
            return
        self._fwd_live[self._state] = int(self.probe.live(device))

    def notify_step_end(self, device, t_bwd: float = None, t_fwd: float = None) -> None:
        if not self.probe.available() or self._state == self._ACTIVE:
            return
        s = self._state
        peak, live, t_f, t_b = _sync_max(
            [self.probe.peak(device), self._fwd_live.get(s, 0), t_fwd or 0.0, t_bwd or 0.0], device)
        peak, live = int(peak), int(live)
        self._fwd_live[s] = live
        total = self._effective_total_gpu_bytes(self.probe.total(device))
        limit = self._model_peak_limit_bytes(total)
        if s == self._DEFERRED:
            self._deferred_baseline = (peak, live, t_f, t_b)
            return
        if s == self._WARMUP_RECOMPUTE:
            self._warmup_samples.append((peak, t_f, t_b))
            if len(self._warmup_samples) >= self._warmup_target:
                self._finish_warmup()
            return
        self._peak[s], self._t_fwd[s], self._t_bwd[s] = peak, t_f, t_b
        base_live = self._fwd_live.get(self._WARMUP_RECOMPUTE, 0)
        if s == self._CALIBRATE_MHA:
            self._peak_mha_last = self._peak_mha = peak
            self._m_layer_mha = max(0, live - base_live)
            self._t_fwd_mha, self._t_bwd_mha = t_f, t_b
            if self.n_layers > 1 and self._peak_warmup + self._m_layer_mha > limit:
                self._t1_nonlast_infeasible = True          # skip the FRONT probe (reference :594-611)
                self._state = self._CALIBRATE_RETAIN
            else:
                self._state = self._CALIBRATE_MHA_FRONT if self.n_layers > 1 else self._CALIBRATE_RETAIN
        elif s == self._CALIBRATE_MHA_FRONT:
            self._peak_mha = max(self._peak_mha_last, peak)
            self._m_layer_mha = max(self._m_layer_mha, live - base_live)
            self._t_fwd_mha, self._t_bwd_mha = max(self._t_fwd_mha, t_f), max(self._t_bwd_mha, t_b)
            self._state = self._CALIBRATE_RETAIN
        elif s == self._CALIBRATE_RETAIN:
            self._peak_retain_last = self._peak_retain = peak
            self._m_layer_full = max(0, live - base_live)
            self._t_fwd_retain, self._t_bwd_retain = t_f, t_b
            if self.n_layers > 1 and self._peak_warmup + self._m_layer_full > limit:
                self._t4_nonlast_infeasible = True
                self._run_active_plan(device, total)
            elif self.n_layers > 1:
                self._state = self._CALIBRATE_RETAIN_FRONT
            else:
                self._run_active_plan(device, total)
        elif s == self._CALIBRATE_RETAIN_FRONT:
            self._peak_retain = max(self._peak_retain_last, peak)
            self._m_layer_full = max(self._m_layer_full, live - base_live)
            self._t_fwd_retain, self._t_bwd_retain = max(self._t_fwd_retain, t_f), max(self._t_bwd_retain, t_b)
            self._run_active_plan(device, total)

    def _finish_warmup(self) -> None:
        samples = self._warmup_samples[1:] if len(self._warmup_samples) > 1 else self._warmup_samples
        self._peak_warmup = max(s[0] for s in samples)
        self._t_fwd_recompute = sum(s[1] for s in samples) / len(samples)
        self._t_bwd_recompute = sum(s[2] for s in samples) / len(samples)
        self._state = self._CALIBRATE_MHA
        self._log(f"warm-up done: peak={self._peak_warmup / 2**20:.0f} MiB "
                  f"t_fwd={self._t_fwd_recompute * 1e3:.1f} ms t_bwd={self._t_bwd_recompute * 1e3:.1f} ms")

    # ------------------------------------------------------------------ planning
    def _enumerate_structured_plans(self, peak_limit: int, cpu_budget: int, edge_peak: int, build_peak: int = 0):
        L = self.n_layers
        if L == 0 or self._t_bwd_recompute <= 0:
            return []
        t_f_r = self._t_fwd_recompute / L
        t_f_k = max(t_f_r + (self._t_fwd_mha - self._t_fwd_recompute), 0.0)
        t_f_n = max(t_f_r + (self._t_fwd_retain - self._t_fwd_recompute), 0.0)
        t_r = self._t_bwd_recompute / L
        t_k = max(t_r + (self._t_bwd_mha - self._t_bwd_recompute), 0.0)
        t_n = max(t_r + (self._t_bwd_retain - self._t_bwd_recompute), 0.0)
        t_k, t_f_k = min(t_k, t_r), min(t_f_k, t_f_r)          # physical ordering retain <= keep <= recompute
        t_n, t_f_n = min(t_n, t_k), min(t_f_n, t_f_k)
        m_full, m_mha = int(self._m_layer_full), int(self._m_layer_mha)
        mha_delta_last = max(self._peak_mha_last - self._peak_warmup, 0)
        retain_delta_last = max(self._peak_retain_last - self._peak_warmup, 0)
        out = []
        for k_keep in range(L + 1):
            if k_keep > 0 and self._t1_infeasible:
                continue
            for k_ret in range(L - k_keep + 1):
                if k_ret > 0 and self._t4_infeasible:
                    continue
                k_rec = L - k_keep - k_ret
                if self._t1_nonlast_infeasible and k_keep > 0 and not (k_keep == 1 and k_ret == 0):
                    continue
                if self._t4_nonlast_infeasible and k_ret > 1:
                    continue
                if k_ret > 0:
                    nr, nk = k_ret - 1, k_keep
                    retain_extra = retain_delta_last + nr * int(m_full * (1.0 + _FRAG_FACTOR * max(0, nr - 1)))
                    mha_extra = nk * int(m_mha * (1.0 + _FRAG_FACTOR * max(0, nk - 1)))
                elif k_keep > 0:
                    nk = k_keep - 1
                    mha_extra = mha_delta_last + nk * int(m_mha * (1.0 + _FRAG_FACTOR * max(0, nk - 1)))
                    retain_extra = 0
                else:
                    mha_extra = retain_extra = 0
                peak_est = max(int(build_peak), self._peak_warmup + edge_peak + max(0, mha_extra + retain_extra))
                if peak_est > peak_limit:
                    continue
                tiers = [T0_RECOMPUTE] * k_rec + [T1_KEEP_MHA] * k_keep + [T4_RETAIN] * k_ret
                t_fwd_est = k_rec * t_f_r + k_keep * t_f_k + k_ret * t_f_n
                t_bwd_est = k_rec * t_r + k_keep * t_k + k_ret * t_n
                out.append((tiers, -(2 * k_ret + k_keep), 0, peak_est, t_fwd_est, t_bwd_est, t_fwd_est + t_bwd_est))
        return out

    def _run_active_plan(self, device, total_gpu: int) -> None:
        cpu_budget = self.probe.cpu_available()
        peak_limit = self._model_peak_limit_bytes(total_gpu)
        self._active_peak_limit = peak_limit
        best_key = best_np_key = None
        best = {"policy": EDGE_GPU_EPHEMERAL, "tiers": [T0_RECOMPUTE] * self.n_layers, "rw_gpu": False,
                "t_step": float("inf"), "t_model": 0.0, "t_edge": 0.0}
        best_np = (EDGE_GPU_EPHEMERAL, [T0_RECOMPUTE] * self.n_layers)
        log: Dict[str, tuple] = {}
        for policy, prof in self._edge_policy_profiles():
            if policy in self._gpu_infeasible_policies:
                log[policy] = ("skip:gpu_infeasible", None)
                continue
            if prof["cpu_delta_bytes"] > cpu_budget:
                log[policy] = ("skip:cpu_budget", None)
                continue
            edge_peak = int(prof["live_edge_bytes"])
            variants = [(prof["gpu_peak_bytes"], prof["serial_time_s"], prof["overlap_time_s"], False,
                         prof["cpu_delta_bytes"])]
            if policy == EDGE_GPU_PERSIST and prof["rw_gpu_extra_bytes"] > 0:
                variants.append((max(prof["gpu_peak_bytes"], edge_peak + prof["rw_gpu_extra_bytes"]),
                                 prof["serial_time_s"], 0.0, True, 0))
            policy_best = float("inf")
            for v_peak, v_serial, v_overlap, v_gpu, v_cpu in variants:
                for tiers, tie, cpu_est, peak_est, t_f, t_b, t_model in self._enumerate_structured_plans(
                        peak_limit, cpu_budget, edge_peak, v_peak):
                    t_edge = v_serial + max(0.0, v_overlap - t_model)
                    t_est = t_model + t_edge
                    policy_best = min(policy_best, t_est)
                    key = (t_est, tie, cpu_est, int(edge_peak > 0), v_cpu, v_peak)
                    if best_key is None or key < best_key:
                        best_key = key
                        best = {"policy": policy, "tiers": tiers, "rw_gpu": v_gpu, "t_step": t_est,
                                "t_model": t_model, "t_edge": t_edge}
                    if edge_peak == 0 and (best_np_key is None or key < best_np_key):
                        best_np_key, best_np = key, (policy, tiers)
            log[policy] = ("ok", policy_best * 1e3) if policy_best < float("inf") else ("skip:no_feasible_tier", None)
        self.last_plan_log = log
        self._edge_policy = best["policy"]
        self._best_nonpersistent_edge_policy, self._best_nonpersistent_tiers = best_np
        self._cache_edge = best["policy"] == EDGE_GPU_PERSIST
        self._rw_on_gpu = bool(best["rw_gpu"])
        self._set_modes(best["tiers"])
        self._state = self._ACTIVE
        parts = [f"{p}:{v[1]:.0f}ms{' [SELECTED]' if p == best['policy'] else ''}" if v[0] == "ok" else f"{p}:{v[0]}"
                 for p, v in log.items()]
        self._log(f"ACTIVE plan: edge_policy={best['policy']} rw_device={'GPU' if self._rw_on_gpu else 'auto'} "
                  f"tiers={self._tier_counts(best['tiers'])} peak_limit={peak_limit / 2**20:.0f} MiB "
                  f"est_T_step={best['t_step'] * 1e3 if best['t_step'] < float('inf') else 0:.0f} ms "
                  f"(model={best['t_model'] * 1e3:.0f} ms edge_prep={best['t_edge'] * 1e3:.0f} ms)")
        self._log("  policy candidates: " + " | ".join(parts))

    @staticmethod
    def _tier_counts(tiers) -> dict:
        out: Dict[str, int] = {}
        for t in tiers:
            out[t] = out.get(t, 0) + 1
        return out

    # ------------------------------------------------------------------ accessors
    def mode(self, layer_idx: int) -> str:
        return self._modes[layer_idx]

    def modes(self) -> List[str]:
        return list(self._modes)

    def is_active(self) -> bool:
        return self._state == self._ACTIVE

    def state_name(self) -> str:
        return self._STATE_NAMES[self._state]

    def needs_precise_timing(self) -> bool:
        return self._state not in (self._ACTIVE, self._DEFERRED)

    @property
    def cache_edge(self) -> bool:
        return self._cache_edge

    @property
    def edge_policy(self) -> str:
        return self._edge_policy

    @property
    def rw_on_gpu(self) -> bool:
        return self._rw_on_gpu

    @property
    def best_nonpersistent_edge_policy(self) -> str:
        return self._best_nonpersistent_edge_policy

    @property
    def best_nonpersistent_tiers(self) -> list:
        return list(self._best_nonpersistent_tiers)

    def override_cache_decision(self, cache: bool) -> None:
        self._cache_edge = bool(cache)
        if not cache and self._edge_policy == EDGE_GPU_PERSIST:
            self._edge_policy = self._best_nonpersistent_edge_policy
            self._set_modes(self._best_nonpersistent_tiers)

    def override_active_plan(self, edge_policy: str, modes: List[str]) -> None:
        """Install an externally agreed plan (cross-rank consensus or ``--force_multi_tier_plan``)."""
        if len(modes) != self.n_layers:
            raise ValueError(f"plan has {len(modes)} tiers for {self.n_layers} layers")
        for m in modes:
            if m not in TIER_IDS:
                raise ValueError(f"unknown tier {m!r}")
        self._edge_policy = str(edge_policy)
        self._cache_edge = edge_policy == EDGE_GPU_PERSIST
        self._set_modes(list(modes))
        self._state = self._ACTIVE
        self._log(f"ACTIVE plan (override): edge_policy={edge_policy} tiers={self._tier_counts(modes)}")

    # ------------------------------------------------------------------ runtime feedback
    def reconsider_with_actual_timing(self, device, t_model_actual: float, t_edge_wait_actual: float,
                                      gpu_policy_serial_s: Optional[float] = None) -> Optional[str]:
        """One-way CPU -> GPU switch: when the measured wait for a CPU-built graph exceeds what a GPU build
        would cost by more than 0.5 s, re-plan with the CPU policy's overlap replaced by the measurement
        (reference :1230-1379).  Returns the new policy name or ``None``."""
        if not self.is_active() or self._edge_policy not in (EDGE_CPU_RANK_LOCAL_PREFETCH, EDGE_CPU_BROADCAST_PREFETCH):
            return None
        cur = self._edge_profiles.get(self._edge_policy)
        if cur is None:
            return None
        gpu_candidates = [p for p in (EDGE_GPU_PERSIST, EDGE_GPU_EPHEMERAL)
                          if p in self._edge_profiles and p not in self._gpu_infeasible_policies]
        if not gpu_candidates:
            return None
        best_gpu = min(gpu_candidates, key=lambda p: self._edge_profiles[p]["serial_time_s"])
        gpu_cost = gpu_policy_serial_s if gpu_policy_serial_s is not None else self._edge_profiles[best_gpu]["serial_time_s"]
        if t_edge_wait_actual - gpu_cost <= _RECONSIDER_THRESHOLD_S:
            return None
        cur["overlap_time_s"] = float(t_model_actual + t_edge_wait_actual)
        old = self._edge_policy
        total = self._effective_total_gpu_bytes(self.probe.total(device))
        self._run_active_plan(device, total)
        if self._edge_policy != old:
            self._log(f"timing feedback: {old} waited {t_edge_wait_actual:.2f}s -> switched to {self._edge_policy}")
            return self._edge_policy
        return None

    def report_runtime_edge_gpu_infeasible(self, device) -> bool:
        """The GPU edge build fell back at run time: exclude GPU policies and re-plan (reference :1381-1431)."""
        changed = False
        for p in (EDGE_GPU_EPHEMERAL, EDGE_GPU_PERSIST):
            if p not in self._gpu_infeasible_policies:
                self._gpu_infeasible_policies.add(p)
                changed = True
        if changed and self.is_active():
            total = self._effective_total_gpu_bytes(self.probe.total(device))
            self._run_active_plan(device, total)
        return changed

    def mark_current_calibration_infeasible(self, device) -> bool:
        """A CALIBRATE_* step ran out of memory: disable that tier and move on (reference :1456-1517)."""
        s = self._state
        total = self._effective_total_gpu_bytes(self.probe.total(device)) if self.probe.available() else 0
        if s == self._CALIBRATE_MHA:
            self._t1_infeasible = True
            self._state = self._CALIBRATE_RETAIN
        elif s == self._CALIBRATE_MHA_FRONT:
            self._t1_nonlast_infeasible = True
            self._state = self._CALIBRATE_RETAIN
        elif s == self._CALIBRATE_RETAIN:
            self._t4_infeasible = True
            self._run_active_plan(device, total)
        elif s == self._CALIBRATE_RETAIN_FRONT:
            self._t4_nonlast_infeasible = True
            self._run_active_plan(device, total)
        else:
            return False
        self._log(f"calibration step ran out of memory -> {self.state_name()}")
        return True

    def apply_oom_fallback(self, device, sp_group=None, sp_world_size: int = 1) -> bool:
        """Demote one tier (retain -> keep_mha -> recompute, shallowest kept layer first) and make all
        ranks agree by taking the element-wise minimum tier (reference :1519-1562)."""
        ids = [TIER_IDS[m] for m in self._modes]
        for i, t in enumerate(ids):
            if t > 0:
                ids[i] = t - 1
                break
        else:
            if self._cache_edge:
                self.override_cache_decision(False)
                return True
            return False
        if sp_world_size > 1 and dist.is_initialized():
            dev = torch.device(device) if dist.get_backend(sp_group) == "nccl" else torch.device("cpu")
            t = torch.tensor(ids, dtype=torch.int64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=sp_group)
            ids = [int(x) for x in t.tolist()]
        self._set_modes([TIER_FROM_ID[i] for i in ids])
        self._log(f"OOM fallback -> tiers={self._tier_counts(self._modes)}")
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
