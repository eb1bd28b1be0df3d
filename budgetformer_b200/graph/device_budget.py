"""Where the per-epoch edge build runs: device resolution and the "does it fit on the GPU" decision.

Counterpart of the device-decision state of the reference's edge library (gt_sp/utils.py:133-157
``resolve_edge_build_device``; :243-322 memory cap, planner override and the sticky "GPU build failed" registry;
:325-487 ``_gpu_concurrent_overhead_bytes`` / ``_rw_gpu_usable_bytes`` / ``_gpu_can_fit_rw`` / ``_safe_rw_device``).
The rules:

* usable = driver-reported free memory (+ the allocator's reserved-but-unallocated slack when expandable segments
  are on and the driver still has at least 256 MiB to grow into), clamped to ``cap - reserved`` when a per-process
  cap is registered (the driver does not know about it), minus 512 MiB for library handles and workspaces;
* a planner that profiled a GPU build as feasible can force the answer to "fits" (a real out-of-memory error is
  still caught where the build runs);
* a build that failed at run time is remembered per (device, edge count) for the rest of the run, so that it is not
  retried every epoch.

The state lives in one ``DeviceBuildBudget`` object (``BUDGET`` is the process-wide one); the memory probe is
injectable, which is how the rules are tested without a GPU.
"""
from __future__ import annotations

import os
from typing import Callable, Optional, Set, Tuple

import torch

LIBRARY_OVERHEAD_BYTES = 512 * 2 ** 20
MIN_DRIVER_FREE_FOR_SLACK = 256 * 2 ** 20

# (free, reserved, allocated) in bytes, or None when no limit applies (not a CUDA device)
Probe = Callable[[torch.device], Optional[Tuple[int, int, int]]]


def expandable_segments_enabled() -> bool:
    return "expandable_segments:true" in os.environ.get("PYTORCH_CUDA_ALLOC_CONF", "").lower()


def _cuda_probe(device: torch.device) -> Optional[Tuple[int, int, int]]:
    if device.type != "cuda" or not torch.cuda.is_available():
        return None
    try:
        free, _total = torch.cuda.mem_get_info(device)
        return int(free), int(torch.cuda.memory_reserved(device)), int(torch.cuda.memory_allocated(device))
    except (RuntimeError, AttributeError):
        return None


def resolve_edge_build_device(args, default_device) -> torch.device:
    """``--edge_build_device``: ``gpu`` (or the old alias ``same``) = the training device, ``cpu``, ``cuda`` = the
    training device's index (or the current device), ``cuda:N``."""
    spec = getattr(args, "edge_build_device", "gpu")
    default = torch.device(default_device)
    if spec in (None, "", "gpu", "same"):
        return default
    try:
        dev = torch.device(spec)
    except (TypeError, RuntimeError) as exc:
        raise ValueError(f"invalid --edge_build_device={spec!r}; expected gpu, cpu, cuda or cuda:N") from exc
    if dev.type == "cuda":
        if not torch.cuda.is_available():
            raise ValueError("--edge_build_device asks for CUDA, but CUDA is not available")
        if dev.index is None:
            index = default.index if default.type == "cuda" and default.index is not None else torch.cuda.current_device()
            return torch.device("cuda", index)
    return dev


class DeviceBuildBudget:
    def __init__(self, probe: Probe = _cuda_probe):
        self.probe = probe
        self.cap_bytes = 0                    # per-process allocator cap; 0 = none
        self.force_gpu = False                # planner override
        self._infeasible: Set[Tuple[str, int]] = set()
        self._logged: Set[tuple] = set()

    # ---- registered state -------------------------------------------------------------------------
    def set_gpu_memory_cap(self, cap_bytes: int) -> None:
        self.cap_bytes = max(0, int(cap_bytes))

    def set_force_gpu_build(self, value: bool) -> None:
        self.force_gpu = bool(value)

    def mark_infeasible(self, device, num_edges: int) -> None:
        self._infeasible.add((str(torch.device(device)), int(num_edges)))

    def is_infeasible(self, device, num_edges: int) -> bool:
        return (str(torch.device(device)), int(num_edges)) in self._infeasible

    def any_infeasible(self) -> bool:
        return bool(self._infeasible)

    def reset(self) -> None:
        self.cap_bytes, self.force_gpu = 0, False
        self._infeasible.clear()
        self._logged.clear()

    def clear_decision_log(self) -> None:
        """Forget which decisions were already printed (called before the policies are profiled again)."""
        self._logged.clear()

    # ---- the decision -----------------------------------------------------------------------------
    def usable_bytes(self, device) -> int:
        """Bytes a build may take on ``device``; ``-1`` when no GPU limit applies."""
        m = self.probe(torch.device(device))
        if m is None:
            return -1
        free, reserved, allocated = m
        if expandable_segments_enabled() and free >= MIN_DRIVER_FREE_FOR_SLACK:
            free += max(0, reserved - allocated)
        if self.cap_bytes > 0:
            free = min(free, max(0, self.cap_bytes - reserved))
        return max(0, free - LIBRARY_OVERHEAD_BYTES)

    def can_fit(self, device, need_bytes: int) -> bool:
        usable = self.usable_bytes(device)
        if usable < 0:
            return True
        return True if self.force_gpu else int(need_bytes) <= usable

    def safe_build_device(self, requested, need_bytes: int, num_edges: int = 0, log=None) -> torch.device:
        """``requested`` when the build fits there (or it is not a GPU), else the CPU; the reason is logged once per
        (device, edge count)."""
        dev = torch.device(requested)
        if dev.type != "cuda":
            return dev
        if not self.is_infeasible(dev, num_edges) and self.can_fit(dev, need_bytes):
            return dev
        key = (str(dev), int(num_edges))
        if log is not None and key not in self._logged:
            why = "failed earlier in this run" if self.is_infeasible(dev, num_edges) else \
                f"estimated working set {need_bytes / 2 ** 20:.0f} MiB exceeds the usable {self.usable_bytes(dev) / 2 ** 20:.0f} MiB"
            log(f"[edge-device] GPU build on {dev} skipped ({why}; edges={int(num_edges):,}); building on the CPU")
        self._logged.add(key)
        return torch.device("cpu")


BUDGET = DeviceBuildBudget()

# module-level spellings of the process-wide object
set_gpu_memory_cap = BUDGET.set_gpu_memory_cap
set_force_gpu_build = BUDGET.set_force_gpu_build
mark_gpu_build_infeasible = BUDGET.mark_infeasible
gpu_build_infeasible = BUDGET.is_infeasible
gpu_build_infeasible_any = BUDGET.any_infeasible
gpu_can_fit = BUDGET.can_fit
gpu_usable_bytes = BUDGET.usable_bytes
