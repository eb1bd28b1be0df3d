"""Opt-in timing / byte / scalar registry for communication and edge-construction phases.

API and metric names follow the reference's ``gt_sp/comm_profiler.py`` (``enable_comm_profiler``
:14, ``profile_call`` :29, ``record_scalar`` :56, ``get_comm_profile_summary`` :78): CUDA-event pairs
on the current stream for GPU work, ``perf_counter`` on the host otherwise; events are resolved only
when a summary is requested, so recording never synchronises the device.
"""
from __future__ import annotations

import time
from typing import Callable, Dict

import torch

_ENABLED = False
_NVTX = False
_TIMES: Dict[str, dict] = {}
_SCALARS: Dict[str, float] = {}

KNOWN_PHASES = (
    "seq_all_to_all_fwd", "seq_all_to_all_bwd", "grad_all_reduce", "edge_broadcast", "edge_full_h2d",
    "edge_build_local", "edge_real_sample", "edge_rw_build", "edge_rw_sample", "edge_merge",
    "qkv_gemm_push", "ctx_pull_outproj", "edge_attention",
)


def enable_comm_profiler(enabled: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(enabled)


def comm_profiler_enabled() -> bool:
    return _ENABLED


def enable_nvtx(enabled: bool = True) -> None:
    """NVTX ranges around every ``profile_call`` and every ``nvtx_range`` (visible in Nsight timelines); independent of
    the timing registry, costs nothing when off."""
    global _NVTX
    _NVTX = bool(enabled) and torch.cuda.is_available()


class nvtx_range:
    """``with nvtx_range("fwd"): ...`` - a named range when NVTX output is enabled, otherwise a no-op."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _NVTX:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        return False


def reset_comm_profiler() -> None:
    _TIMES.clear()
    _SCALARS.clear()


def _slot(name: str) -> dict:
    s = _TIMES.get(name)
    if s is None:
        s = {"host_s": 0.0, "events": [], "count": 0, "bytes": 0}
        _TIMES[name] = s
    return s


def profile_call(name: str, fn: Callable, device=None, payload_bytes: int = 0):
    """Run ``fn()``; when profiling is on, time it under ``name``."""
    if not _ENABLED:
        if _NVTX:
            with nvtx_range(name):
                return fn()
        return fn()
    slot = _slot(name)
    dev = torch.device(device) if device is not None else None
    if dev is not None and dev.type == "cuda" and torch.cuda.is_available():
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record(torch.cuda.current_stream(dev))
        out = fn()
        end.record(torch.cuda.current_stream(dev))
        slot["events"].append((start, end))
    else:
        t0 = time.perf_counter()
        out = fn()
        slot["host_s"] += time.perf_counter() - t0
    slot["count"] += 1
    slot["bytes"] += int(payload_bytes)
    return out


def record_scalar(name: str, value, reduce: str = "last") -> None:
    if not _ENABLED:
        return
    v = float(value)
    if name not in _SCALARS or reduce == "last":
        _SCALARS[name] = v
    elif reduce == "sum":
        _SCALARS[name] += v
    elif reduce == "max":
        _SCALARS[name] = max(_SCALARS[name], v)
    else:
        raise ValueError(f"unknown reduce {reduce!r}")


def get_comm_profile_summary(reset: bool = False) -> dict:
    """``{name: {total_s, count, avg_s, bytes}}`` plus ``"scalars"``; synchronises once if GPU events exist."""
    if any(s["events"] for s in _TIMES.values()) and torch.cuda.is_available():
        torch.cuda.synchronize()
    out = {}
    for name, s in _TIMES.items():
        total = s["host_s"] + sum(a.elapsed_time(b) for a, b in s["events"]) / 1e3
        out[name] = {"total_s": total, "count": s["count"], "avg_s": total / max(1, s["count"]), "bytes": s["bytes"]}
    out["scalars"] = dict(_SCALARS)
    if reset:
        reset_comm_profiler()
    return out
