"""Edge-build device resolution and the GPU-fit decision (graph/device_budget.py) with a fake memory probe."""
import types

import pytest
import torch

from budgetformer_b200.graph import device_budget as db

GIB = 2 ** 30


def _budget(free, reserved=0, allocated=0):
    return db.DeviceBuildBudget(probe=lambda dev: (free, reserved, allocated) if dev.type == "cuda" else None)


def test_usable_bytes_subtracts_library_overhead_and_respects_the_cap(monkeypatch):
    monkeypatch.delenv("PYTORCH_CUDA_ALLOC_CONF", raising=False)
    b = _budget(10 * GIB, reserved=3 * GIB, allocated=1 * GIB)
    assert b.usable_bytes("cuda:0") == 10 * GIB - db.LIBRARY_OVERHEAD_BYTES
    assert b.usable_bytes("cpu") == -1 and b.can_fit("cpu", 10 ** 15)
    b.set_gpu_memory_cap(5 * GIB)                         # headroom = cap - reserved = 2 GiB
    assert b.usable_bytes("cuda:0") == 2 * GIB - db.LIBRARY_OVERHEAD_BYTES
    assert b.can_fit("cuda:0", 1 * GIB) and not b.can_fit("cuda:0", 2 * GIB)
    b.set_gpu_memory_cap(2 * GIB)                         # cap already exceeded by what is reserved
    assert b.usable_bytes("cuda:0") == 0
    # reserved-but-unallocated slack counts only with expandable segments and a driver that can still grow
    monkeypatch.setenv("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    b.set_gpu_memory_cap(0)
    assert b.usable_bytes("cuda:0") == 12 * GIB - db.LIBRARY_OVERHEAD_BYTES
    tight = _budget(100 * 2 ** 20, reserved=3 * GIB, allocated=1 * GIB)
    assert tight.usable_bytes("cuda:0") == 0


def test_planner_override_and_sticky_failures():
    logs = []
    b = _budget(1 * GIB)
    assert b.safe_build_device("cuda:0", 4 * GIB, 1000, log=logs.append) == torch.device("cpu")
    assert b.safe_build_device("cuda:0", 4 * GIB, 1000, log=logs.append) == torch.device("cpu")
    assert len(logs) == 1 and "exceeds" in logs[0]                       # logged once per (device, edge count)
    b.set_force_gpu_build(True)
    assert b.safe_build_device("cuda:0", 4 * GIB, 1000) == torch.device("cuda:0")
    b.mark_infeasible("cuda:0", 1000)                                    # observed failure beats the override
    assert b.is_infeasible("cuda:0", 1000) and not b.is_infeasible("cuda:0", 999) and b.any_infeasible()
    b.clear_decision_log()
    assert b.safe_build_device("cuda:0", 1, 1000, log=logs.append) == torch.device("cpu")
    assert "failed earlier" in logs[-1]
    assert b.safe_build_device("cuda:0", 1, 999) == torch.device("cuda:0")
    assert b.safe_build_device("cpu", 10 ** 15) == torch.device("cpu")
    b.reset()
    assert not b.any_infeasible() and not b.force_gpu and b.cap_bytes == 0


def test_resolve_edge_build_device():
    ns = lambda v: types.SimpleNamespace(edge_build_device=v)
    assert db.resolve_edge_build_device(ns("gpu"), "cpu") == torch.device("cpu")
    assert db.resolve_edge_build_device(ns("same"), "cuda:3") == torch.device("cuda:3")
    assert db.resolve_edge_build_device(ns("cpu"), "cuda:3") == torch.device("cpu")
    assert db.resolve_edge_build_device(types.SimpleNamespace(), "cuda:1") == torch.device("cuda:1")
    with pytest.raises(ValueError):
        db.resolve_edge_build_device(ns("tpu:0!"), "cpu")
    if not torch.cuda.is_available():
        with pytest.raises(ValueError):
            db.resolve_edge_build_device(ns("cuda"), "cpu")


def test_engine_skips_the_driver_query_without_cap_or_failure():
    from budgetformer_b200.graph.engine import EdgeEngine, resolve_budget_state
    from budgetformer_b200.config import parse_fullgraph_args as parse_args
    args = parse_args(["--dataset", "x", "--model", "gt", "--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4"])
    n = 64
    s = torch.arange(n)
    eng = EdgeEngine(args, torch.stack([s, (s + 1) % n]), n, "cpu", nodes_per_rank=n)
    try:
        db.BUDGET.reset()
        assert eng._gpu_build_ruled_out(resolve_budget_state(args)) is False
        db.BUDGET.mark_infeasible("cpu", eng.topo_cpu.num_edges)          # CPU "device": never ruled out
        assert eng._gpu_build_ruled_out(resolve_budget_state(args)) is False
    finally:
        db.BUDGET.reset()
        eng.shutdown()
