"""Self-checks that stand in for a memory sanitizer on machines where none can be run.

Enabled by ``--debug_checks`` or ``BF_DEBUG=1``.  Three kinds of check, all on the host or with ordinary tensor ops
(nothing here can fault a GPU):

* ``validate_graph``: structural invariants of an attention graph before any kernel indexes with it (monotone row
  pointers, keys inside ``[0, n)``, consistent by-key view and work list);
* ``poison``: reusable symmetric buffers are filled with NaN once their consumer has read them, so a kernel that reads
  a buffer before its producer (a missing barrier, a stale epoch) propagates NaN instead of plausible numbers;
* ``assert_finite``: loss and gradient buckets are checked after every step and the step that introduced a NaN is named.

The reference has no counterpart (its race avoidance is structural: a synchronous reducer and a prefetch thread that
only touches CPU tensors, gt_sp/reducer.py:36-43, main_node_fullgraph_sp.py:512-521)."""
from __future__ import annotations

import os

import torch

_FORCED = None


def enable(on: bool = True) -> None:
    global _FORCED
    _FORCED = bool(on)


def enabled() -> bool:
    if _FORCED is not None:
        return _FORCED
    return os.environ.get("BF_DEBUG", "0") not in ("", "0", "false", "False")


def validate_graph(g) -> None:
    """Raise ``ValueError`` naming the first broken invariant of an ``AttnGraph`` (one host read per check)."""
    n, e = int(g.num_rows), int(g.col.numel())
    rp = g.rowptr.to(torch.int64)
    if rp.numel() != n + 1:
        raise ValueError(f"rowptr has {rp.numel()} entries for {n} rows")
    if n and (int(rp[0]) != 0 or int(rp[-1]) != e):
        raise ValueError(f"rowptr spans [{int(rp[0])}, {int(rp[-1])}] but there are {e} edges")
    if n and bool((rp[1:] < rp[:-1]).any()):
        raise ValueError("rowptr is not monotone")
    if e and (int(g.col.min()) < 0 or int(g.col.max()) >= n):
        raise ValueError(f"key ids outside [0, {n}): min {int(g.col.min())}, max {int(g.col.max())}")
    if g.max_degree is not None and n and int((rp[1:] - rp[:-1]).max()) > int(g.max_degree):
        raise ValueError("a query row is longer than the declared max_degree")
    if g.etype is not None and g.etype.numel() != e:
        raise ValueError("edge types do not match the edge count")
    if g.t_rowptr is not None:
        trp = g.t_rowptr.to(torch.int64)
        if trp.numel() != n + 1 or (n and (int(trp[0]) != 0 or int(trp[-1]) != e)) or bool((trp[1:] < trp[:-1]).any()):
            raise ValueError("by-key row pointers are inconsistent")
        if e:
            eid = g.t_eid.to(torch.int64)
            if int(eid.min()) < 0 or int(eid.max()) >= e or int(torch.unique(eid).numel()) != e:
                raise ValueError("by-key edge ids are not a permutation of the edges")
            keys = g.col.to(torch.int64)[eid]
            if bool((keys[1:] < keys[:-1]).any()):
                raise ValueError("by-key view is not grouped by key")
            if g.t_row is not None and not torch.equal(g.t_row.to(torch.int64), g.row_ids()[eid]):
                raise ValueError("by-key query ids do not match the edges")
        if g.t_task is not None and g.t_task.numel():
            t = g.t_task.to(torch.int64)
            if bool((t[:, 1] > t[:, 2]).any()) or int(t[:, 2].max()) > e or int(t[:, 0].max()) >= n:
                raise ValueError("dK/dV work items out of range")
            if int((t[:, 2] - t[:, 1]).sum()) != e:
                raise ValueError("dK/dV work items do not cover every edge exactly once")
            if int(t[:, 3].max()) >= max(int(g.kv_slots), 1) and int(t[:, 3].max()) >= 0:
                raise ValueError("partial slot index beyond the slot count")


def poison(t: torch.Tensor) -> None:
    """Fill a floating-point buffer with NaN (stream-ordered: enqueue it after the buffer's last consumer)."""
    if enabled() and t.is_floating_point():
        t.fill_(float("nan"))


def assert_finite(what: str, *tensors) -> None:
    if not enabled():
        return
    for t in tensors:
        if t is not None and t.is_floating_point() and not bool(torch.isfinite(t).all()):
            raise FloatingPointError(f"non-finite values in {what}")
