"""Backend-neutral collectives used by the framework layer.

NCCL and gloo are reached through ``torch.distributed``.  gloo has no native all-to-all on some
builds, so ``all_to_all_single`` falls back to paired ``isend/irecv`` there — this is what makes
the 2-rank CPU configuration work, which the reference cannot run at all
(gt_sp/initialize.py:53 asserts a GPU before creating the process group).
The fused GPU paths (``parallel/symm.py``) bypass this module and move data with in-kernel peer stores.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_A2A_NATIVE_OK = {}
_CONTROL_TWIN = {}          # id of a device (NCCL) group, 0 for the default group -> host-side (gloo) group of the same ranks


def _key(group) -> int:
    return 0 if group is None or group is dist.group.WORLD else id(group)


def register_control_group(group, host_group) -> None:
    """Pair a device group with a host-side group of the same ranks.  Control scalars (votes, plan consensus, timing
    maxima) then travel over the host group: a vote costs a loopback round trip and never waits for the GPU queue,
    where an NCCL all-reduce followed by ``.item()`` drains the stream on every call."""
    if host_group is None:
        _CONTROL_TWIN.pop(_key(group), None)
    else:
        _CONTROL_TWIN[_key(group)] = host_group


def control_group(group):
    return _CONTROL_TWIN.get(_key(group)) if dist.is_initialized() else None


def _route(group, device):
    """(group, device) a control tensor should use."""
    twin = control_group(group)
    if twin is not None:
        return twin, torch.device("cpu")
    return group, device


def group_size(group) -> int:
    if not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if not dist.is_initialized():
        return 0
    return dist.get_rank(group)


def all_to_all_single(out: torch.Tensor, inp: torch.Tensor, group=None) -> None:
    """Equal-split all-to-all over dim 0 (``inp``/``out`` are ``[P, ...]`` contiguous)."""
    p = group_size(group)
    if p == 1:
        out.copy_(inp)
        return
    backend = dist.get_backend(group)
    key = (backend, inp.device.type)
    if _A2A_NATIVE_OK.get(key, True):
        try:
            dist.all_to_all_single(out, inp, group=group)
            _A2A_NATIVE_OK[key] = True
            return
        except (RuntimeError, NotImplementedError):
            _A2A_NATIVE_OK[key] = False
    me = dist.get_rank(group)
    out[me].copy_(inp[me])
    reqs = []
    for off in range(1, p):
        dst = (me + off) % p
        src = (me - off) % p
        reqs.append(dist.isend(inp[dst], dist.get_global_rank(group, dst) if group is not None else dst, group=group))
        reqs.append(dist.irecv(out[src], dist.get_global_rank(group, src) if group is not None else src, group=group))
    for r in reqs:
        r.wait()


def all_reduce_scalar(value: float, op: str = "max", group=None, device="cpu") -> float:
    """Control-plane reduction of one python scalar (host round trip by design)."""
    if group_size(group) == 1:
        return float(value)
    group, device = _route(group, device)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "sum": dist.ReduceOp.SUM}[op], group=group)
    return float(t.item())


def all_reduce_scalars(values, op: str = "max", group=None, device="cpu"):
    """Several control scalars in one collective (the reference issues one blocking call per vote)."""
    vals = [float(v) for v in values]
    if group_size(group) == 1 or not vals:
        return vals
    group, device = _route(group, device)
    t = torch.tensor(vals, dtype=torch.float64, device=device)
    dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "sum": dist.ReduceOp.SUM}[op], group=group)
    return [float(x) for x in t.tolist()]


def comm_device(group, default) -> torch.device:
    """Device a control tensor must live on for this group's backend (CPU when the group has a host-side twin)."""
    if control_group(group) is not None:
        return torch.device("cpu")
    if dist.is_initialized() and dist.get_backend(group) == "nccl":
        return torch.device(default if str(default).startswith("cuda") else f"cuda:{torch.cuda.current_device()}")
    return torch.device("cpu")


def barrier(group=None) -> None:
    """Host rendezvous of the group's ranks (over the host-side twin when there is one: no device work is queued)."""
    if group_size(group) > 1:
        twin = control_group(group)
        dist.barrier(group=twin if twin is not None else group)


def broadcast(t: torch.Tensor, src: int, group=None) -> None:
    if group_size(group) > 1:
        dist.broadcast(t, src=src, group=group)
