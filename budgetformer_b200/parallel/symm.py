"""Symmetric (peer-mapped) device memory and the collectives built on it.

``SymmWorld`` allocates buffers that every rank of the group can address directly over
NVLink / NVSwitch (``torch.distributed._symmetric_memory`` does the handle exchange; all data
movement is done by this package's kernels with peer loads/stores or NVSwitch ``multimem``
instructions).  It owns one flag page for ``barrier()`` — a device-side barrier with a bounded spin
whose expiry is reported through the status word checked by ``ops.gemm.check_status``.

With a world of one (single GPU) the same interface degenerates to ordinary tensors, so the fused
model path is identical at every scale.
"""
from __future__ import annotations

import os
from typing import Dict, List

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops.gemm import status_tensor
from . import comm

_WORLDS: Dict[int, "SymmWorld"] = {}
FLAG_CHANNELS = 64
MAX_PEERS = 8


class SymmBuffer:
    """One symmetric allocation: the local tensor plus every rank's mapped pointer."""

    def __init__(self, tensor: torch.Tensor, ptrs: List[int], multicast_ptr: int = 0, handle=None):
        self.tensor, self.ptrs, self.multicast_ptr, self.handle = tensor, ptrs, int(multicast_ptr), handle

    def nbytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()


class SymmWorld:
    def __init__(self, group, device):
        self.group = group
        self.device = torch.device(device)
        self.world = comm.group_size(group)
        self.rank = comm.group_rank(group)
        if self.world > MAX_PEERS:
            raise RuntimeError(f"symmetric-memory kernels support up to {MAX_PEERS} ranks, got {self.world}")
        self.bytes_allocated = 0
        # one counter per channel: a channel is driven by one host thread and sees the same sequence on every rank
        self._epochs = [0] * FLAG_CHANNELS
        self.use_multimem = os.environ.get("BF_DISABLE_MULTIMEM", "0") != "1"
        self._live = []                    # weak references to every buffer handed out (multicast_bound walks them)
        self.flags = self.alloc((FLAG_CHANNELS * MAX_PEERS,), torch.int32, zero=True)
        if self.world > 1:
            # every rank must have zeroed its flag page before anyone raises a flag in it
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)

    def alloc(self, shape, dtype, zero: bool = False) -> SymmBuffer:
        numel = 1
        for s in shape:
            numel *= int(s)
        numel = max(numel, 1)
        if self.world == 1:
            t = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=self.device)
            buf = SymmBuffer(t.view(*shape) if numel == t.numel() and shape else t, [t.data_ptr()], 0, None)
        else:
            import torch.distributed._symmetric_memory as symm_mem
            t = symm_mem.empty(numel, dtype=dtype, device=self.device)
            if zero:
                t.zero_()
            hdl = symm_mem.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            mc = int(hdl.multicast_ptr) if (self.use_multimem and hdl.multicast_ptr) else 0
            buf = SymmBuffer(t.view(*shape), ptrs, mc, hdl)
        self.bytes_allocated += buf.nbytes()
        import weakref
        self._live.append(weakref.ref(buf))
        return buf

    def multicast_bound(self) -> bool:
        """Is any live allocation of this world bound to an NVSwitch multicast object (whether or not the kernels use
        it)?  A rank must not leave the job while one is: ``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` before the first
        allocation keeps them unbound."""
        for ref in self._live:
            buf = ref()
            if buf is not None and buf.handle is not None and int(getattr(buf.handle, "multicast_ptr", 0) or 0) != 0:
                return True
        return False

    def barrier(self, channel: int = 0) -> None:
        """Device-side barrier over all ranks on the current stream (no host synchronisation)."""
        if self.world == 1:
            return
        self._epochs[channel] += 1
        # the kernel compares epochs by signed 32-bit distance, so the counter wraps over the full 32 bits
        _ext.load().peer_barrier(self.flags.ptrs, self.rank, int(channel), self._epochs[channel] & 0xFFFFFFFF,
                                 status_tensor(self.device))
        _ext.count_launches(1)

    def resync(self) -> None:
        """Bring every rank's barrier epoch back together after a step that some rank abandoned on the host (it issued
        fewer barriers than its peers, so its counters lag and its next barriers would pass at once on flags that are
        already ahead).  Drains this rank's queue (barriers still waiting for the rank that stopped give up after
        their bound; once the status word is set the remaining ones return immediately), clears the status word, takes
        the maximum counter over the ranks on the host and meets the others there."""
        if self.world == 1:
            return
        torch.cuda.synchronize(self.device)
        status_tensor(self.device).zero_()
        dev = comm.comm_device(self.group, self.device)
        self._epochs = [int(v) for v in comm.all_reduce_scalars([float(e) for e in self._epochs], "max", self.group, dev)]
        torch.cuda.synchronize(self.device)
        comm.barrier(self.group)


def get_world(group, device) -> SymmWorld:
    key = id(group) if group is not None else 0
    w = _WORLDS.get(key)
    if w is None or w.device != torch.device(device):
        w = SymmWorld(group, device)
        _WORLDS[key] = w
    return w


def reset_worlds() -> None:
    _WORLDS.clear()


def symmetric_bytes() -> int:
    """Bytes held in symmetric buffers by this process (outside PyTorch's caching allocator for world > 1);
    the execution planner adds them to its memory readings."""
    return sum(w.bytes_allocated for w in _WORLDS.values())


# ---- gradient buckets ------------------------------------------------------------------------------
def attach_buckets(buckets, group) -> bool:
    """Move the reducer's flat fp32 buckets into symmetric memory so that ``bucket_all_reduce_mean`` can run."""
    if not buckets or buckets[0].flat.device.type != "cuda" or comm.group_size(group) == 1:
        return False
    world = get_world(group, buckets[0].flat.device)
    # one array of squared-norm parts for all buckets: row i holds, after bucket i's all-reduce, the sum of squares of
    # the slice each rank reduced (unused slots stay zero), so the optimizer clips on the sum of the whole array
    parts = world.alloc((len(buckets) * MAX_PEERS,), torch.float32, zero=True)
    for i, b in enumerate(buckets):
        if b.flat.dtype != torch.float32:
            continue
        sb = world.alloc((b.flat.numel(),), torch.float32, zero=True)
        b.rebind_to(sb.tensor)
        b.symm = (world, sb)
        grid = int(_ext.load().allreduce_mean_grid(b.flat.numel(), world.world))
        b.norm = {"scratch": torch.zeros(grid + 1, dtype=torch.float32, device=b.flat.device),
                  "ptrs": [p + 4 * i * MAX_PEERS for p in parts.ptrs], "all": parts.tensor, "ready": False}
    if world.world > 1:
        torch.cuda.synchronize(world.device)
        dist.barrier(group=world.group)                # every rank's parts array is zero before anyone writes into it
    return True


def bucket_all_reduce_mean(bucket) -> None:
    """In-place mean over ranks of a symmetric fp32 bucket: barrier, fused scale + two-shot (or in-switch
    multimem) all-reduce, barrier."""
    world, sb = bucket.symm
    ext = _ext.load()
    norm = getattr(bucket, "norm", None)
    world.barrier(1)                       # every rank's gradients are complete
    ext.allreduce_mean(sb.ptrs, sb.multicast_ptr, world.rank, sb.tensor.numel(), sb.tensor,
                       norm["scratch"] if norm else None, norm["ptrs"] if norm else [])
    _ext.count_launches(1)
    world.barrier(1)                       # every slice (and every rank's norm part) has been written everywhere
    if norm:
        norm["ready"] = True
