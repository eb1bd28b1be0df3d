"""Replicated-parameter synchronisation: initial broadcast and bucketed gradient averaging.

Behaviour of the reference's ``gt_sp/reducer.py`` (``sync_params_and_buffers`` :11-19,
``GradientReducer`` :35-156): parameters are replicated on every SP rank, each rank's loss is the
mean over its local training nodes, and gradients are averaged over ranks.  Differences:

* the initial sync packs the whole ``state_dict`` into one flat buffer per dtype (one broadcast
  instead of one per tensor);
* gradients live permanently inside flat fp32 buckets (``param.grad`` is a view), so there is no
  copy-in / copy-out around the collective;
* on GPUs with symmetric memory the bucket is reduced by a one-shot kernel that reads every peer's
  bucket over NVLink, applies the 1/P scale and writes the result (``parallel/symm.py``); otherwise a
  single ``all_reduce`` is issued.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.comm_profiler import profile_call
from . import comm
from .initialize import get_sequence_parallel_group, get_sequence_parallel_src_rank


def sync_params_and_buffers(model: torch.nn.Module, group=None, src: Optional[int] = None) -> None:
    group = group if group is not None else get_sequence_parallel_group()
    if comm.group_size(group) == 1:
        return
    src = get_sequence_parallel_src_rank() if src is None else src
    by_key: Dict[tuple, List[torch.Tensor]] = {}
    for t in model.state_dict().values():
        if isinstance(t, torch.Tensor) and t.numel() > 0:
            by_key.setdefault((t.device, t.dtype), []).append(t)
    for (_dev, _dt), tensors in by_key.items():
        flat = torch.cat([t.detach().reshape(-1) for t in tensors])
        dist.broadcast(flat, src=src, group=group)
        off = 0
        for t in tensors:
            n = t.numel()
            with torch.no_grad():
                t.copy_(flat[off:off + n].view_as(t))
            off += n


class _Bucket:
    ALIGN = 8                                      # elements: every tensor starts on a 16-byte boundary (fp32/16-bit)

    def __init__(self, params: List[torch.nn.Parameter], device, dtype):
        self.params = params
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.n_valid = off                         # padded slots stay zero and are harmless to reduce / update
        n_pad = (off + 1023) // 1024 * 1024
        self.flat = torch.zeros(n_pad, dtype=dtype, device=device)
        self.symm = None                           # filled by parallel.symm when available
        self._bind()

    def _bind(self):
        for p, off in zip(self.params, self.offsets):
            p.grad = self.flat[off:off + p.numel()].view_as(p)

    def rebind_to(self, flat: torch.Tensor):
        flat[: self.flat.numel()].copy_(self.flat)
        self.flat = flat
        self._bind()


class GradientReducer:
    """``prepare_backward()`` before ``loss.backward()``; ``finalize_backward()`` after it."""

    def __init__(self, model: torch.nn.Module, process_group=None, bucket_cap_mb: float = 25.0,
                 world_size: Optional[int] = None, use_symmetric_memory: bool = True):
        self.group = process_group if process_group is not None else get_sequence_parallel_group()
        self.world_size = int(world_size) if world_size else comm.group_size(self.group)
        self.buckets: List[_Bucket] = []
        cap = int(bucket_cap_mb * 1024 * 1024)
        params = [p for p in model.parameters() if p.requires_grad]
        cur: List[torch.nn.Parameter] = []
        cur_key, cur_bytes = None, 0
        for p in reversed(params):                 # reverse order ~ order in which backward produces grads
            key = (p.device, p.dtype)
            nbytes = p.numel() * p.element_size()
            if cur and (key != cur_key or cur_bytes + nbytes > cap):
                self.buckets.append(_Bucket(cur, cur_key[0], cur_key[1]))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_key = key
            cur_bytes += nbytes
        if cur:
            self.buckets.append(_Bucket(cur, cur_key[0], cur_key[1]))
        self._symm_ok = False
        if use_symmetric_memory and self.world_size > 1:
            self._try_enable_symmetric()

    def _try_enable_symmetric(self):
        try:
            from . import symm
            self._symm_ok = symm.attach_buckets(self.buckets, self.group)
        except Exception:
            self._symm_ok = False

    def prepare_backward(self) -> None:
        """Grads accumulate into the bucket views; they must start from zero every step."""
        for b in self.buckets:
            for p in b.params:
                if p.grad is None or p.grad.data_ptr() < b.flat.data_ptr() or \
                        p.grad.data_ptr() >= b.flat.data_ptr() + b.flat.numel() * b.flat.element_size():
                    b._bind()
                    break
            b.flat.zero_()
            if getattr(b, "norm", None) is not None:
                b.norm["ready"] = False

    def finalize_backward(self) -> None:
        if self.world_size <= 1:
            return
        for b in self.buckets:
            nbytes = b.flat.numel() * b.flat.element_size()
            if self._symm_ok and b.symm is not None:
                from . import symm
                profile_call("grad_all_reduce", lambda: symm.bucket_all_reduce_mean(b), device=b.flat.device,
                             payload_bytes=nbytes)
            else:
                def _run():
                    b.flat.div_(self.world_size)
                    dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group)
                profile_call("grad_all_reduce", _run, device=b.flat.device, payload_bytes=nbytes)

    def grad_views_ok(self) -> bool:
        return all(p.grad is not None for b in self.buckets for p in b.params)


def build_gradient_reducer(model, process_group=None, bucket_cap_mb: float = 25.0, world_size: Optional[int] = None,
                           use_symmetric_memory: bool = True) -> GradientReducer:
    return GradientReducer(model, process_group, bucket_cap_mb, world_size, use_symmetric_memory)
