"""Sequence-parallel autograd collectives and the distributed-attention wrappers.

Ulysses-style: activations are sharded by node (``N/P`` rows per rank); attention is sharded by
head after an all-to-all (nodes -> heads), and a second all-to-all brings the context back
(heads -> nodes).  Restates ``gt_sp/layer.py:29-153,235-281`` and ``gt_sp/gt_layer.py:30-139,209-253``
with a single-buffer all-to-all (the reference splits into P chunks, copies each, and concatenates
again: two extra full copies per call).

These framework-layer ops are the portable path (CPU/gloo, or NCCL as a baseline).  On B200 the
models replace "projection + all-to-all" by the fused kernels in ``ops/fused_sp.py``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from ..utils.comm_profiler import profile_call
from . import comm
from .initialize import get_global_token_indices, get_sequence_parallel_group


def _a2a_heads_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[b, s, H, d] (all heads, local nodes) -> [b, P*s, H/P, d] (local heads, all nodes)."""
    p = comm.group_size(group)
    b, s, h, d = x.shape
    send = x.reshape(b, s, p, h // p, d).permute(2, 0, 1, 3, 4).contiguous()
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send, group)
    return recv.permute(1, 0, 2, 3, 4).reshape(b, p * s, h // p, d)


def _a2a_seq_to_heads(x: torch.Tensor, group) -> torch.Tensor:
    """[b, P*s, Hl, d] -> [b, s, P*Hl, d]."""
    p = comm.group_size(group)
    b, ps, hl, d = x.shape
    s = ps // p
    send = x.reshape(b, p, s, hl, d).permute(1, 0, 2, 3, 4).contiguous()
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send, group)
    return recv.permute(1, 2, 0, 3, 4).reshape(b, s, p * hl, d)


class _SeqAllToAll(torch.autograd.Function):
    """``apply(group, x, scatter_idx, gather_idx)``; (2, 1) scatters heads / gathers nodes and (1, 2) is
    its inverse.  Backward is the same op with the indices swapped (gt_sp/layer.py:55-63)."""

    @staticmethod
    def forward(ctx, group, x, scatter_idx, gather_idx):
        ctx.group, ctx.scatter_idx, ctx.gather_idx = group, scatter_idx, gather_idx
        return _SeqAllToAll._run(group, x, scatter_idx, gather_idx, "seq_all_to_all_fwd")

    @staticmethod
    def _run(group, x, scatter_idx, gather_idx, name):
        if comm.group_size(group) == 1:
            return x
        squeeze = False
        if x.dim() == 3:                      # [b, s, h]: treat hidden as (heads=P, rest)
            squeeze = True
            p = comm.group_size(group)
            if scatter_idx == 2:
                x = x.reshape(x.size(0), x.size(1), p, -1)
            else:
                x = x.unsqueeze(2)
        nbytes = x.numel() * x.element_size()
        if scatter_idx == 2 and gather_idx == 1:
            fn = lambda: _a2a_heads_to_seq(x, group)
        elif scatter_idx == 1 and gather_idx == 2:
            fn = lambda: _a2a_seq_to_heads(x, group)
        else:
            raise ValueError(f"unsupported all-to-all axes scatter={scatter_idx} gather={gather_idx}")
        out = profile_call(name, fn, device=x.device, payload_bytes=nbytes)
        if squeeze:
            out = out.reshape(out.size(0), out.size(1), -1)
        return out

    @staticmethod
    def backward(ctx, grad):
        out = _SeqAllToAll._run(ctx.group, grad.contiguous(), ctx.gather_idx, ctx.scatter_idx, "seq_all_to_all_bwd")
        return None, out, None, None


class _SeqGather(torch.autograd.Function):
    """Forward all-gather along the node axis, backward slice (gt_sp/layer.py:66-110)."""

    @staticmethod
    def forward(ctx, group, x, dim=1):
        ctx.group, ctx.dim = group, dim
        p = comm.group_size(group)
        if p == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(p)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=dim)

    @staticmethod
    def backward(ctx, grad):
        p = comm.group_size(ctx.group)
        if p == 1:
            return None, grad, None
        r = comm.group_rank(ctx.group)
        return None, grad.chunk(p, dim=ctx.dim)[r].contiguous(), None


class _SeqScatter(torch.autograd.Function):
    """Forward slice of this rank's heads, backward all-gather (gt_sp/layer.py:113-153)."""

    @staticmethod
    def forward(ctx, group, x, dim=2):
        ctx.group, ctx.dim = group, dim
        p = comm.group_size(group)
        if p == 1:
            return x
        assert x.size(dim) % p == 0, "head count must be divisible by the sequence-parallel size"
        return x.chunk(p, dim=dim)[comm.group_rank(group)].contiguous()

    @staticmethod
    def backward(ctx, grad):
        p = comm.group_size(ctx.group)
        if p == 1:
            return None, grad, None
        parts = [torch.empty_like(grad) for _ in range(p)]
        dist.all_gather(parts, grad.contiguous(), group=ctx.group)
        return None, torch.cat(parts, dim=ctx.dim), None


def copy_global_token0(x: torch.Tensor, token_rows) -> torch.Tensor:
    """Overwrite every per-rank copy of the virtual node with row ``token_rows[0]``
    (gt_sp/utils.py:2365-2386).  Differentiable: gradients of the copies sum into row 0."""
    if token_rows is None or len(token_rows) <= 1:
        return x
    idx = torch.as_tensor(list(token_rows[1:]), device=x.device, dtype=torch.long)
    src = x[:, token_rows[0]:token_rows[0] + 1]
    return x.index_copy(1, idx, src.expand(-1, idx.numel(), *([-1] * (x.dim() - 2))))


class DistributedAttentionNodeLevel(nn.Module):
    """GT / GraphGPS / Exphormer wrapper (gt_sp/gt_layer.py:209-253): q, k, v all-to-all (heads
    scattered, nodes gathered), local attention on ``H/P`` heads over all nodes, reverse all-to-all."""

    def __init__(self, local_attention: nn.Module, sequence_process_group=None, scatter_idx: int = 2, gather_idx: int = 1):
        super().__init__()
        self.local_attn = local_attention
        self.spg = sequence_process_group
        self.scatter_idx, self.gather_idx = scatter_idx, gather_idx

    def _group(self):
        return self.spg if self.spg is not None else get_sequence_parallel_group()

    def forward(self, query, key, value, attn_bias=None, edge_index=None, attn_type=None, **kw):
        g = self._group()
        q = _SeqAllToAll.apply(g, query, self.scatter_idx, self.gather_idx)
        k = _SeqAllToAll.apply(g, key, self.scatter_idx, self.gather_idx)
        v = _SeqAllToAll.apply(g, value, self.scatter_idx, self.gather_idx)
        if attn_bias is not None and comm.group_size(g) > 1:
            attn_bias = _SeqAllToAll.apply(g, attn_bias, 1, 2)
        ctx = self.local_attn(q, k, v, attn_bias, edge_index, attn_type, **kw)
        return _SeqAllToAll.apply(g, ctx, self.gather_idx, self.scatter_idx)


class DistributedAttentionNoMerge(DistributedAttentionNodeLevel):
    """Graphormer wrapper (gt_sp/layer.py:235-281): same as above, and every rank's copy of the virtual
    node is overwritten with copy 0's attention output before the reverse all-to-all."""

    def forward(self, query, key, value, attn_bias=None, edge_index=None, attn_type=None, **kw):
        g = self._group()
        q = _SeqAllToAll.apply(g, query, self.scatter_idx, self.gather_idx)
        k = _SeqAllToAll.apply(g, key, self.scatter_idx, self.gather_idx)
        v = _SeqAllToAll.apply(g, value, self.scatter_idx, self.gather_idx)
        if attn_bias is not None and comm.group_size(g) > 1:
            attn_bias = _SeqAllToAll.apply(g, attn_bias, 1, 2)
        ctx = self.local_attn(q, k, v, attn_bias, edge_index, attn_type, **kw)
        if comm.group_size(g) > 1:
            ctx = copy_global_token0(ctx, get_global_token_indices())
        return _SeqAllToAll.apply(g, ctx, self.gather_idx, self.scatter_idx)
