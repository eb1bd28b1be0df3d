"""Budgeted sparse edge attention.

For every edge ``(j -> i)`` of the attention graph and every local head::

    s = clamp(<q_i, k_j> / sqrt(hn) [elementwise * E_type], -5, 5)       w = exp(s)
    out_i = sum_j w * v_j / (sum_j w + 1e-6)

which is the reference's un-normalised clamp-exp softmax
(models/graphormer_dist_node_level.py:231-263, models/gt_dist_node_level.py:224-262).
Variants: ``"gps"`` normalises per edge and applies dropout to the normalised weights
(models/graphgps_dist_node_level.py:151-177); ``"exphormer"`` modulates the score with a
2-row edge-type table (models/exphormer_dist_node_level.py:92-121).  The clamp's gradient is
zero outside (-5, 5) and a query with no in-edges outputs 0.

Two implementations share this module:

* ``edge_attention_reference`` — plain differentiable PyTorch (any device/dtype); this is
  the numerics oracle and the CPU path.
* ``edge_attention`` — dispatches to the sm_100a kernels (forward, dQ pass over queries,
  dK/dV pass over the transposed graph; no atomics on regular rows) whenever the inputs live
  on a GPU, and raises if the extension is missing there.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..graph.attn_graph import AttnGraph

EPS = 1e-6
CLAMP = 5.0


def dropout_keep_mask(seed: int, eid: torch.Tensor, head: torch.Tensor, p: float) -> torch.Tensor:
    """Counter-based keep mask shared with the CUDA kernels: one 32-bit mix of (seed, edge, head)."""
    x = (eid.to(torch.int64) * 0x9E3779B1 + head.to(torch.int64) * 0x85EBCA77 + (int(seed) & 0xFFFFFFFF)) & 0xFFFFFFFF
    x = (x ^ (x >> 16)) * 0x7FEB352D & 0xFFFFFFFF
    x = (x ^ (x >> 15)) * 0x846CA68B & 0xFFFFFFFF
    x = x ^ (x >> 16)
    thresh = int(p * 4294967296.0)
    return x >= thresh


def edge_attention_reference(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    graph: AttnGraph,
    *,
    variant: str = "plain",
    etable: Optional[torch.Tensor] = None,
    edge_bias: Optional[torch.Tensor] = None,
    dropout_p: float = 0.0,
    dropout_seed: int = 0,
    return_z: bool = False,
):
    """q, k, v: ``[n, Hl, hn]``.  ``etable``: ``[T, Hl, hn]`` (Exphormer).  ``edge_bias``: ``[E, Hl]``
    added after the clamp (Graphormer, only when a bias tensor exists)."""
    n, hl, hn = q.shape
    src = graph.col.to(torch.int64)
    dst = graph.row_ids()
    scale = 1.0 / math.sqrt(hn)
    kq = k.float()[src] * q.float()[dst] * scale
    if variant == "exphormer" and etable is not None and graph.etype is not None:
        kq = kq * etable.float()[graph.etype.to(torch.int64)]
    s = kq.sum(-1).clamp(-CLAMP, CLAMP)
    if edge_bias is not None:
        s = s + edge_bias.float()
    w = torch.exp(s)                                        # [E, Hl]
    z = torch.zeros(n, hl, dtype=torch.float32, device=q.device).index_add_(0, dst, w)
    if variant == "gps":
        a = w / (z[dst] + EPS)
        if dropout_p > 0.0:
            eid = torch.arange(src.numel(), device=q.device)
            heads = torch.arange(hl, device=q.device)
            keep = dropout_keep_mask(dropout_seed, eid[:, None], heads[None, :], dropout_p)
            a = a * keep.to(a.dtype) / (1.0 - dropout_p)
        out = torch.zeros(n, hl, hn, dtype=torch.float32, device=q.device).index_add_(
            0, dst, a.unsqueeze(-1) * v.float()[src])
    else:
        num = torch.zeros(n, hl, hn, dtype=torch.float32, device=q.device).index_add_(
            0, dst, w.unsqueeze(-1) * v.float()[src])
        out = num / (z.unsqueeze(-1) + EPS)
    out = out.to(q.dtype)
    return (out, z) if return_z else out


class _EdgeAttentionCUDA(torch.autograd.Function):
    """sm_100a kernels; see csrc/edge_attn.cu."""

    @staticmethod
    def forward(ctx, q, k, v, etable, graph, variant_id, dropout_p, dropout_seed):
        from . import _ext
        ext = _ext.load()
        n, hl, hn = q.shape
        out = torch.empty((n, hl, hn), dtype=q.dtype, device=q.device)
        z = torch.empty((n, hl), dtype=torch.float32, device=q.device)
        kmax = -1 if graph.max_degree is None else int(graph.max_degree)
        ext.edge_attn_fwd(q, k, v, out, z, graph.rowptr, graph.col, graph.etype,
                          etable, int(variant_id), float(dropout_p), int(dropout_seed), kmax, [], [])
        _ext.count_launches(1)
        ctx.save_for_backward(q, k, v, out, z, etable if etable is not None else q.new_empty(0))
        ctx.graph = graph
        ctx.cfg = (int(variant_id), float(dropout_p), int(dropout_seed), etable is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import _ext
        ext = _ext.load()
        q, k, v, out, z, etable = ctx.saved_tensors
        variant_id, dropout_p, dropout_seed, has_tab = ctx.cfg
        graph = ctx.graph.ensure_transpose()
        dout = dout.contiguous()
        dq = torch.empty_like(out)
        dk = torch.empty_like(out)
        dv = torch.empty_like(out)
        zd = torch.empty(z.shape + (2,), dtype=torch.float32, device=q.device)
        detab = torch.zeros(etable.shape, dtype=torch.float32, device=q.device) if has_tab else None
        kmax = -1 if graph.max_degree is None else int(graph.max_degree)
        ext.edge_attn_bwd(q, k, v, out, z, dout, dq, dk, dv, zd,
                          graph.rowptr, graph.col, graph.etype,
                          graph.t_rowptr, graph.t_row, graph.t_eid,
                          etable if has_tab else None, detab,
                          variant_id, dropout_p, dropout_seed, kmax, graph.t_task, graph.t_split, int(graph.kv_slots), [], [])
        _ext.count_launches(3)
        return dq, dk, dv, (detab.to(etable.dtype) if has_tab else None), None, None, None, None


_VARIANTS = {"plain": 0, "gps": 1, "exphormer": 2}


def edge_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    graph: AttnGraph,
    *,
    variant: str = "plain",
    etable: Optional[torch.Tensor] = None,
    edge_bias: Optional[torch.Tensor] = None,
    dropout_p: float = 0.0,
    dropout_seed: int = 0,
) -> torch.Tensor:
    """``[n, Hl, hn]`` context.  GPU tensors in bf16/fp16/fp32 take the CUDA kernels."""
    use_cuda = q.is_cuda and edge_bias is None and q.shape[-1] in (8, 16, 32, 64, 128) \
        and q.dtype in (torch.bfloat16, torch.float16, torch.float32)
    if not use_cuda:
        return edge_attention_reference(q, k, v, graph, variant=variant, etable=etable, edge_bias=edge_bias,
                                        dropout_p=dropout_p, dropout_seed=dropout_seed)
    if variant == "exphormer" and (etable is None or graph.etype is None):
        variant = "plain"
    tab = etable.to(torch.float32).contiguous() if (variant == "exphormer") else None
    return _EdgeAttentionCUDA.apply(q, k, v, tab, graph, _VARIANTS[variant], float(dropout_p), int(dropout_seed))
