"""Evaluation helpers of the mini-batch mode (gt_sp/evaluate.py in the reference: ``calc_acc`` :11,
``sparse_eval_gpu`` :341-404 and its CPU / subset-batch variants)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..parallel.initialize import get_sequence_parallel_group, get_sequence_parallel_rank, get_sequence_parallel_world_size
from .legacy_batch import get_batch_blockize


def calc_acc(y: torch.Tensor, pred: torch.Tensor) -> float:
    if y.numel() == 0:
        return 0.0
    if pred.dim() > 1:
        pred = pred.argmax(dim=-1)
    return float((pred.reshape(-1).cpu() == y.reshape(-1).cpu()).float().mean())


@torch.no_grad()
def sparse_eval_subset_batch(args, model, feature, y, idx: torch.Tensor, edge_index_global, num_nodes: int, device,
                             batch_size: Optional[int] = None, topo=None) -> float:
    """Accuracy over ``idx`` evaluated sequence by sequence with the sparse attention graph of each sequence."""
    model.eval()
    p, r = get_sequence_parallel_world_size(), get_sequence_parallel_rank()
    bs = int(batch_size or getattr(args, "seq_len", 0) or idx.numel())
    correct, total = 0.0, 0.0
    for batch in torch.split(idx, bs):
        x_i, y_i, graph, bias, ok = get_batch_blockize(args, feature, y, batch, edge_index_global, num_nodes, r, p, topo=topo)
        out = model(x_i.to(device), None if bias is None else bias.to(device), graph.to(device), attn_type=args.attn_type)
        pred = out.argmax(1).cpu()
        m = ok & (y_i >= 0)
        correct += float((pred[m] == y_i[m]).sum())
        total += float(m.sum())
    if p > 1:
        t = torch.tensor([correct, total], dtype=torch.float64,
                         device=device if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(t, group=get_sequence_parallel_group())
        correct, total = t.tolist()
    model.train()
    return correct / max(total, 1.0)


def sparse_eval_gpu(args, model, feature, y, idx, edge_index_global, num_nodes, device, topo=None) -> float:
    return sparse_eval_subset_batch(args, model, feature, y, idx, edge_index_global, num_nodes, device, topo=topo)


def sparse_eval_cpu_subset_batch(args, model, feature, y, idx, edge_index_global, num_nodes, batch_size=None) -> float:
    return sparse_eval_subset_batch(args, model.to("cpu"), feature, y, idx, edge_index_global, num_nodes, "cpu", batch_size)


@torch.no_grad()
def eval_cpu_fullgraph(args, model, feature, y, idx, edge_index_global, num_nodes) -> float:
    """Whole graph as a single sequence on the CPU (small graphs only)."""
    return sparse_eval_subset_batch(args, model.to("cpu"), feature, y, torch.arange(num_nodes), edge_index_global, num_nodes,
                                    "cpu", batch_size=num_nodes) if idx is None else \
        sparse_eval_subset_batch(args, model.to("cpu"), feature, y, idx, edge_index_global, num_nodes, "cpu", batch_size=idx.numel())


@torch.no_grad()
def collect_hop_stats(args, model, feature, y, idx, edge_index_global, num_nodes: int, device, epoch: int, topo=None):
    """``--full_attn_hop_stats``: how the attention mass of every layer spreads over hop distance, on the first
    validation sequences of the epoch (main_node_sp.py:494-540 in the reference).  For a sample of query nodes the hop
    distance of every key is found by BFS over the sequence's own edges; the core attention modules accumulate the
    normalised edge weights per hop while the model runs; rank 0 writes one JSON file per epoch."""
    from ..utils import analytics
    cores = list(model.core_attention_modules())
    if not cores:
        return None
    p, r = get_sequence_parallel_world_size(), get_sequence_parallel_rank()
    max_q = int(getattr(args, "full_attn_hop_max_queries", 64))
    max_hop = int(getattr(args, "full_attn_hop_max_hop", 64))
    max_batches = max(1, int(getattr(args, "full_attn_hop_max_batches", 1)))
    for c in cores:
        c.enable_hop_mass_tracking(float(getattr(args, "full_attn_hop_mass", 0.95)), max_q,
                                   str(getattr(args, "full_attn_hop_query_sampling", "random")), max_batches, max_hop)
    model.eval()
    bs = int(getattr(args, "seq_len", 0) or idx.numel())
    gen = torch.Generator().manual_seed(int(args.seed) + int(epoch))
    try:
        for b, batch in enumerate(torch.split(idx, bs)):
            if b >= max_batches:
                break
            x_i, y_i, graph, bias, ok = get_batch_blockize(args, feature, y, batch, edge_index_global, num_nodes, r, p, topo=topo)
            ei = graph.edge_index()[:2].cpu()
            n_seq = graph.num_rows
            if str(getattr(args, "full_attn_hop_query_sampling", "random")) == "random":
                queries = torch.randperm(n_seq, generator=gen)[:max_q]
            else:
                queries = torch.arange(min(max_q, n_seq))
            dist_q = analytics.bfs_hop_matrix(ei, n_seq, queries, max_hop)          # [Q, n_seq]
            slot = torch.full((n_seq,), -1, dtype=torch.long)
            slot[queries] = torch.arange(queries.numel())
            qslot = slot[ei[1]]
            hops = torch.where(qslot >= 0, dist_q[qslot.clamp_min(0), ei[0]], torch.full_like(qslot, -1))
            for c in cores:
                c.edge_hops = hops.to(device)
            model(x_i.to(device), None if bias is None else bias.to(device), graph.to(device), attn_type=args.attn_type)
        per_layer = [c.get_hop_mass_stats() for c in cores]
    finally:
        for c in cores:
            c.disable_hop_mass_tracking()
            c.edge_hops = None
        model.train()
    if getattr(args, "rank", 0) == 0:
        return analytics.write_hop_stats(args, epoch, per_layer)
    return None
