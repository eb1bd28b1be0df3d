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
