"""Minimal pure-PyTorch stand-in for ``torch_cluster.random_walk`` (CSR calling form): uniform next neighbour,
walkers at a sink stay in place."""
import torch


def random_walk(rowptr, col, start, walk_length, p=1.0, q=1.0, coalesced=True, num_nodes=None, return_edge_indices=False):
    if rowptr.numel() == col.numel() and rowptr.numel() != 0 and not bool((rowptr[1:] >= rowptr[:-1]).all()):
        raise RuntimeError("size mismatch: COO form is not supported by this shim, expected CSR rowptr")
    cur = start.to(torch.long)
    out = [cur]
    deg_all = rowptr[1:] - rowptr[:-1]
    for _ in range(int(walk_length)):
        deg = deg_all[cur]
        pick = (torch.rand(cur.numel(), device=cur.device) * deg).to(torch.long)
        pick = torch.minimum(pick, (deg - 1).clamp_min(0))
        nxt = col[(rowptr[cur] + pick).clamp_max(col.numel() - 1)] if col.numel() else cur
        cur = torch.where(deg > 0, nxt, cur)
        out.append(cur)
    return torch.stack(out, dim=1)
