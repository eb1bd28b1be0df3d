import torch


def coalesce(edge_index, edge_attr=None, num_nodes=None, reduce="sum", is_sorted=False, sort_by_row=True):
    n = int(num_nodes) if num_nodes is not None else int(edge_index.max()) + 1
    key = torch.unique(edge_index[0].to(torch.long) * n + edge_index[1].to(torch.long))
    return torch.stack([torch.div(key, n, rounding_mode="floor"), key % n], 0)


def degree(index, num_nodes=None, dtype=None):
    n = int(num_nodes) if num_nodes is not None else int(index.max()) + 1
    out = torch.bincount(index.to(torch.long), minlength=n)
    return out.to(dtype) if dtype is not None else out.to(torch.float)


def remove_self_loops(edge_index, edge_attr=None):
    m = edge_index[0] != edge_index[1]
    return edge_index[:, m], (edge_attr[m] if edge_attr is not None else None)


def add_self_loops(edge_index, edge_attr=None, fill_value=None, num_nodes=None):
    n = int(num_nodes) if num_nodes is not None else int(edge_index.max()) + 1
    loops = torch.arange(n, device=edge_index.device, dtype=edge_index.dtype)
    return torch.cat([edge_index, torch.stack([loops, loops])], 1), edge_attr


def subgraph(subset, edge_index, edge_attr=None, relabel_nodes=False, num_nodes=None, return_edge_mask=False):
    n = int(num_nodes) if num_nodes is not None else int(edge_index.max()) + 1
    mask = torch.zeros(n, dtype=torch.bool, device=edge_index.device)
    mask[subset] = True
    em = mask[edge_index[0]] & mask[edge_index[1]]
    ei = edge_index[:, em]
    if relabel_nodes:
        remap = torch.full((n,), -1, dtype=torch.long, device=edge_index.device)
        remap[subset] = torch.arange(int(mask.sum()) if subset.dtype == torch.bool else subset.numel(), device=edge_index.device)
        ei = remap[ei]
    return (ei, edge_attr, em) if return_edge_mask else (ei, edge_attr)
