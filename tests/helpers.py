import torch

from budgetformer_b200.graph.attn_graph import AttnGraph, Topology


def random_topology(n=300, e=2500, hub_in=0, hub_out=0, seed=0):
    g = torch.Generator().manual_seed(seed)
    ei = torch.randint(0, n, (2, e), generator=g)
    if hub_in:
        ei = torch.cat([ei, torch.stack([torch.randint(0, n, (hub_in,), generator=g), torch.zeros(hub_in, dtype=torch.long)])], 1)
    if hub_out:
        ei = torch.cat([ei, torch.stack([torch.ones(hub_out, dtype=torch.long), torch.randint(0, n, (hub_out,), generator=g)])], 1)
    return Topology.from_edge_index(ei, n), ei


def random_attn_graph(n=200, e=1500, hub_row=0, hub_col=0, seed=0, typed=False):
    """COO with optional one very long query row and one very popular key."""
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (e,), generator=g)
    dst = torch.randint(0, n, (e,), generator=g)
    if hub_row:
        src = torch.cat([src, torch.randint(0, n, (hub_row,), generator=g)])
        dst = torch.cat([dst, torch.full((hub_row,), 3)])
    if hub_col:
        src = torch.cat([src, torch.full((hub_col,), 5)])
        dst = torch.cat([dst, torch.randint(0, n, (hub_col,), generator=g)])
    rows = [src, dst]
    if typed:
        rows.append(torch.randint(0, 2, (src.numel(),), generator=g))
    return AttnGraph.from_edge_index(torch.stack(rows), n)
