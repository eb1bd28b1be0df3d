"""Small helpers of the legacy mini-batch / graph-level paths: padding, scoped seeding, dense-bias batchers,
global-token plumbing, per-group random-walk subgraphs and the attention-graph sanity check.

Restates, on this package's containers, the helper families of the reference's utility library
(gt_sp/utils.py): ``fixed_random_seed[_cpu]`` (:497-537), the ``pad_*`` family (:620-743), ``get_batch`` (:822-866),
``compute_hops_random_walk`` (:1013-1071), ``compute_hop_buckets_random_walk`` / ``build_head_hop_edges`` (:1074-1278),
``compute_group_nodes_random_walk`` (:1476-1536),
``get_batch_papers100m`` / ``get_batch_from_loader[_malnet]`` (:2082-2233), ``split_tensor_along_second_dim`` /
``merge_global_token[0]`` / ``extend_global_token[0]`` (:2236-2362), ``broadcast_data`` (:2389-2406) and
``check_conditions`` (:2494-2515; here on SciPy's connected components, the reference's version needs a module it
never imports).  The padding family is one function, ``pad_to``, with the named variants as thin wrappers.
"""
from __future__ import annotations

import contextlib
import random
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..graph.attn_graph import Topology
from ..graph.builder_spec import random_walks
from ..parallel.initialize import (get_global_token_indices, get_last_batch_flag, get_sequence_parallel_group,
                                   get_sequence_parallel_rank, get_sequence_parallel_src_rank,
                                   get_sequence_parallel_world_size, last_batch_flag, sequence_parallel_is_initialized)

IGNORE_LABEL = -100


# ----------------------------------------------------------------------------------------------- scoped seeding
@contextlib.contextmanager
def fixed_random_seed(seed: int):
    """Seed python / numpy / torch (CPU and every CUDA generator) inside the block, restore all states after it."""
    states = (random.getstate(), np.random.get_state(), torch.random.get_rng_state(),
              torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None)
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    try:
        yield
    finally:
        random.setstate(states[0])
        np.random.set_state(states[1])
        torch.random.set_rng_state(states[2])
        if states[3] is not None:
            torch.cuda.set_rng_state_all(states[3])


@contextlib.contextmanager
def fixed_random_seed_cpu(seed: int):
    """Like ``fixed_random_seed`` but leaves the CUDA generators alone (only the CPU default generator is seeded)."""
    states = (random.getstate(), np.random.get_state(), torch.random.get_rng_state())
    random.seed(seed)
    np.random.seed(seed)
    torch.default_generator.manual_seed(seed)
    try:
        yield
    finally:
        random.setstate(states[0])
        np.random.set_state(states[1])
        torch.random.set_rng_state(states[2])


# ----------------------------------------------------------------------------------------------- padding
def pad_to(x: torch.Tensor, sizes: Sequence[Optional[int]], value=0) -> torch.Tensor:
    """``x`` copied into the leading corner of a tensor whose dim i has ``sizes[i]`` entries (``None`` = keep).
    Dimensions that are already long enough are kept, so the call never truncates."""
    target = [x.size(i) if s is None else max(int(s), x.size(i)) for i, s in enumerate(sizes)]
    target += list(x.shape[len(target):])
    if target == list(x.shape):
        return x
    out = x.new_full(target, value)
    out[tuple(slice(0, n) for n in x.shape)] = x
    return out


def _sp() -> int:
    return get_sequence_parallel_world_size() if sequence_parallel_is_initialized() else 1


def pad_y(y, padlen):                       # labels: padded rows are ignored by the loss
    return pad_to(y, [padlen], IGNORE_LABEL)


def pad_2d(x, padlen):                      # [s, d] -> [padlen, d]
    return pad_to(x, [padlen, None])


def pad_attn_bias(b, padlen):               # [s, s, d] -> [padlen, padlen, d]
    return pad_to(b, [padlen, padlen, None])


def pad_2d_bs(x, padlen):                   # [bs, s] -> [bs, padlen]
    return pad_to(x, [None, padlen])


def pad_x_bs(x, padlen):                    # [bs, s, d] -> [bs, padlen, d]
    return pad_to(x, [None, padlen, None])


def pad_3d_bs(x, padlen):                   # [bs, s_local, s] -> [bs, padlen, padlen * P]
    return pad_to(x, [None, padlen, padlen * _sp()])


def pad_4d_bs(x, padlen):                   # [bs, s, a, b] -> [bs, padlen, a, b]
    return pad_to(x, [None, padlen, None, None])


def pad_5d_bs(x, padlen):                   # [bs, s_local, s, a, b] -> [bs, padlen, padlen * P, a, b]
    return pad_to(x, [None, padlen, padlen * _sp(), None, None])


def pad_attn_bias_bs(x, padlen):            # rows include one global token: [bs, padlen, (padlen - 1) * P + 1]
    return pad_to(x, [None, padlen, (padlen - 1) * _sp() + 1])


def pad_attn_bias_bs_unsplit(x, padlen, graph_node_num):
    """Whole-sequence bias ``[bs, L, L]`` with ``L = padlen * P + 1``: new entries are ``-inf`` except that padded
    query rows may attend to the real nodes of their own graph (so that their softmax stays finite)."""
    full = padlen * _sp() + 1
    rows = x.size(1)
    if rows >= full:
        return x
    out = pad_to(x, [None, full, full], float("-inf"))
    for i, real in enumerate(graph_node_num.tolist()):
        out[i, rows:, : int(real)] = 0
    return out


def pad_spatial_pos_bs_unsplit(x, padlen):  # [bs, s, s] -> [bs, padlen * P, padlen * P]
    return pad_to(x, [None, padlen * _sp(), padlen * _sp()])


def pad_edge_input_bs_unsplit(x, padlen):   # [bs, s, s, a, b] -> [bs, padlen * P, padlen * P, a, b]
    return pad_to(x, [None, padlen * _sp(), padlen * _sp(), None, None])


# ----------------------------------------------------------------------------------------------- virtual-node edge lists
def fix_edge_index(edge_index: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """COO form of the Graphormer virtual node: ids shifted by one, node 0 linked with every node both ways."""
    nodes = torch.arange(1, int(num_nodes) + 1, dtype=edge_index.dtype, device=edge_index.device)
    zeros = torch.zeros_like(nodes)
    return torch.cat([edge_index + 1, torch.stack([nodes, zeros]), torch.stack([zeros, nodes])], 1)


def adjust_edge_index_nomerge(edge_index: torch.Tensor, sub_seq_len: int) -> torch.Tensor:
    """Ids > 0 moved to their row in the sequence that carries one global-token copy per rank:
    ``id + (id - 1) // sub_seq_len``."""
    shift = torch.div(edge_index - 1, int(sub_seq_len), rounding_mode="floor")
    return torch.where(edge_index > 0, edge_index + shift, edge_index)


# ----------------------------------------------------------------------------------------------- dense-bias batchers
def dense_bias_from_adjs(adjs, idx: torch.Tensor) -> torch.Tensor:
    """``[s, s, d]`` bias of a sequence: channel c is the ``idx x idx`` block of the c-th SciPy sparse matrix
    (the powers of the normalised adjacency in the reference's preprocessing)."""
    rows = idx.cpu().numpy()
    blocks = [torch.from_numpy(np.asarray(a[rows, :][:, rows].todense(), dtype=np.float32)) for a in adjs]
    return torch.stack(blocks, -1)


def get_batch(args, x, y, idx_batch, adjs, rest_split_sizes=None, device="cpu"):
    """Rows of this rank for one sequence with a dense ``[s_local, s, d]`` attention bias.  A short last sequence is
    cut by ``rest_split_sizes`` and every piece padded to the longest (features 0, labels ignored, bias 0)."""
    p = _sp()
    r = get_sequence_parallel_rank() if sequence_parallel_is_initialized() else 0
    seq_len = int(args.seq_len)
    x_i, y_i, bias = x[idx_batch], y[idx_batch], dense_bias_from_adjs(adjs, idx_batch)
    if idx_batch.numel() < seq_len:
        assert rest_split_sizes is not None, "a short sequence needs its per-rank split sizes"
        padlen = max(rest_split_sizes)
        xs, ys, bs = (torch.split(t, list(rest_split_sizes), 0) for t in (x_i, y_i, bias))
        last_batch_flag(True)
        return (pad_2d(xs[r], padlen).to(device), pad_y(ys[r], padlen).to(device),
                pad_attn_bias(bs[r], padlen).to(device))
    assert seq_len % p == 0
    s = seq_len // p
    last_batch_flag(False)
    return x_i[r * s:(r + 1) * s].to(device), y_i[r * s:(r + 1) * s].to(device), bias[r * s:(r + 1) * s].to(device)


def get_batch_papers100m(args, x, y, idx_batch, attn_bias, rest_split_sizes, device, edge_index, num_nodes):
    """Whole (unsharded) sequence with its induced edge list and a caller-supplied dummy bias; for Graphormer the
    edge list gets the virtual node and is re-indexed for one global-token copy per rank."""
    from .legacy_batch import induced_subgraph
    world = int(getattr(args, "world_size", 0) or _sp())
    seq_len = int(args.seq_len)
    sub = seq_len // world
    x_i, y_i = x[idx_batch], y[idx_batch]
    ei = induced_subgraph(edge_index, idx_batch, num_nodes)
    graphormer = str(getattr(args, "model", "")) == "graphormer"
    if graphormer:
        ei = fix_edge_index(ei, idx_batch.numel())
    if idx_batch.numel() < seq_len:
        assert rest_split_sizes is not None, "a short sequence needs its per-rank split sizes"
        sub = max(rest_split_sizes)
        x_i, y_i = pad_2d(x_i, sub * world), pad_y(y_i, sub * world)
    if graphormer:
        ei = adjust_edge_index_nomerge(ei, sub)
    return x_i, y_i, attn_bias, ei


def _split_pad_graph_batch(batch, num_global_node: int, world: int):
    lens = list(batch.sub_split_seq_lens)
    padlen = max(lens)
    xs = [pad_x_bs(t, padlen) for t in torch.split(batch.x, lens, 1)]
    ins = [pad_2d_bs(t, padlen) for t in torch.split(batch.in_degree, lens, 1)]
    outs = [pad_2d_bs(t, padlen) for t in torch.split(batch.out_degree, lens, 1)]
    real = padlen + int(num_global_node)
    return xs, ins, outs, list(range(0, world * real, real))


def get_batch_from_loader(args, batch) -> None:
    """Graph-level collated batch (``x [bs, s, d]``, ``in_degree`` / ``out_degree [bs, s]``, ``sub_split_seq_lens``):
    keeps this rank's slice, padded to the longest slice, and records where the global tokens sit; in place."""
    p = _sp()
    r = get_sequence_parallel_rank() if sequence_parallel_is_initialized() else 0
    xs, ins, outs, tokens = _split_pad_graph_batch(batch, getattr(args, "num_global_node", 1), p)
    batch.x, batch.in_degree, batch.out_degree = xs[r], ins[r], outs[r]
    if getattr(args, "dummy_bias", False):
        batch.attn_bias = None
    batch.global_token_indices = tokens
    del batch.sub_split_seq_lens


def get_batch_from_loader_malnet(args, batch):
    """Same cut, but every rank's slice is returned (one process feeding ``args.world_size`` logical ranks)."""
    world = int(args.world_size)
    xs, ins, outs, tokens = _split_pad_graph_batch(batch, getattr(args, "num_global_node", 1), world)
    batch.x, batch.in_degree, batch.out_degree = xs, ins, outs
    if getattr(args, "dummy_bias", False):
        batch.attn_bias = None
    batch.global_token_indices = tokens
    return xs, ins, outs, tokens


def broadcast_data(args, dataset_train, batch, device) -> torch.Tensor:
    """Node / graph ids of the batch, broadcast from the SP source rank so that every rank collates the same one."""
    import torch.distributed as dist
    idx = batch.idx.to(device) if get_sequence_parallel_rank() == 0 else \
        torch.empty(batch.idx.numel(), dtype=torch.int64, device=device)
    if _sp() > 1:
        dist.broadcast(idx, get_sequence_parallel_src_rank(), group=get_sequence_parallel_group())
    return idx


# ----------------------------------------------------------------------------------------------- global-token plumbing
def split_tensor_along_second_dim(tensor: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False):
    chunks = torch.split(tensor, tensor.size(1) // int(num_partitions), dim=1)
    return tuple(c.contiguous() for c in chunks) if contiguous_split_chunks else chunks


def _token_rows(x: torch.Tensor, dim: int) -> Tuple[torch.Tensor, torch.Tensor]:
    tokens = torch.as_tensor(get_global_token_indices(last_batch=get_last_batch_flag()), dtype=torch.long, device=x.device)
    keep = torch.ones(x.size(dim), dtype=torch.bool, device=x.device)
    keep[tokens] = False
    return tokens, torch.nonzero(keep).flatten()


def merge_global_token(x: torch.Tensor, merge_dim: int) -> torch.Tensor:
    """The per-rank global-token copies averaged into one token appended after the node rows."""
    tokens, rest = _token_rows(x, merge_dim)
    avg = x.index_select(merge_dim, tokens).mean(merge_dim, keepdim=True)
    return torch.cat([x.index_select(merge_dim, rest), avg], merge_dim).contiguous()


def merge_global_token0(x: torch.Tensor, merge_dim: int) -> torch.Tensor:
    """Same, with the merged token placed in front."""
    tokens, rest = _token_rows(x, merge_dim)
    avg = x.index_select(merge_dim, tokens).mean(merge_dim, keepdim=True)
    return torch.cat([avg, x.index_select(merge_dim, rest)], merge_dim).contiguous()


def extend_global_token(x: torch.Tensor, extend_dim: int) -> torch.Tensor:
    """``[b, P*c, ...]`` cut into P chunks along dim 1, the last chunk appended to every chunk along ``extend_dim``."""
    chunks = split_tensor_along_second_dim(x, _sp())
    return torch.cat([torch.cat([c, chunks[-1]], extend_dim) for c in chunks[: _sp()]], extend_dim).contiguous()


def extend_global_token0(x: torch.Tensor, extend_dim: int) -> torch.Tensor:
    """``[b, 1 + P*s, ...]`` (token first) to ``[b, P*(1+s), ...]``: the token in front of every rank's slice."""
    p = _sp()
    assert (x.size(extend_dim) - 1) % p == 0
    s = (x.size(extend_dim) - 1) // p
    parts = torch.split(x, [1] + [s] * p, extend_dim)
    return torch.cat([torch.cat([parts[0], parts[i]], extend_dim) for i in range(1, p + 1)], extend_dim).contiguous()


# ----------------------------------------------------------------------------------------------- per-group random-walk subgraphs
def _emitted(walks: np.ndarray, d: int) -> np.ndarray:
    ok = walks[:, d] >= 0
    if d > 1:
        ok &= walks[:, d] != walks[:, d - 1]          # a walk that stayed put (dead end) emits nothing
    return ok


def compute_hops_random_walk(topo: Topology, walk_length: int = 6, walks_per_node: int = 2, num_groups: int = 4,
                             seed: int = 0) -> List[torch.Tensor]:
    """One edge list ``[2, E_g]`` (start node, node reached) per head group: hop d feeds group ``(d-1) % groups`` from
    that group's own walks, and a node serves as an end point in one hop only (the first that reaches it)."""
    length, groups, w = max(1, int(walk_length)), max(1, int(num_groups)), max(1, int(walks_per_node))
    n = topo.num_nodes
    walks = random_walks(topo, w * groups, length, seed).reshape(n, groups, w, length + 1)
    seen = np.zeros(n, dtype=bool)
    out: List[List[np.ndarray]] = [[] for _ in range(groups)]
    for d in range(1, length + 1):
        g = (d - 1) % groups
        wg = walks[:, g].reshape(-1, length + 1)
        ok = _emitted(wg, d)
        src, dst = wg[ok, 0], wg[ok, d]
        fresh = ~seen[dst]
        seen[dst[fresh]] = True
        if fresh.any():
            out[g].append(np.stack([src[fresh], dst[fresh]]))
    return [torch.from_numpy(np.concatenate(e, 1)) if e else torch.zeros(2, 0, dtype=torch.long) for e in out]


def compute_hop_buckets_random_walk(topo: Topology, num_buckets: int, walk_length: int = 4, walks_per_node: int = 2,
                                    min_hop: int = 1, seed: int = 0) -> List[torch.Tensor]:
    """The walk edges ``(node reached at hop d, start node)`` grouped by hop: bucket ``min(d - 1, num_buckets - 1)``
    holds hop d, for d from ``min_hop`` (2 = only nodes at least two steps away) to ``walk_length``
    (gt_sp/utils.py:1074-1248).  Row 0 is the key / value node, row 1 the query, as attention expects."""
    length, buckets = max(1, int(walk_length)), max(1, int(num_buckets))
    walks = random_walks(topo, max(1, int(walks_per_node)), length, seed)
    out: List[List[np.ndarray]] = [[] for _ in range(buckets)]
    for d in range(max(1, int(min_hop)), length + 1):
        ok = _emitted(walks, d)
        out[min(d - 1, buckets - 1)].append(np.stack([walks[ok, d], walks[ok, 0]]))
    return [torch.from_numpy(np.concatenate(e, 1)) if e else torch.zeros(2, 0, dtype=torch.long) for e in out]


def build_head_hop_edges(topo: Topology, walk_length: int = 4, walks_per_node: int = 2, min_hop: int = 1,
                         seed: int = 0) -> torch.Tensor:
    """One walk-edge pool shared by all heads (gt_sp/utils.py:1251-1278): the single bucket of the function above."""
    return compute_hop_buckets_random_walk(topo, 1, walk_length, walks_per_node, min_hop, seed)[0]


def compute_group_nodes_random_walk(topo: Topology, walk_length: int = 6, walks_per_node: int = 2, num_groups: int = 4,
                                    max_nodes_per_group: int = 2048, seed: int = 0) -> List[torch.Tensor]:
    """Node list per group: seeds ``g, g+groups, ...`` (at most ``max_nodes_per_group``) followed by the distinct nodes
    their walks reach, hop by hop, until the group is full.  Groups may overlap."""
    length, groups, w = max(1, int(walk_length)), max(1, int(num_groups)), max(1, int(walks_per_node))
    cap = max(1, int(max_nodes_per_group))
    n = topo.num_nodes
    walks = random_walks(topo, w, length, seed).reshape(n, w, length + 1)
    result = []
    for g in range(groups):
        seeds = np.arange(g, n, groups)[:cap]
        if seeds.size == 0:
            result.append(torch.zeros(0, dtype=torch.long))
            continue
        wg = walks[seeds].reshape(-1, length + 1)
        seen = np.zeros(n, dtype=bool)
        seen[seeds] = True
        nodes, total = [seeds], int(seeds.size)
        for d in range(1, length + 1):
            if total >= cap:
                break
            dst = wg[_emitted(wg, d), d]
            dst = dst[~seen[dst]]
            if dst.size == 0:
                continue
            _, first = np.unique(dst, return_index=True)         # distinct, in order of first appearance
            dst = dst[np.sort(first)][: cap - total]
            seen[dst] = True
            nodes.append(dst)
            total += int(dst.size)
        result.append(torch.from_numpy(np.concatenate(nodes)).long())
    return result


# ----------------------------------------------------------------------------------------------- sanity check
def check_conditions(edge_index: torch.Tensor, num_nodes: int, verbose: bool = False) -> bool:
    """The two structural conditions of the sparse-attention error bound: every node attends to itself, and the
    attention graph is (weakly) connected."""
    from scipy.sparse import coo_matrix
    from scipy.sparse.csgraph import connected_components
    n = int(num_nodes)
    s, d = edge_index[0].long().cpu(), edge_index[1].long().cpu()
    has_loop = torch.zeros(n, dtype=torch.bool)
    has_loop[s[s == d]] = True
    if not bool(has_loop.all()):
        if verbose:
            print(f"Condition 1 failed: node {int(torch.nonzero(~has_loop)[0])} does not attend to itself.")
        return False
    a = coo_matrix((np.ones(s.numel(), dtype=np.int8), (s.numpy(), d.numpy())), shape=(n, n))
    parts, _ = connected_components(a, directed=True, connection="weak")
    if parts != 1:
        if verbose:
            print(f"Condition 3 failed: the graph has {parts} weakly connected components.")
        return False
    return True
