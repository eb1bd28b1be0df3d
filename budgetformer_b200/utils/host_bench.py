"""Wall-clock benchmarks of the host-side (C++/OpenMP) components; no GPU involved.

    python -m budgetformer_b200.utils.host_bench build --nodes 500000 --edges 2500000 [--spec]
    python -m budgetformer_b200.utils.host_bench partition --nodes 1000000 --parts 8
    torchrun --nnodes=1 --nproc-per-node=4 --master-addr 127.0.0.1 -m budgetformer_b200.utils.host_bench shard \\
        --nodes 1000000 --edges 5000000

``build``      the CPU attention-graph builders on a Chung-Lu graph: fixed-width (B = 4 + 4), general two-pass
               (no budget; fan-out 10,5), and with ``--spec`` the numpy specification they are bit-identical to.
``partition``  the multilevel partitioner on a shuffled ring lattice with random long edges and on a shuffled
               stochastic block model (cut fraction against id order and against the planted blocks).
``shard``      under a multi-process launcher (gloo): whole build on every rank with the launcher's single OpenMP
               thread, with cores / ranks threads, and sharded with an all-gather.
Each case prints one JSON line per measurement (best of ``--iters`` runs after one warm-up)."""
from __future__ import annotations

import argparse
import json
import time

import torch


def _best(fn, iters: int):
    fn()
    out, best = None, float("inf")
    for _ in range(max(1, iters)):
        t = time.perf_counter()
        out = fn()
        best = min(best, time.perf_counter() - t)
    return best, out


def _emit(name: str, seconds: float, **extra) -> None:
    print(json.dumps({"case": name, "seconds": round(seconds, 4), **extra}), flush=True)


def case_build(a) -> None:
    from ..graph.attn_graph import Topology
    from ..graph.builder import build_attn_graph
    from ..graph.builder_spec import build_attn_graph_spec
    from ..graph.synthetic import chung_lu_edges
    topo = Topology.from_edge_index(chung_lu_edges(a.nodes, a.edges, seed=1), a.nodes)
    seeds = iter(range(10 ** 6))
    cases = [("fixed 4+4, walks", (4, 4, 2, 4), {}), ("no budget, walks", (None, None, 2, 4), {}),
             ("fixed 4+4, fan-out 10,5", (4, 4, 2, 4), {"fanout": [10, 5]})]
    for label, args, kw in cases:
        s, g = _best(lambda: build_attn_graph(topo, *args, next(seeds), num_threads=a.threads, **kw), a.iters)
        _emit("native: " + label, s, nodes=a.nodes, raw_edges=topo.num_edges, graph_edges=g.num_edges, threads=a.threads)
        if a.spec:
            seed = next(seeds)
            s2, ref = _best(lambda: build_attn_graph_spec(topo, *args, seed, **kw), 1)
            same = torch.equal(ref.col, build_attn_graph(topo, *args, seed, num_threads=a.threads, **kw).col)
            _emit("numpy specification: " + label, s2, identical=bool(same))


def _lattice(n: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    s = torch.arange(n).repeat(5)
    d = (s + torch.randint(1, 20, (5 * n,), generator=g)) % n
    rs, rd = torch.randint(0, n, (n // 4,), generator=g), torch.randint(0, n, (n // 4,), generator=g)
    ei = torch.stack([torch.cat([s, rs]), torch.cat([d, rd])])
    return torch.randperm(n, generator=g)[ei]                          # ids carry no locality


def case_partition(a) -> None:
    from ..graph import partition as P
    from ..graph.synthetic import sbm_graph
    ranges = lambda n, k: torch.arange(n) * k // n
    ei = _lattice(a.nodes)
    s, part = _best(lambda: P.partition_assignment(ei, a.nodes, a.parts), 1)
    e = ei.size(1)
    sizes = torch.bincount(part, minlength=a.parts)
    _emit("lattice + random edges", s, nodes=a.nodes, edges=e, parts=a.parts, cut=round(P.edge_cut(ei, part) / e, 4),
          cut_id_order=round(P.edge_cut(ei, ranges(a.nodes, a.parts)) / e, 4), min_part=int(sizes.min()), max_part=int(sizes.max()))
    n = min(a.nodes, 50_000)
    _, y, ei = sbm_graph(n, blocks=a.parts, p_in=40.0 / n * a.parts / 8, p_out=1.0 / n, feat_dim=4, seed=1)
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(0))
    ei, truth = perm[ei], torch.empty(n, dtype=torch.long)
    truth[perm] = y
    s, part = _best(lambda: P.partition_assignment(ei, n, a.parts), 1)
    e = ei.size(1)
    _emit("stochastic block model", s, nodes=n, edges=e, parts=a.parts, cut=round(P.edge_cut(ei, part) / e, 4),
          cut_planted=round(P.edge_cut(ei, truth) / e, 4), cut_id_order=round(P.edge_cut(ei, ranges(n, a.parts)) / e, 4))


def case_shard(a) -> None:
    import torch.distributed as dist
    from ..config import parse_fullgraph_args
    from ..graph.engine import EdgeEngine, resolve_budget_state
    from ..graph.synthetic import chung_lu_edges
    dist.init_process_group("gloo")
    r, p = dist.get_rank(), dist.get_world_size()
    n = a.nodes - a.nodes % p
    ei = chung_lu_edges(n, a.edges, seed=1)
    base = ["--dataset", "x", "--model", "gt", "--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4"]
    for label, flags in (("whole, 1 thread", ["--edge_build_threads", "1"]), ("whole, cores / ranks threads", []),
                         ("sharded + all-gather", ["--shard_cpu_edge_build"])):
        args = parse_fullgraph_args(base + flags)
        eng = EdgeEngine(args, ei, n, "cpu", nodes_per_rank=n // p, sp_group=dist.group.WORLD, sp_rank=r, sp_world=p)
        state = resolve_budget_state(args)
        seeds = iter(range(100, 10 ** 6))

        def step():
            dist.barrier()
            g = eng.build(next(seeds), state, record=False)
            dist.barrier()
            return g
        s, g = _best(step, a.iters)
        if r == 0:
            _emit(label, s, ranks=p, threads=eng.build_threads, nodes=n, graph_edges=g.num_edges)
        eng.shutdown()
    dist.destroy_process_group()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="case", required=True)
    for name in ("build", "partition", "shard"):
        p = sub.add_parser(name)
        p.add_argument("--nodes", type=int, default=500_000)
        p.add_argument("--edges", type=int, default=2_500_000)
        p.add_argument("--iters", type=int, default=3)
        p.add_argument("--threads", type=int, default=0, help="OpenMP threads (0 = library default)")
        p.add_argument("--parts", type=int, default=8)
        p.add_argument("--spec", action="store_true", help="also time the numpy specification (slow)")
    a = ap.parse_args(argv)
    {"build": case_build, "partition": case_partition, "shard": case_shard}[a.case](a)


if __name__ == "__main__":
    main()
