"""Microbenchmarks of the package's kernels against the measured roofline of the machine.

    python -m budgetformer_b200.utils.kernel_bench gemm --m 2923922 --n 384 --k 128
    python -m budgetformer_b200.utils.kernel_bench attn --nodes 2923922 --heads 8 --head_dim 16 --degree 8
    python -m budgetformer_b200.utils.kernel_bench ln --rows 2923922 --hidden 128
    python -m budgetformer_b200.utils.kernel_bench build --nodes 2923922 --edges 13975788
    python -m budgetformer_b200.utils.kernel_bench dw --m 2923922 --n 128 --k 128 --compare
    python -m budgetformer_b200.utils.kernel_bench pull --m 800000 --n 128 --k 128 --sources 8
    python -m budgetformer_b200.utils.kernel_bench ffn --m 2923922 --compare

Each case runs ``--warmup`` untimed and ``--iters`` timed launches bracketed by CUDA events on the launching
stream, with operands larger than the 126 MB L2 (or ``--flush_l2``), and prints one JSON line: milliseconds,
algorithmic bytes / FLOPs, achieved GB/s / TFLOP/s and their fraction of the copy bandwidth and bf16 GEMM rate
in ``MEASURED_PEAKS.json`` (fallback 6650 GB/s, 1590 TFLOP/s when the file is absent).  ``--once`` launches every
kernel of the case a single time after warm-up (for profilers)."""
from __future__ import annotations

import argparse
import json
import os

import torch


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def timed(fn, warmup, iters, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        tot += s.elapsed_time(e)
    return tot / max(1, iters)


def report(name, ms, nbytes, flops, extra):
    bw, tf, src = peaks()
    gbs = nbytes / ms / 1e6
    tfl = flops / ms / 1e9
    rec = {"kernel": name, "ms": round(ms, 4), "bytes": int(nbytes), "flops": int(flops), "GBps": round(gbs, 1),
           "TFLOPs": round(tfl, 2), "frac_hbm": round(gbs / bw, 3), "frac_bf16": round(tfl / tf, 3), "peaks": src}
    rec.update(extra)
    print(json.dumps(rec), flush=True)


def case_gemm(a):
    from ..ops import gemm
    dev = "cuda"
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev) * 0.05).bfloat16()
    bias = torch.zeros(a.n, device=dev)
    res = torch.randn(a.m, a.n, device=dev).bfloat16() if a.residual else None
    out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    fn = lambda: gemm.gemm_tn(x, w, bias, a.act or None, residual=res, out=out)
    ms = timed(fn, a.warmup, 1 if a.once else a.iters)
    nbytes = 2 * (a.m * a.k + a.n * a.k + a.m * a.n * (2 if a.residual else 1))
    report("gemm_tn_tcgen05", ms, nbytes, 2.0 * a.m * a.n * a.k, {"m": a.m, "n": a.n, "k": a.k})
    if a.compare:
        ms2 = timed(lambda: torch.nn.functional.linear(x, w, bias.bfloat16()), a.warmup, a.iters)
        report("cublas_linear", ms2, nbytes, 2.0 * a.m * a.n * a.k, {"m": a.m, "n": a.n, "k": a.k})
    gemm.check_status(dev)


def case_dw(a):
    """Weight-gradient GEMM dW = dY^T X (+ bias gradient) against the bytes of its two operands."""
    from ..ops import gemm
    dy = torch.randn(a.m, a.n, device="cuda").bfloat16()
    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    fn = lambda: gemm.weight_grad(dy, x, want_bias=True)
    ms = timed(fn, a.warmup, 1 if a.once else a.iters)
    report("gemm_dw_tcgen05", ms, 2 * a.m * (a.n + a.k), 2.0 * a.m * a.n * a.k, {"m": a.m, "n": a.n, "k": a.k})
    if a.compare:
        ms2 = timed(lambda: (torch.matmul(dy.t(), x), dy.float().sum(0)), a.warmup, a.iters)
        report("library matmul + column sum", ms2, 2 * a.m * (a.n + a.k), 2.0 * a.m * a.n * a.k, {"m": a.m, "n": a.n, "k": a.k})
    gemm.check_status("cuda")


def case_ffn(a):
    """Forward feed-forward block (model width 128, hidden 256): one kernel with the hidden tile on chip against the two
    GEMM launches that write and re-read the hidden matrix.  Algorithmic bytes = X in + Y out."""
    from ..ops import ffn as ffn_mod, gemm
    x = torch.randn(a.m, 128, device="cuda").bfloat16()
    l1, l2 = torch.nn.Linear(128, 256).cuda(), torch.nn.Linear(256, 128).cuda()
    act = a.act or "relu"
    nbytes = 2 * 2 * a.m * 128
    flops = 2.0 * a.m * 128 * 256 * 2
    with torch.no_grad():
        fn = lambda: ffn_mod.ffn_onchip(x, l1.weight, l1.bias, l2.weight, l2.bias, act=act, residual=True)
        ms = timed(fn, a.warmup, 1 if a.once else a.iters)
        report("ffn_fused_tcgen05 (hidden tile on chip)", ms, nbytes, flops, {"m": a.m, "act": act})
        if a.compare:
            w1, w2 = gemm.operand_copy(l1.weight, x.dtype), gemm.operand_copy(l2.weight, x.dtype)
            def two():
                h = gemm.gemm_tn(x, w1, l1.bias, act)
                return gemm.gemm_tn(h, w2, l2.bias, None, residual=x)
            ms2 = timed(two, a.warmup, a.iters)
            report("two tcgen05 GEMMs (hidden matrix through HBM)", ms2, nbytes, flops, {"m": a.m, "act": act})
            # training forward: hidden matrix and ReLU bits kept for the backward pass
            hbuf = torch.empty(a.m, 256, device="cuda", dtype=torch.bfloat16)
            bits = torch.empty(16, a.m, device="cuda", dtype=torch.int16)
            fn3 = lambda: ffn_mod.ffn_onchip(x, l1.weight, l1.bias, l2.weight, l2.bias, act=act, residual=True, p1=0.1, seed1=5,
                                             h_out=hbuf, relu_bits_out=bits)
            ms3 = timed(fn3, a.warmup, a.iters)
            report("ffn_fused_tcgen05 + hidden matrix and ReLU bits as side outputs", ms3, nbytes + 2 * a.m * 256, flops, {"m": a.m})
            def two_train():
                h = gemm.gemm_tn(x, w1, l1.bias, act, dropout_p=0.1, dropout_seed=5, relu_bits_out=bits)
                return gemm.gemm_tn(h, w2, l2.bias, None, residual=x)
            ms4 = timed(two_train, a.warmup, a.iters)
            report("two tcgen05 GEMMs, training forward (bits written)", ms4, nbytes + 2 * a.m * 256, flops, {"m": a.m})
    gemm.check_status("cuda")


def case_pull(a):
    """Gathered-operand GEMM on one GPU: the sources are local buffers standing in for the peers' (same kernel, same
    loader warps; the bytes cross HBM instead of NVLink), so the kernel's own counters can be read under a profiler."""
    from ..ops import fused_sp, gemm
    cps = a.k // a.sources
    srcs = [torch.randn(a.m, cps, device="cuda").bfloat16() for _ in range(a.sources)]
    w = (torch.randn(a.n, a.k, device="cuda") * 0.05).bfloat16()
    bias = torch.zeros(a.n, device="cuda")
    res = torch.randn(a.m, a.n, device="cuda").bfloat16()
    ptrs = [t.data_ptr() for t in srcs]
    fn = lambda: fused_sp._pull_gemm(ptrs, 0, cps, cps, a.m, w, bias=bias, residual=res, keep_copy=bool(a.keep_copy))
    ms = timed(fn, a.warmup, 1 if a.once else a.iters)
    nbytes = 2 * (a.m * a.k * (2 if a.keep_copy else 1) + a.n * a.k + 2 * a.m * a.n)
    report("gemm_tn_pull (local sources)", ms, nbytes, 2.0 * a.m * a.n * a.k,
           {"m": a.m, "n": a.n, "k": a.k, "sources": a.sources, "keep_copy": bool(a.keep_copy)})
    gemm.check_status("cuda")


def _graph(nodes, degree, seed=0, key_window=0):
    """``degree`` keys per query, uniform over all nodes, or (``key_window > 0``) within that many ids of the query:
    the gather pattern of a graph whose nodes were relabelled by locality (``--locality_reorder_parts``)."""
    from ..graph.attn_graph import AttnGraph
    g = torch.Generator(device="cuda").manual_seed(seed)
    if key_window > 0:
        rows = torch.arange(nodes, device="cuda", dtype=torch.int64).repeat_interleave(degree)
        off = torch.randint(-int(key_window), int(key_window) + 1, (nodes * degree,), device="cuda", generator=g)
        col = ((rows + off) % nodes).to(torch.int32)
    else:
        col = torch.randint(0, nodes, (nodes * degree,), device="cuda", generator=g, dtype=torch.int32)
    rowptr = torch.arange(0, nodes * degree + 1, degree, device="cuda", dtype=torch.int32)
    return AttnGraph(nodes, rowptr, col, None, max_degree=degree).ensure_transpose()


def case_attn(a):
    from ..ops.edge_attention import edge_attention
    n, hl, hn = a.nodes, a.heads, a.head_dim
    g = _graph(n, a.degree, key_window=a.key_window)
    qkv = torch.randn(n, 3, hl, hn, device="cuda").bfloat16()
    q, k, v = (qkv[:, i].detach().requires_grad_(True) for i in range(3))
    e = n * a.degree
    w = hl * hn * 2
    fwd = lambda: edge_attention(q, k, v, g)
    ms = timed(fwd, a.warmup, 1 if a.once else a.iters)
    report("edge_attn_fwd", ms, e * (2 * w + 4) + n * 2 * w, 4.0 * e * hl * hn, {"nodes": n, "edges": e, "hl": hl, "hn": hn})
    out = fwd()
    dout = torch.randn_like(out)
    def bwd():
        q.grad = k.grad = v.grad = None
        out.backward(dout, retain_graph=True)
    ms = timed(bwd, a.warmup, 1 if a.once else a.iters)
    report("edge_attn_bwd(q+kv passes)", ms, 2 * e * (2 * w + 12) + n * 8 * w, 12.0 * e * hl * hn,
           {"nodes": n, "edges": e, "hl": hl, "hn": hn})


def case_ln(a):
    from ..ops.norm import layer_norm
    x = torch.randn(a.rows, a.hidden, device="cuda").bfloat16().requires_grad_(True)
    ln = torch.nn.LayerNorm(a.hidden).cuda()
    fwd = lambda: layer_norm(x, ln.weight, ln.bias, ln.eps)
    ms = timed(fwd, a.warmup, 1 if a.once else a.iters)
    report("ln_fwd", ms, 4 * a.rows * a.hidden, 0, {"rows": a.rows, "h": a.hidden})
    y = fwd()
    dy = torch.randn_like(y)
    def bwd():
        x.grad = None
        y.backward(dy, retain_graph=True)
    ms = timed(bwd, a.warmup, 1 if a.once else a.iters)
    report("ln_bwd", ms, 6 * a.rows * a.hidden, 0, {"rows": a.rows, "h": a.hidden})


def case_build(a):
    from ..graph.attn_graph import Topology
    from ..graph.builder import build_attn_graph
    from ..graph.synthetic import chung_lu_edges_device, citation_dag_edges
    if a.graph == "dag":
        ei = citation_dag_edges(a.nodes, a.edges, seed=1)
    else:                                       # power-law graphs of the large configurations: in-degrees up to 10^5 - 10^6
        ei = chung_lu_edges_device(a.nodes, a.edges, 2.1, a.graph == "chung_lu_directed", 1, torch.device("cuda"))
    topo = Topology.from_edge_index(ei.to("cuda"), a.nodes)
    indeg = topo.in_rowptr[1:] - topo.in_rowptr[:-1]
    seeds = iter(range(10 ** 6))
    fn = lambda: build_attn_graph(topo, a.b_real, a.b_rw, a.walks, a.walk_len, next(seeds))
    ms = timed(fn, a.warmup, 1 if a.once else a.iters)
    g = fn()
    report("budget_select+ell_to_csr", ms, topo.nbytes() + g.nbytes(), 0, {"nodes": a.nodes, "raw_edges": int(ei.size(1)),
                                                                             "graph_edges": g.num_edges,
                                                                             "max_in_degree": int(indeg.max()),
                                                                             "block_ranked_rows": int((indeg > 4096).sum()),
                                                                             "block_prepass": os.environ.get("BF_BUILD_HUB_BLOCKS", "1") != "0"})
    ms = timed(lambda: build_attn_graph(topo, a.b_real, a.b_rw, a.walks, a.walk_len, 7).ensure_transpose(), a.warmup, a.iters)
    report("build+transpose+kv_tasks", ms, 0, 0, {"nodes": a.nodes})


def case_sp(a):
    """Fused sequence-parallel ops against their NCCL + cuBLAS equivalents.  Run under torchrun, one rank per GPU."""
    import torch.distributed as dist
    from ..ops import fused_sp, gemm
    from ..parallel import symm
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_loc = a.nodes // world
    h, heads = a.hidden, a.heads
    # the pull form of heads->nodes is what this case times (the routed form has no kernel of its own to time: its
    # transfer rides on the attention kernels' stores)
    sp = fused_sp.SPContext(dist.group.WORLD if world > 1 else None, dev, world, n_loc, h, heads, 1, torch.bfloat16,
                            routed=False)
    x = torch.randn(n_loc, h, device=dev).bfloat16()
    wq, wk, wv = (torch.randn(h, h, device=dev) * 0.05 for _ in range(3))
    wo = (torch.randn(h, h, device=dev) * 0.05)
    link_gbs = 770.0
    esz = 2

    def tmax(ms):
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def emit(name, ms, link_bytes, flops):
        if rank != 0:
            return
        _, tf, src = peaks()
        t_link = link_bytes / (link_gbs * 1e6)           # ms
        t_flop = flops / (tf * 1e9)
        bound = max(t_link, t_flop, 1e-9)
        print(json.dumps({"op": name, "world": world, "ms": round(ms, 4), "nvlink_bytes_per_rank": int(link_bytes),
                          "flops": int(flops), "roofline_ms": round(bound, 4), "frac_of_roofline": round(bound / ms, 3),
                          "bound": "nvlink" if t_link >= t_flop else "compute", "link_GBps_assumed": link_gbs,
                          "peaks": src}), flush=True)

    frac = (world - 1) / world
    # ---- nodes -> heads: fused GEMM + push vs cuBLAS + 3 NCCL all-to-alls -----------------------------------
    fused = lambda: fused_sp._QKVPush.apply(x, wq, wk, wv, None, None, None, sp, 0)
    ms = tmax(timed(fused, a.warmup, a.iters))
    emit("qkv_gemm_push (fused)", ms, frac * n_loc * 3 * h * esz, 2.0 * n_loc * h * 3 * h)
    w16 = [w.bfloat16() for w in (wq, wk, wv)]

    def baseline_push():
        outs = []
        for w in w16:
            y = torch.nn.functional.linear(x, w)
            if world > 1:
                send = y.view(n_loc, world, h // world).permute(1, 0, 2).contiguous()
                recv = torch.empty_like(send)
                dist.all_to_all_single(recv, send)
                outs.append(recv)
            else:
                outs.append(y)
        return outs
    ms = tmax(timed(baseline_push, a.warmup, a.iters))
    emit("qkv cuBLAS + 3x NCCL all_to_all (baseline)", ms, frac * n_loc * 3 * h * esz, 2.0 * n_loc * h * 3 * h)
    # ---- heads -> nodes: pull + out-proj GEMM vs NCCL all-to-all + cuBLAS ---------------------------------------
    ctx_full = sp.ctx[0].tensor
    ctx_full.normal_()
    pull = lambda: fused_sp._CtxPullOutProj.apply(ctx_full, wo, None, x, sp, 0.0, 0.0, 0, 0)
    ms = tmax(timed(pull, a.warmup, a.iters))
    emit("ctx_pull_outproj (fused)", ms, frac * n_loc * h * esz, 2.0 * n_loc * h * h)
    wo16 = wo.bfloat16()

    def baseline_pull():
        c = ctx_full
        if world > 1:
            send = c.view(world, n_loc, h // world).contiguous()
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send)
            c = recv.permute(1, 0, 2).reshape(n_loc, h)
        return torch.nn.functional.linear(c, wo16) + x
    ms = tmax(timed(baseline_pull, a.warmup, a.iters))
    emit("NCCL all_to_all + cuBLAS out-proj (baseline)", ms, frac * n_loc * h * esz, 2.0 * n_loc * h * h)
    # ---- gradient all-reduce -----------------------------------------------------------------------------------
    if world > 1:
        for mib in (2.2, 8.4, 64.0):
            nfl = int(mib * 2 ** 20 / 4) // 1024 * 1024
            buf = sp.sw.alloc((nfl,), torch.float32)
            class _B: pass
            b = _B(); b.symm = (sp.sw, buf)
            ms = tmax(timed(lambda: symm.bucket_all_reduce_mean(b), a.warmup, a.iters))
            emit(f"grad all-reduce {mib} MiB (own kernel, multimem={bool(buf.multicast_ptr)})", ms, 2 * frac * nfl * 4, 0)
            t = torch.randn(nfl, device=dev)
            def nccl():
                t.div_(world)
                dist.all_reduce(t)
            ms = tmax(timed(nccl, a.warmup, a.iters))
            emit(f"grad all-reduce {mib} MiB (div_ + NCCL baseline)", ms, 2 * frac * nfl * 4, 0)
        gemm.check_status(dev)
        dist.barrier()
        dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="case", required=True)
    common = dict(warmup=3, iters=10)
    for name in ("gemm", "attn", "ln", "build", "sp", "dw", "pull", "ffn"):
        p = sub.add_parser(name)
        p.add_argument("--warmup", type=int, default=common["warmup"])
        p.add_argument("--iters", type=int, default=common["iters"])
        p.add_argument("--once", action="store_true")
        if name == "ffn":
            p.add_argument("--m", type=int, default=1_000_000)
            p.add_argument("--act", default="relu")
            p.add_argument("--compare", action="store_true")
        elif name in ("dw", "pull"):
            p.add_argument("--m", type=int, default=1_000_000)
            p.add_argument("--n", type=int, default=128)
            p.add_argument("--k", type=int, default=128)
            p.add_argument("--compare", action="store_true")
            p.add_argument("--sources", type=int, default=8)
            p.add_argument("--keep_copy", type=int, default=1)
        elif name == "gemm":
            p.add_argument("--m", type=int, default=1_000_000)
            p.add_argument("--n", type=int, default=384)
            p.add_argument("--k", type=int, default=128)
            p.add_argument("--act", default="")
            p.add_argument("--residual", action="store_true")
            p.add_argument("--compare", action="store_true")
        elif name == "attn":
            p.add_argument("--nodes", type=int, default=1_000_000)
            p.add_argument("--heads", type=int, default=8)
            p.add_argument("--head_dim", type=int, default=16)
            p.add_argument("--degree", type=int, default=8)
            p.add_argument("--key_window", type=int, default=0,
                           help="keys within this many ids of the query (0 = uniform over all nodes)")
        elif name == "sp":
            p.add_argument("--nodes", type=int, default=2_923_920)
            p.add_argument("--hidden", type=int, default=128)
            p.add_argument("--heads", type=int, default=8)
        elif name == "ln":
            p.add_argument("--rows", type=int, default=1_000_000)
            p.add_argument("--hidden", type=int, default=128)
        else:
            p.add_argument("--nodes", type=int, default=1_000_000)
            p.add_argument("--edges", type=int, default=5_000_000)
            p.add_argument("--b_real", type=int, default=4)
            p.add_argument("--b_rw", type=int, default=4)
            p.add_argument("--walks", type=int, default=2)
            p.add_argument("--walk_len", type=int, default=4)
            p.add_argument("--graph", default="dag", choices=["dag", "chung_lu_directed", "chung_lu_undirected"])
    a = ap.parse_args(argv)
    {"gemm": case_gemm, "attn": case_attn, "ln": case_ln, "build": case_build, "sp": case_sp, "dw": case_dw,
     "pull": case_pull, "ffn": case_ffn}[a.case](a)


if __name__ == "__main__":
    main()
