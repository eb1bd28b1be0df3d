"""sm_100a kernels against plain PyTorch fp32 references of the same ops."""
import pytest
import torch

from budgetformer_b200.graph.attn_graph import Topology
from budgetformer_b200.graph.builder import build_attn_graph
from budgetformer_b200.ops.edge_attention import edge_attention, edge_attention_reference
from tests.helpers import random_attn_graph, random_topology

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (2e-4, 2e-4), torch.bfloat16: (3e-2, 3e-2), torch.float16: (5e-3, 5e-3)}


def _run(variant, dtype, hl, hn, hub_row=0, hub_col=0, dropout=0.0, n=257, e=2100):
    dev = torch.device("cuda")
    g = random_attn_graph(n, e, hub_row, hub_col, seed=hl * 7 + hn, typed=(variant == "exphormer")).to(dev)
    torch.manual_seed(1)
    q, k, v = (torch.randn(n, hl, hn, device=dev).mul(1.5).to(dtype).requires_grad_(True) for _ in range(3))
    etab = torch.randn(2, hl, hn, device=dev, requires_grad=True) if variant == "exphormer" else None
    dout = torch.randn(n, hl, hn, device=dev).to(dtype)
    out = edge_attention(q, k, v, g, variant=variant, etable=etab, dropout_p=dropout, dropout_seed=1234)
    out.backward(dout)
    got = [out.detach().float(), q.grad.float(), k.grad.float(), v.grad.float()]
    if etab is not None:
        got.append(etab.grad.float())
    q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    e2 = etab.detach().clone().requires_grad_(True) if etab is not None else None
    ref = edge_attention_reference(q2, k2, v2, g, variant=variant, etable=e2, dropout_p=dropout, dropout_seed=1234)
    ref.backward(dout.float())
    want = [ref.detach(), q2.grad, k2.grad, v2.grad] + ([e2.grad] if e2 is not None else [])
    rtol, atol = TOL[dtype]
    names = ["out", "dq", "dk", "dv", "detab"]
    for name, a, b in zip(names, got, want):
        scale = max(1.0, float(b.abs().max()))
        err = float((a - b).abs().max())
        assert err <= atol * scale + rtol * scale, f"{variant}/{dtype}/{name}: max err {err} (scale {scale})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hl,hn", [(8, 16), (1, 16), (4, 32), (2, 64), (3, 16), (1, 32)])
def test_edge_attention_plain(dtype, hl, hn):
    _run("plain", dtype, hl, hn)


@pytest.mark.parametrize("variant", ["gps", "exphormer"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_edge_attention_variants(variant, dtype):
    _run(variant, dtype, 4, 16)
    _run(variant, dtype, 1, 32)


def test_edge_attention_gps_dropout():
    _run("gps", torch.float32, 4, 16, dropout=0.4)
    _run("gps", torch.bfloat16, 2, 32, dropout=0.25)


@pytest.mark.parametrize("variant", ["plain", "gps", "exphormer"])
def test_edge_attention_hub_rows(variant):
    """A query with 5000 in-edges and a key used by 4000 queries take the chunked hub kernels."""
    _run(variant, torch.float32, 4, 16, hub_row=5000, hub_col=4000, n=4500, e=9000)
    _run(variant, torch.bfloat16, 1, 16, hub_row=20000, hub_col=3000, n=4500, e=9000)


@pytest.mark.parametrize("variant,hl,hn", [("plain", 2, 16), ("plain", 1, 16), ("gps", 4, 16), ("exphormer", 2, 32)])
def test_edge_attention_routed_rows_match_local_rows(variant, hl, hn):
    """Routed stores on one GPU (the "destinations" are local buffers standing in for the peers' mappings): every context
    row also lands in its owner's slab, and routed dq / dk / dv rows equal the unrouted gradients - regular rows, a
    5,000-edge query row, a key used by 4,000 queries (split into work items), typed edges."""
    from budgetformer_b200.ops import _ext
    from budgetformer_b200.ops.edge_attention import _VARIANTS
    ext = _ext.load()
    dev = torch.device("cuda")
    torch.manual_seed(2)
    n_dest, rows_per = 4, 1200
    n = n_dest * rows_per
    g = random_attn_graph(n, 9000, hub_row=5000, hub_col=4000, seed=9, typed=(variant == "exphormer")).to(dev).ensure_transpose()
    w = hl * hn
    q, k, v = (torch.randn(n, hl, hn, device=dev).bfloat16() for _ in range(3))
    etab = (torch.randn(2, hl, hn, device=dev) * 0.5 + 1.0) if variant == "exphormer" else None
    vid = _VARIANTS[variant]
    src = 2                                                          # this "rank" is source 2 of 4
    out = torch.empty(n, hl, hn, device=dev, dtype=torch.bfloat16)
    z = torch.empty(n, hl, device=dev)
    slabs = [torch.full((n_dest * rows_per, w), 7.0, device=dev, dtype=torch.bfloat16) for _ in range(n_dest)]
    route = [rows_per, src * rows_per, w] + [t.data_ptr() for t in slabs]
    ext.edge_attn_fwd(q, k, v, out, z, g.rowptr, g.col, g.etype, etab, vid, 0.0, 0, -1, [], route)
    torch.cuda.synchronize()
    for d in range(n_dest):
        mine = slabs[d][src * rows_per:(src + 1) * rows_per]
        assert torch.equal(mine, out.view(n, w)[d * rows_per:(d + 1) * rows_per]), f"context rows of destination {d}"
        other = torch.cat([slabs[d][:src * rows_per], slabs[d][(src + 1) * rows_per:]])
        assert float((other - 7.0).abs().max()) == 0.0               # nobody else's slab was touched
    # backward: unrouted into a packed [n, ld] buffer, routed into slabs of the same row layout (k | v | q)
    ld = (3 * w + 63) // 64 * 64
    dout = torch.randn(n, hl, hn, device=dev).bfloat16()
    def grads(route):
        buf = torch.full((n, ld), 3.0, device=dev, dtype=torch.bfloat16)
        part = lambda i: buf[:, i * w:(i + 1) * w].view(n, hl, hn)
        zd = torch.empty(n, hl, 2, device=dev)
        detab = torch.zeros(2, hl, hn, device=dev) if etab is not None else None
        ext.edge_attn_bwd(q, k, v, out, z, dout, part(2), part(0), part(1), zd, g.rowptr, g.col, g.etype, g.t_rowptr, g.t_row,
                          g.t_eid, etab, detab, vid, 0.0, 0, -1, g.t_task, g.t_split, int(g.kv_slots), [], route)
        torch.cuda.synchronize()
        return buf
    plain = grads([])
    gslabs = [torch.full((n_dest * rows_per, ld), 5.0, device=dev, dtype=torch.bfloat16) for _ in range(n_dest)]
    untouched = grads([rows_per, src * rows_per, ld, 2 * w, 0, w] + [t.data_ptr() for t in gslabs])
    assert float((untouched - 3.0).abs().max()) == 0.0               # routed gradients never touch the local buffer
    for d in range(n_dest):
        got = gslabs[d][src * rows_per:(src + 1) * rows_per, :3 * w]
        want = plain[d * rows_per:(d + 1) * rows_per, :3 * w]
        # (the 5,000-edge query row adds its dq partials with atomics: last-bit differences between two runs)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), f"gradient rows of destination {d}"
        if 3 * w < ld:                                               # the padding columns of a packed row stay untouched
            assert float((gslabs[d][src * rows_per:(src + 1) * rows_per, 3 * w:] - 5.0).abs().max()) == 0.0
        other = torch.cat([gslabs[d][:src * rows_per], gslabs[d][(src + 1) * rows_per:]])
        assert float((other - 5.0).abs().max()) == 0.0
    # a route that does not cover the rows is refused before anything is launched
    with pytest.raises(RuntimeError):
        ext.edge_attn_fwd(q, k, v, out, z, g.rowptr, g.col, g.etype, etab, vid, 0.0, 0, -1, [], [rows_per + 1, 0, w] + [t.data_ptr() for t in slabs])


def test_edge_attention_strided_qkv_views():
    dev = torch.device("cuda")
    n, hl, hn = 300, 4, 16
    g = random_attn_graph(n, 2000, seed=3).to(dev)
    qkv = torch.randn(n, 3, hl, hn, device=dev, dtype=torch.bfloat16)
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    out = edge_attention(q, k, v, g)
    ref = edge_attention_reference(q.float(), k.float(), v.float(), g)
    assert torch.allclose(out.float(), ref, atol=3e-2, rtol=3e-2)


def test_edge_attention_empty_rows_and_determinism():
    dev = torch.device("cuda")
    n, hl, hn = 128, 2, 16
    g = random_attn_graph(n, 100, seed=5).to(dev)          # most queries have no in-edges
    q, k, v = (torch.randn(n, hl, hn, device=dev, dtype=torch.bfloat16) for _ in range(3))
    a = edge_attention(q, k, v, g)
    b = edge_attention(q, k, v, g)
    assert torch.equal(a, b)
    deg = (g.rowptr[1:] - g.rowptr[:-1])
    assert float(a[deg == 0].abs().max()) == 0.0


@pytest.mark.parametrize("exph", [False, True])
@pytest.mark.parametrize("cfg", [(4, 4, 2, 4), (2, 6, 3, 5), (8, 0, 2, 4), (0, 5, 2, 3), (32, 32, 8, 8), (16, 16, 4, 6)])
def test_gpu_builder_matches_cpu_builder(cfg, exph):
    br, bw, w, l = cfg
    topo, _ = random_topology(700, 6000, hub_in=900, hub_out=400, seed=11)
    cpu = build_attn_graph(topo, br, bw, w, l, 77, exphormer=exph)
    gpu = build_attn_graph(topo.to("cuda"), br, bw, w, l, 77, exphormer=exph)
    assert torch.equal(cpu.rowptr, gpu.rowptr.cpu())
    assert torch.equal(cpu.col, gpu.col.cpu())
    if exph:
        assert torch.equal(cpu.etype, gpu.etype.cpu())
    assert cpu._totals.tolist() == gpu._totals.cpu().tolist()


@pytest.mark.parametrize("exph", [False, True])
@pytest.mark.parametrize("cfg", [(4, 4, 2, 4), (8, 8, 2, 4), (32, 16, 4, 6), (1, 0, 2, 4)])
def test_gpu_builder_ranks_long_rows_with_a_block_per_row(cfg, exph, monkeypatch):
    """Queries with more in-edges than the block threshold (one of 30,000 with many repeated sources, one just above
    the threshold, one just below it) are ranked by a thread block each: same graph as the CPU builder, as the device
    builder with the pre-pass switched off, and as a build of row ranges that cut between the long rows."""
    from budgetformer_b200.ops import _ext
    br, bw, w, l = cfg
    thr = int(_ext.load().BUILD_HUB_DEGREE)
    g = torch.Generator().manual_seed(5)
    n = 3000
    ei = torch.randint(0, n, (2, 20000), generator=g)
    extra = [torch.stack([torch.randint(0, 500, (30000,), generator=g), torch.full((30000,), 0)]),
             torch.stack([torch.randint(0, n, (thr + 1,), generator=g), torch.full((thr + 1,), 1700)]),
             torch.stack([torch.randint(0, n, (thr - 30,), generator=g), torch.full((thr - 30,), 2999)])]
    topo = Topology.from_edge_index(torch.cat([ei] + extra, 1), n)
    dev = topo.to("cuda")
    assert dev.in_hub_rows(thr).tolist() == [0, 1700]
    cpu = build_attn_graph(topo, br, bw, w, l, 91, exphormer=exph)
    gpu = build_attn_graph(dev, br, bw, w, l, 91, exphormer=exph)
    assert torch.equal(cpu.rowptr, gpu.rowptr.cpu()) and torch.equal(cpu.col, gpu.col.cpu())
    if exph:
        assert torch.equal(cpu.etype, gpu.etype.cpu())
    assert cpu._totals.tolist() == gpu._totals.cpu().tolist()
    # row ranges (what one rank of a sharded build selects): [0, 1500) holds the first long row, [1500, 3000) the second
    ext = _ext.load()
    cap = max(br + bw + (1 if exph else 0), 1)
    cols, cnts = [], []
    for begin in (0, 1500):
        ell_col = torch.empty(1500 * cap, dtype=torch.int32, device="cuda")
        ell_cnt = torch.empty(1500, dtype=torch.int32, device="cuda")
        ell_typ = torch.empty(1500 * cap, dtype=torch.uint8, device="cuda") if exph else None
        totals = torch.zeros(2, dtype=torch.int64, device="cuda")
        ext.budget_select_rows(dev.in_rowptr, dev.in_src, dev.out_rowptr, dev.out_col, n, br, bw, w, l, exph, 91, begin, 1500,
                               ell_col, ell_cnt, ell_typ, totals, dev.in_hub_rows(thr))
        cols.append(ell_col); cnts.append(ell_cnt)
    rowptr, col, _ = ext.ell_rows_to_csr(torch.cat(cols), torch.cat(cnts), None, n, cap)
    assert torch.equal(rowptr.cpu(), cpu.rowptr) and torch.equal(col.cpu(), cpu.col)
    monkeypatch.setenv("BF_BUILD_HUB_BLOCKS", "0")
    plain = build_attn_graph(dev, br, bw, w, l, 91, exphormer=exph)
    assert torch.equal(plain.col, gpu.col) and torch.equal(plain.rowptr, gpu.rowptr)


def test_gpu_builder_seed_changes_graph_and_is_reproducible():
    topo, _ = random_topology(500, 5000, seed=2)
    t = topo.to("cuda")
    a = build_attn_graph(t, 4, 4, 2, 4, 1)
    b = build_attn_graph(t, 4, 4, 2, 4, 1)
    c = build_attn_graph(t, 4, 4, 2, 4, 2)
    assert torch.equal(a.col, b.col) and torch.equal(a.rowptr, b.rowptr)
    assert not (a.col.numel() == c.col.numel() and torch.equal(a.col, c.col))


def test_extension_is_loaded_from_tree():
    from budgetformer_b200.ops import _ext
    mod = _ext.load()
    assert "budgetformer_b200/csrc/build" in mod.__file__.replace("\\", "/")


@pytest.mark.parametrize("hub", [False, True])
def test_device_transpose_matches_torch_path(hub):
    """csrc/graph_transpose.cu (radix sort over node-id bits + compaction) gives the same by-key view and the same
    dK/dV work list as the PyTorch construction used for CPU graphs."""
    from budgetformer_b200.graph.attn_graph import AttnGraph, add_virtual_node
    n = 5000
    g = random_attn_graph(n, 30000, hub_col=700, seed=3)
    if hub:
        g = add_virtual_node(g, n, n)                     # row 0 holds every node; key 0 is used by every query
    ref = AttnGraph(g.num_rows, g.rowptr.cpu(), g.col.cpu(), None).ensure_transpose()
    dev = AttnGraph(g.num_rows, g.rowptr.cuda(), g.col.cuda(), None).ensure_transpose()
    for name in ("t_rowptr", "t_row", "t_eid", "t_task", "t_split"):
        a, b = getattr(ref, name), getattr(dev, name).cpu()
        assert a.shape == b.shape and torch.equal(a.to(b.dtype), b), name
    assert ref.kv_slots == dev.kv_slots
    if hub:
        assert dev.kv_slots > 0 and dev.t_split.size(0) >= 1


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_batch_norm_kernels_match_pytorch(dtype):
    """Forward, running statistics and all three gradients of the row BatchNorm against nn.BatchNorm1d in fp32."""
    from budgetformer_b200.ops.norm import batch_norm
    torch.manual_seed(0)
    rows, h = 5003, 64
    x = (torch.randn(rows, h, device="cuda") * 1.7 + 0.6).to(dtype)
    bn = torch.nn.BatchNorm1d(h).cuda()
    ref = torch.nn.BatchNorm1d(h).cuda()
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5); bn.bias.uniform_(-0.5, 0.5)
        ref.weight.copy_(bn.weight); ref.bias.copy_(bn.bias)
    xa = x.clone().requires_grad_(True)
    xb = x.float().clone().requires_grad_(True)
    g = torch.randn(rows, h, device="cuda")
    for _ in range(2):                                   # second call uses a non-zero running mean as the shift
        ya = batch_norm(xa, bn)
        yb = ref(xb)
    (ya.float() * g).sum().backward()
    (yb * g).sum().backward()
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert ya.dtype == dtype and (ya.float() - yb).abs().max() < tol
    assert (bn.running_mean - ref.running_mean).abs().max() < 1e-3
    assert (bn.running_var - ref.running_var).abs().max() < 2e-3
    scale = xb.grad.abs().max()
    assert (xa.grad.float() - xb.grad).abs().max() < (4e-2 if dtype == torch.bfloat16 else 1e-4) * max(1.0, float(scale))
    ptol = 2e-2 if dtype == torch.bfloat16 else 2e-3
    assert (bn.weight.grad - ref.weight.grad).abs().max() < ptol * ref.weight.grad.abs().max() + 5e-2
    assert (bn.bias.grad - ref.bias.grad).abs().max() < ptol * ref.bias.grad.abs().max() + 5e-2
    bn.eval(); ref.eval()
    assert (batch_norm(x, bn).float() - ref(x.float())).abs().max() < tol


@pytest.mark.parametrize("variant", ["plain", "gps", "exphormer"])
def test_edge_attention_kernels_against_coo_oracle(variant):
    """Forward and backward of the CUDA kernels against the float32 oracle written on the reference's COO layout
    (hub row and hub key included)."""
    from budgetformer_b200 import oracle
    from tests.helpers import random_attn_graph
    torch.manual_seed(12)
    n, h, hn = 700, 4, 16
    g = random_attn_graph(n, 5000, hub_row=1500, hub_col=1400, seed=8, typed=variant == "exphormer").to("cuda")
    ei = g.edge_index()
    q, k, v = (torch.randn(n, h, hn, device="cuda", requires_grad=True) for _ in range(3))
    emb = torch.randn(2, h * hn, device="cuda")
    proj = torch.randn(h * hn, h * hn, device="cuda") * 0.1
    table = (emb @ proj.t()).view(2, h, hn) if variant == "exphormer" else None
    out = edge_attention(q, k, v, g, variant=variant, etable=table)
    if variant == "plain":
        ref = oracle.attention.sparse_attention(q, k, v, ei)
    elif variant == "gps":
        ref = oracle.attention.gps_attention(q, k, v, ei)
    else:
        ref = oracle.attention.exphormer_attention(q, k, v, ei, emb, proj)
    assert torch.allclose(out, ref, atol=2e-4, rtol=2e-4), float((out - ref).abs().max())
    dout = torch.randn_like(out)
    got = torch.autograd.grad(out, (q, k, v), dout)
    want = torch.autograd.grad(ref, (q, k, v), dout)
    for a, b, name in zip(got, want, "qkv"):
        assert torch.allclose(a, b, atol=5e-4, rtol=1e-3), (name, float((a - b).abs().max()))


def test_edge_attention_with_understated_degree_bound():
    """``max_degree`` is a hint from the graph builder.  A hint below the true maximum must not drop edges: rows longer
    than the hint are either walked by the regular kernels (no hub list) or by hub blocks that stride over their chunks."""
    from tests.helpers import random_attn_graph
    torch.manual_seed(3)
    n, hl, hn = 3000, 2, 16
    g = random_attn_graph(n, 6000, hub_row=20000, hub_col=2500, seed=5).to("cuda")
    q, k, v = (torch.randn(n, hl, hn, device="cuda") for _ in range(3))
    ref = edge_attention_reference(q, k, v, g)
    for wrong in (8, 1500):                     # below the hub threshold (no hub list at all) / above it but far too small
        g.max_degree = wrong
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        out = edge_attention(qq, kk, vv, g)
        assert torch.allclose(out, ref, atol=2e-4, rtol=2e-4), (wrong, float((out - ref).abs().max()))
        out.sum().backward()
        q2, k2, v2 = (t.clone().requires_grad_(True) for t in (q, k, v))
        edge_attention_reference(q2, k2, v2, g).sum().backward()
        for a, b in ((qq, q2), (kk, k2), (vv, v2)):
            assert torch.allclose(a.grad, b.grad, atol=1e-3, rtol=1e-3), wrong
