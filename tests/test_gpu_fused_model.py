"""Fused B200 layer path against the portable PyTorch path of the same model (single GPU)."""
import copy

import pytest
import torch

from budgetformer_b200.config import parse_fullgraph_args
from budgetformer_b200.graph.synthetic import sbm_graph
from budgetformer_b200.ops import gemm
from budgetformer_b200.train.data import GraphData, random_split_idx
from budgetformer_b200.train.engine import FullGraphTrainer

pytestmark = pytest.mark.gpu


def _trainer(model, fused, extra=()):
    n = 1536
    x, y, ei = sbm_graph(n, feat_dim=64, seed=3)
    data = GraphData(x, y, ei, random_split_idx(n, 3), n, 7)
    argv = ["--model", model, "--dataset", "t", "--n_layers", "2", "--hidden_dim", "128", "--num_heads", "8",
            "--ffn_dim", "256", "--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4",
            "--amp_dtype", "bf16", "--force_random_split", "--device", "cuda:0", "--fused_sp", "on" if fused else "off",
            "--dropout_rate", "0.0", "--attention_dropout_rate", "0.0", "--input_dropout_rate", "0.0", "--seed", "5"]
    argv += list(extra)
    return FullGraphTrainer(parse_fullgraph_args(argv), data=data, log=lambda *a, **k: None)


@pytest.mark.parametrize("model", ["gt", "graphormer", "graphgps", "exphormer"])
def test_fused_forward_backward_matches_portable(model):
    a = _trainer(model, fused=False)
    b = _trainer(model, fused=True)
    assert b.fused_sp and not a.fused_sp
    b.model.load_state_dict(a.model.state_dict())
    graph = a.build_edges(1)
    la, outa = a._loss(graph, a.local_idx["train"])
    lb, outb = b._loss(graph, b.local_idx["train"])
    assert torch.allclose(outa.float(), outb.float(), atol=6e-2, rtol=6e-2), float((outa.float() - outb.float()).abs().max())
    a.reducer.prepare_backward(); b.reducer.prepare_backward()
    la.backward(); lb.backward()
    gemm.check_status("cuda")
    gmax = max(float(p.grad.abs().max()) for p in a.model.parameters() if p.grad is not None)
    for (na, pa), (nb, pb) in zip(a.model.named_parameters(), b.model.named_parameters()):
        if pa.grad is None:
            continue
        ga, gb = pa.grad.float(), pb.grad.float()
        err = float((ga - gb).abs().max())
        # gradients that are analytically ~0 (e.g. the key bias under a normalised softmax) are pure rounding noise:
        # accept either a small relative error or an error far below the model's gradient scale
        ok = err <= 0.12 * max(float(ga.abs().max()), 1e-6) or err <= 5e-3 * gmax
        assert ok, f"{model}: grad mismatch on {na}: err {err} vs max {float(ga.abs().max())} (global {gmax})"
    assert abs(float(la.detach()) - float(lb.detach())) < 2e-2


@pytest.mark.parametrize("model", ["gt", "graphormer"])
def test_fused_training_reduces_loss(model):
    t = _trainer(model, fused=True, extra=["--peak_lr", "5e-3", "--dropout_rate", "0.1"])
    losses = [t.train_step(e)["loss"] for e in range(1, 26)]
    gemm.check_status("cuda")
    assert losses[-1] < losses[0] - 0.05, losses


def test_fused_path_with_activation_tiers():
    t = _trainer("gt", fused=True, extra=["--activation_checkpoint_mode", "all"])
    u = _trainer("gt", fused=True, extra=["--activation_checkpoint_mode", "ffn_only"])
    u.model.load_state_dict(t.model.state_dict())
    g = t.build_edges(1)
    t.model.train(); u.model.train()
    lt, _ = t._loss(g, t.local_idx["train"])
    lu, _ = u._loss(g, u.local_idx["train"])
    t.reducer.prepare_backward(); u.reducer.prepare_backward()
    lt.backward(); lu.backward()
    assert abs(float(lt) - float(lu)) < 1e-3
    for pa, pb in zip(t.model.parameters(), u.model.parameters()):
        assert torch.allclose(pa.grad, pb.grad, atol=1e-3 + 0.02 * float(pa.grad.abs().max()))


@pytest.mark.parametrize("graph", [False, True])
def test_flat_adamw_matches_torch_adamw_with_clipping(graph):
    """Eager launches and the CUDA-graph replay of the step (--cuda_graph) against torch.optim.AdamW + clip_grad_norm_,
    with a learning rate that changes every step."""
    from budgetformer_b200.ops.optim import FlatAdamW
    from budgetformer_b200.parallel.reducer import GradientReducer
    torch.manual_seed(0)
    net_a = torch.nn.Sequential(torch.nn.Linear(37, 64), torch.nn.LayerNorm(64), torch.nn.Linear(64, 5)).cuda()
    net_b = copy.deepcopy(net_a)
    red = GradientReducer(net_a, None, world_size=1)
    opt_a = FlatAdamW(red.buckets, lr=3e-3, weight_decay=0.05, max_grad_norm=0.5, cuda_graph=graph)
    opt_b = torch.optim.AdamW(net_b.parameters(), lr=3e-3, weight_decay=0.05)
    x = torch.randn(256, 37, device="cuda")
    for it in range(5):
        for opt in (opt_a, opt_b):
            opt.param_groups[0]["lr"] = 3e-3 * (1.0 - 0.1 * it)
        red.prepare_backward()
        (net_a(x) ** 2).sum().backward()
        opt_a.step()
        opt_b.zero_grad()
        (net_b(x) ** 2).sum().backward()
        torch.nn.utils.clip_grad_norm_(net_b.parameters(), 0.5)
        opt_b.step()
    for pa, pb in zip(net_a.parameters(), net_b.parameters()):
        assert torch.allclose(pa, pb, atol=2e-6, rtol=2e-5), float((pa - pb).abs().max())


def test_context_dropout_fused_into_attention_matches_separate_pass():
    """GT applies dropout to the attention context before the output projection.  Fused into the attention kernel's
    store (and undone in the <dout, out> term of its backward) it must reproduce the separate hash-dropout pass:
    same counter-based mask, same loss, same gradients."""
    from budgetformer_b200.ops import fused_sp
    results = {}
    for fuse in (True, False):
        torch.manual_seed(21)
        t = _trainer("gt", fused=True, extra=["--dropout_rate", "0.3"])
        graph = t.build_edges(1)
        seeds = iter(range(1000, 2000))
        old_flag, old_seed = fused_sp.FUSE_CONTEXT_DROPOUT, fused_sp.new_seed
        fused_sp.FUSE_CONTEXT_DROPOUT = fuse
        fused_sp.new_seed = lambda: next(seeds)          # identical seed sequence in both runs
        try:
            t.model.train()
            loss, out = t._loss(graph, t.local_idx["train"])
            t.reducer.prepare_backward()
            loss.backward()
        finally:
            fused_sp.FUSE_CONTEXT_DROPOUT, fused_sp.new_seed = old_flag, old_seed
            t.edge_engine.shutdown()
        results[fuse] = (float(loss.detach()), out.float().clone(),
                         {n: p.grad.float().clone() for n, p in t.model.named_parameters() if p.grad is not None})
    gemm.check_status("cuda")
    (la, oa, ga), (lb, ob, gb) = results[True], results[False]
    assert abs(la - lb) < 5e-3, (la, lb)
    assert (oa - ob).abs().max() < 5e-2
    gmax = max(float(g.abs().max()) for g in gb.values())
    for n in gb:
        err = float((ga[n] - gb[n]).abs().max())
        assert err <= 0.08 * max(float(gb[n].abs().max()), 1e-6) or err <= 4e-3 * gmax, (n, err)


@pytest.mark.parametrize("model", ["gt", "graphormer", "graphgps", "exphormer"])
def test_fused_layer_matches_fp32_oracle_layer(model):
    """One fused encoder layer (bf16 activations, tcgen05 GEMMs, edge-attention kernels) against the float32 CPU oracle
    of the reference's layer fed with the same weights and the same attention graph."""
    from budgetformer_b200 import oracle
    t = _trainer(model, fused=True, extra=["--num_global_node", "0"])
    t.model.train()                                        # BatchNorm on batch statistics, dropout rates are zero
    torch.manual_seed(9)
    layer = t.model.layers[0]
    for p in layer.parameters():
        torch.nn.init.normal_(p, std=0.08)
    graph = t.build_edges(1)
    n, h = t.nodes_per_rank, 128
    x = torch.randn(1, n, h, device="cuda").bfloat16()
    with torch.no_grad():
        got = layer(x, None, graph, "sparse").squeeze(0).float().cpu()
    gemm.check_status("cuda")
    weights = {k: v.detach().float().cpu() for k, v in layer.state_dict().items()}
    want = oracle.layers.LAYERS[model](x.squeeze(0).float().cpu(), weights, graph.edge_index().cpu(), 8)
    err = (got - want).abs()
    # bf16 keeps 8 bits: activations of order one carry ~4e-3 of rounding per stored tensor, a handful of them per layer
    assert float(err.max()) < 0.12 and float(err.mean()) < 0.012, (float(err.max()), float(err.mean()))


@pytest.mark.parametrize("model", ["gt", "graphgps"])
def test_fused_gradients_against_fp32_portable_run(model):
    """Gradients of the fused bf16 path against the portable path run entirely in float32 (no autocast): per tensor the
    error relative to the tensor's own norm stays within what bf16 storage of the activations explains."""
    a = _trainer(model, fused=False, extra=["--amp_dtype", "none"])
    b = _trainer(model, fused=True)
    b.model.load_state_dict(a.model.state_dict())
    graph = a.build_edges(1)
    la, _ = a._loss(graph, a.local_idx["train"])
    lb, _ = b._loss(graph, b.local_idx["train"])
    a.reducer.prepare_backward(); b.reducer.prepare_backward()
    la.backward(); lb.backward()
    gemm.check_status("cuda")
    assert abs(float(la.detach()) - float(lb.detach())) < 1e-2
    norms = {n: float(p.grad.float().norm()) for n, p in a.model.named_parameters() if p.grad is not None}
    top = max(norms.values())
    worst = 0.0
    for (na, pa), (_nb, pb) in zip(a.model.named_parameters(), b.model.named_parameters()):
        if pa.grad is None or norms[na] < 1e-3 * top:       # analytically (near-)zero gradients are rounding noise
            continue
        rel = float((pa.grad.float() - pb.grad.float()).norm()) / norms[na]
        worst = max(worst, rel)
        assert rel < 0.05, f"{model}: {na}: relative gradient error {rel:.4f}"
    assert worst > 0.0
