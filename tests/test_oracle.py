"""The CPU oracle (``budgetformer_b200.oracle``) against the framework's portable paths: the same mathematics written
twice, once on the reference's int64 COO layout and once on the framework's containers, must agree."""
import numpy as np
import pytest
import torch

from budgetformer_b200 import oracle
from budgetformer_b200.graph.attn_graph import AttnGraph, add_virtual_node
from budgetformer_b200.graph.builder import build_attn_graph
from budgetformer_b200.graph.builder_spec import random_walks
from budgetformer_b200.ops.edge_attention import dropout_keep_mask, edge_attention_reference
from tests.helpers import random_topology


def _graph(n=120, e=900, seed=0, typed=False):
    g = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (e,), generator=g)
    dst = torch.randint(0, n, (e,), generator=g)
    rows = [src, dst]
    if typed:
        rows.append(torch.randint(0, 2, (e,), generator=g))
    ei = torch.stack(rows)
    return ei, AttnGraph.from_edge_index(ei, n)


def _coo(graph: AttnGraph):
    return graph.edge_index()


@pytest.mark.parametrize("variant", ["plain", "gps", "exphormer"])
def test_oracle_attention_equals_portable_attention(variant):
    torch.manual_seed(1)
    n, h, hn = 120, 4, 8
    _, g = _graph(n, typed=variant == "exphormer")
    q, k, v = (torch.randn(n, h, hn) for _ in range(3))
    ei = _coo(g)
    if variant == "plain":
        want = oracle.attention.sparse_attention(q, k, v, ei)
        got = edge_attention_reference(q, k, v, g)
    elif variant == "gps":
        p, seed = 0.3, 77
        eid, heads = torch.arange(ei.size(1))[:, None], torch.arange(h)[None, :]
        keep = dropout_keep_mask(seed, eid, heads, p)
        want = oracle.attention.gps_attention(q, k, v, ei, keep, p)
        got = edge_attention_reference(q, k, v, g, variant="gps", dropout_p=p, dropout_seed=seed)
    else:
        emb, proj = torch.randn(2, h * hn), torch.randn(h * hn, h * hn) * 0.2
        want = oracle.attention.exphormer_attention(q, k, v, ei, emb, proj)
        table = (emb @ proj.t()).view(2, h, hn)
        got = edge_attention_reference(q, k, v, g, variant="exphormer", etable=table)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
    # a query without in-edges outputs zeros
    empty = torch.ones(n, dtype=torch.bool)
    empty[ei[1]] = False
    if empty.any():
        assert float(want[empty].abs().max()) == 0.0


def test_oracle_attention_bias_is_added_after_the_clamp():
    torch.manual_seed(2)
    n, h, hn = 40, 2, 8
    ei, g = _graph(n, 200)
    q, k, v = (torch.randn(n, h, hn) * 4 for _ in range(3))          # large scores: the clamp is active
    bias = torch.randn(g.num_edges, h)
    want = oracle.attention.sparse_attention(q, k, v, _coo(g), bias)
    got = edge_attention_reference(q, k, v, g, edge_bias=bias)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)
    s = oracle.attention.edge_scores(q, k, _coo(g))
    assert float(s.max()) == 5.0 and float(s.min()) == -5.0


@pytest.mark.parametrize("model", ["gt", "graphormer", "graphgps", "exphormer"])
def test_oracle_layer_equals_model_layer(model):
    """One encoder layer of the model classes (portable path, dropout off, BatchNorm on batch statistics) against the
    oracle fed with the layer's own state_dict."""
    from budgetformer_b200.config import parse_fullgraph_args
    from budgetformer_b200.train.engine import build_model
    torch.manual_seed(3)
    n, hdim, heads = 96, 32, 4
    args = parse_fullgraph_args(["--model", model, "--n_layers", "1", "--hidden_dim", str(hdim), "--num_heads", str(heads),
                                 "--ffn_dim", "64", "--dropout_rate", "0", "--attention_dropout_rate", "0",
                                 "--input_dropout_rate", "0", "--num_global_node", "0"])
    m = build_model(args, 16, 5)
    m.train()
    for p in m.parameters():                                   # the default initialisation is tiny: make every term count
        torch.nn.init.normal_(p, std=0.3)
    layer = m.layers[0]
    ei, g = _graph(n, 700, seed=4, typed=model == "exphormer")
    x = torch.randn(1, n, hdim)
    got = layer(x, None, g, "sparse").squeeze(0)
    weights = {k: v.detach() for k, v in layer.state_dict().items()}
    want = oracle.layers.LAYERS[model](x.squeeze(0), weights, _coo(g), heads)
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), float((got - want).abs().max())


def test_oracle_budgeted_edges_equal_the_builders():
    topo, ei = random_topology(150, 1400, hub_in=200, seed=5)
    seed, b_real, b_walk, w, l = 31, 3, 4, 2, 4
    walks = random_walks(topo, w, l, seed)
    ws, wd = oracle.graph.walk_edges(walks)
    src, dst = oracle.graph.budgeted_edges(ei[0].numpy(), ei[1].numpy(), ws, wd, b_real, b_walk, seed)
    g = build_attn_graph(topo, b_real, b_walk, w, l, seed)
    assert g.col.tolist() == src.tolist() and g.row_ids().tolist() == dst.tolist()


def test_oracle_sampler_is_nested_and_keeps_small_rows_whole():
    rng = np.random.default_rng(6)
    src, dst = rng.integers(0, 50, 600), rng.integers(0, 50, 600)
    prev = set()
    for k in (1, 2, 4, 8):
        idx = oracle.graph.sample_per_query(src, dst, k, 99)
        cur = set(zip(src[idx].tolist(), dst[idx].tolist()))
        assert prev <= cur                                       # common random numbers: top-k nested in top-(k+1)
        prev = cur
    few = oracle.graph.sample_per_query(np.array([3, 4]), np.array([9, 9]), 8, 1)
    assert few.tolist() == [0, 1]


def test_oracle_walk_edge_rule():
    walks = np.array([[0, 1, 2, 2, 2],          # reaches a sink at hop 2 and stays: hops 3, 4 emit nothing
                      [5, 5, 6, 5, 5]])         # a sink start repeats itself at hop 1 (kept), moves, comes back, stalls
    s, d = oracle.graph.walk_edges(walks)
    assert sorted(zip(s.tolist(), d.tolist())) == [(1, 0), (2, 0), (5, 5), (5, 5), (6, 5)]


def test_oracle_virtual_node_maps_equal_add_virtual_node():
    n, per = 12, 4
    ei, g = _graph(n, 40, seed=7)
    v = add_virtual_node(g, n, per)
    got = set(zip(v.col.tolist(), v.row_ids().tolist()))
    s, d = oracle.graph.add_virtual_node(_coo(g)[0].numpy(), _coo(g)[1].numpy(), n, per)
    assert got == set(zip(s.tolist(), d.tolist()))
    assert v.num_rows == n + n // per                            # P copies of the token in the gathered sequence


def test_oracle_reducer_and_loss_rule():
    grads = [torch.full((3,), float(r)) for r in range(4)]
    assert torch.allclose(oracle.reducer.mean_of_rank_gradients(grads), torch.full((3,), 1.5))
    lp = torch.log_softmax(torch.randn(6, 3, requires_grad=True), 1)
    y = torch.tensor([0, 1, 2, 0, 1, 2])
    idx = torch.tensor([1, 4])
    assert torch.allclose(oracle.reducer.rank_loss(lp, y, idx), torch.nn.functional.nll_loss(lp[idx], y[idx]))
    zero = oracle.reducer.rank_loss(lp, y, torch.zeros(0, dtype=torch.long))
    assert float(zero) == 0.0 and zero.requires_grad


def test_oracle_schedules_equal_the_schedulers():
    from budgetformer_b200.utils.lr import cosine_with_warmup_value, polynomial_decay_value
    for step in (0, 1, 3, 5, 6, 50, 100, 130):
        assert abs(oracle.schedules.cosine_with_warmup(step, 5, 100, 1e-3) - cosine_with_warmup_value(step, 5, 100, 1e-3)) < 1e-12
        assert abs(oracle.schedules.polynomial_decay(step, 5, 100, 1e-3, 1e-9) - polynomial_decay_value(step, 5, 100, 1e-3, 1e-9, 1.0)) < 1e-12
