"""Model structure: state_dict layouts of the reference, shapes, key-form compatibility."""
import pytest
import torch

from budgetformer_b200.config import parse_fullgraph_args
from budgetformer_b200.graph.attn_graph import AttnGraph, add_virtual_node
from budgetformer_b200.train.checkpoint import normalize_state_dict_keys
from budgetformer_b200.train.engine import build_model


def _model(name, extra=()):
    a = parse_fullgraph_args(["--dataset", "x", "--model", name, "--n_layers", "2", "--hidden_dim", "32", "--num_heads", "4",
                              "--ffn_dim", "48"] + list(extra))
    return build_model(a, 10, 5), a


def test_gt_state_dict_layout():
    m, _ = _model("gt")
    keys = set(m.state_dict())
    for k in ("node_encoder.weight", "layers.0.self_attention.linear_q.weight", "layers.0.self_attention.linear_v.bias",
              "layers.1.O.weight", "layers.1.layer_norm1.weight", "layers.0.FFN_layer1.weight", "layers.0.FFN_layer2.bias",
              "layers.0.layer_norm2.bias", "MLP_layer.FC_layers.0.weight", "MLP_layer.FC_layers.2.bias"):
        assert k in keys, k
    sd = m.state_dict()
    assert sd["layers.0.FFN_layer1.weight"].shape == (64, 32) and sd["MLP_layer.FC_layers.0.weight"].shape == (16, 32)
    assert sd["MLP_layer.FC_layers.1.weight"].shape == (8, 16) and sd["MLP_layer.FC_layers.2.weight"].shape == (5, 8)
    assert not any("output_layer" in k for k in keys)


def test_graphormer_state_dict_layout():
    m, _ = _model("graphormer")
    sd = m.state_dict()
    for k in ("layers.0.self_attention_norm.weight", "layers.0.self_attention.output_layer.bias", "layers.1.ffn_norm.bias",
              "layers.0.ffn.layer1.weight", "layers.0.ffn.layer2.weight", "final_ln.weight", "downstream_out_proj.weight",
              "graph_token.weight", "graph_token_virtual_distance.weight", "attn_bias_proj.weight"):
        assert k in sd, k
    assert sd["layers.0.ffn.layer1.weight"].shape == (48, 32) and sd["graph_token.weight"].shape == (1, 32)
    assert sd["attn_bias_proj.weight"].shape == (4, 1) and "attn_bias_proj.bias" not in sd


def test_graphgps_state_dict_layout():
    m, _ = _model("graphgps")
    sd = m.state_dict()
    assert "layers.0.self_attention.linear_q.bias" not in sd and "layers.0.self_attention.out_proj.bias" in sd
    assert "layers.0.self_attention.dist_attn.local_attn.performer.projection_matrix" in sd
    for k in ("layers.0.norm1.running_mean", "layers.1.norm2.num_batches_tracked", "layers.0.ffn1.weight", "output_proj.weight"):
        assert k in sd, k
    hn = 8
    assert sd["layers.0.self_attention.dist_attn.local_attn.performer.projection_matrix"].shape == (int(hn * torch.log(torch.tensor(float(hn)))), hn)
    full, _ = _model("graphgps", ["--attn_type", "full"])
    assert "layers.0.self_attention.linear_q.bias" in full.state_dict()


def test_exphormer_state_dict_layout():
    m, _ = _model("exphormer")
    sd = m.state_dict()
    assert sd["layers.0.self_attention.dist_attn.local_attn.edge_type_emb.weight"].shape == (2, 32)
    assert sd["layers.0.self_attention.dist_attn.local_attn.edge_proj.weight"].shape == (32, 32)
    assert "layers.0.self_attention.linear_k.bias" not in sd and not any("out_proj" in k or ".O." in k for k in sd)


def test_nagphormer_layout_and_forward():
    m, a = _model("nagphormer", ["--hops", "3"])
    sd = m.state_dict()
    for k in ("att_embeddings_nope.weight", "layers.0.self_attention.output_layer.weight", "final_ln.bias", "out_proj.weight",
              "attn_layer.weight", "Linear1.weight", "scaling"):
        assert k in sd, k
    out = m(torch.randn(7, 4 * 10 // 4 * 4).view(7, 4, 10)[:, :, :2].reshape(7, 8), None, None)
    assert out.shape == (7, 5)


def test_single_process_key_form_is_accepted_on_load():
    m, _ = _model("exphormer")
    sd = {k.replace("dist_attn.local_attn.", "dist_attn."): v for k, v in m.state_dict().items()}
    assert any("dist_attn.edge_proj" in k for k in sd)
    m.load_state_dict(normalize_state_dict_keys(sd, m))


@pytest.mark.parametrize("name", ["gt", "graphgps", "exphormer", "graphormer"])
def test_forward_shapes_and_coo_input(name):
    m, a = _model(name)
    n = 12
    ei = torch.randint(0, n, (2, 40))
    x = torch.randn(n, 10)
    if name == "graphormer":
        g = add_virtual_node(AttnGraph.from_edge_index(ei, n), n, n)
        out = m(x, None, g, attn_type="sparse")
        # the COO form with the virtual node at id 0 gives the same result
        out2 = m.eval()(x, None, g.edge_index(), attn_type="sparse")
        m.train()
    else:
        typed = torch.cat([ei, torch.randint(0, 2, (1, 40))]) if name == "exphormer" else ei
        m.eval()
        out = m(x, None, typed, attn_type="sparse")
        out2 = m(x, None, AttnGraph.from_edge_index(typed, n), attn_type="sparse")
    assert out.shape == (n, 5) and torch.isfinite(out).all()
    if name != "graphormer":
        assert torch.allclose(out, out2, atol=1e-5)
    assert torch.allclose(out.exp().sum(1), torch.ones(n), atol=1e-4)


def test_gt_rejects_dense_attention_and_init_scale():
    m, _ = _model("gt")
    with pytest.raises(ValueError):
        m(torch.randn(4, 10), None, torch.zeros(2, 0, dtype=torch.long), attn_type="full")
    std = float(m.layers[0].O.weight.std())
    assert abs(std - 0.02 / 2 ** 0.5) < 0.004
    assert float(m.layers[0].O.bias.abs().sum()) == 0


def test_dense_attention_capture_extra_bias_and_hop_mass():
    """Research hooks of the dense path: per-layer capture of the head-averaged probabilities, an additive extra bias
    per layer, and hop-mass tracking against a hop matrix of sampled queries."""
    from budgetformer_b200.utils.analytics import bfs_hop_matrix
    m, _ = _model("graphgps", ["--attn_type", "full"])
    m.eval()
    n = 12
    x = torch.randn(n, 10)
    ring = torch.stack([torch.arange(n), (torch.arange(n) + 1) % n])
    m.set_full_attention_capture_layers(True, "all")
    with torch.no_grad():
        base = m(x, None, ring, attn_type="full")
    means = m.get_full_attention_means_per_layer("all")
    assert len(means) == 2 and all(a.shape == (1, n, n) for a in means)
    assert torch.allclose(means[0].sum(-1), torch.ones(1, n), atol=1e-5)
    assert m.get_last_layer_full_attention_mean() is means[1]
    # a bias that forbids every key but the query itself makes the captured attention the identity
    mask = torch.full((n, n), -1e9)
    mask.fill_diagonal_(0.0)
    m.set_last_layer_full_attention_extra_bias(mask)
    with torch.no_grad():
        biased = m(x, None, ring, attn_type="full")
    last = m.get_last_layer_full_attention_mean()
    assert torch.allclose(last[0], torch.eye(n), atol=1e-6) and not torch.allclose(biased, base)
    first = m.get_full_attention_means_per_layer("all")[0]
    assert torch.allclose(first, means[0], atol=1e-6)                    # only the last layer got the bias
    with pytest.raises(ValueError):
        m.set_full_attention_extra_biases([mask], "all")
    m.set_full_attention_extra_biases(None)
    m.set_full_attention_capture_layers(False)
    assert m.get_last_layer_full_attention_mean() is None
    # hop mass on the dense path
    queries = torch.tensor([0, 5])
    hop = bfs_hop_matrix(ring, n, queries, max_hop=6)
    m.enable_hop_mass_tracking(mass=0.9, max_batches=4, max_hop=6)
    for core in m.core_attention_modules():
        core.hop_queries, core.hop_matrix = queries, hop
    with torch.no_grad():
        m(x, None, ring, attn_type="full")
    stats = m.get_hop_mass_stats_per_layer()
    assert len(stats) == 2 and abs(sum(stats[0]["hop_mass"]) - 1.0) < 1e-4
    m.disable_hop_mass_tracking()
    assert m.get_hop_mass_stats_per_layer() == [None, None]


@pytest.mark.parametrize("name", ["gt", "graphormer"])
def test_one_edge_set_per_head_group(name):
    """A list of edge sets: consecutive head groups attend over their own set (the legacy per-head subgraph views).
    Two identical sets reproduce the single-set output; with one set missing its heads contribute nothing."""
    from budgetformer_b200.graph.legacy_samplers import GroupedHeadSubgraphProvider
    m, _ = _model(name, ["--num_global_node", "0"] if name == "graphormer" else [])
    m.eval()
    n = 16
    g = torch.Generator().manual_seed(0)
    x = torch.randn(n, 10, generator=g)
    ei = torch.cat([torch.randint(0, n, (2, 60), generator=g), torch.arange(n).repeat(2, 1)], 1)
    with torch.no_grad():
        single = m(x, None, ei, attn_type="sparse")
        twice = m(x, None, [ei, ei], attn_type="sparse")
        half = m(x, None, [ei, None], attn_type="sparse")
        views = GroupedHeadSubgraphProvider(2).build(ei, 4)                # 4 heads in 2 groups, edges split by source id
        grouped = m(x, None, [views[0], views[2]], attn_type="sparse")
    assert torch.allclose(single, twice, atol=1e-5)
    assert torch.isfinite(half).all() and torch.isfinite(grouped).all()
    # group-wise check at the attention module: heads 0-1 over set A, heads 2-3 over set B
    core = next(iter(m.core_attention_modules()))
    q, k, v = (torch.randn(1, n, 4, 8, generator=g) for _ in range(3))
    a, b = views[0], views[2]
    both = core(q, k, v, None, [a, b], "sparse").reshape(1, n, 4, 8)
    only_a = core(q[:, :, :2].contiguous(), k[:, :, :2].contiguous(), v[:, :, :2].contiguous(), None, a, "sparse").reshape(1, n, 2, 8)
    only_b = core(q[:, :, 2:].contiguous(), k[:, :, 2:].contiguous(), v[:, :, 2:].contiguous(), None, b, "sparse").reshape(1, n, 2, 8)
    assert torch.allclose(both[:, :, :2], only_a, atol=1e-6) and torch.allclose(both[:, :, 2:], only_b, atol=1e-6)
    missing = core(q, k, v, None, [a, None], "sparse").reshape(1, n, 4, 8)
    assert torch.allclose(missing[:, :, :2], only_a, atol=1e-6) and float(missing[:, :, 2:].abs().sum()) == 0.0


def test_graphormer_head_group_sets_with_dense_bias():
    m, _ = _model("graphormer", ["--num_global_node", "0"])
    core = next(iter(m.core_attention_modules()))
    n = 10
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, n, 4, 8, generator=g) for _ in range(3))
    ei = torch.cat([torch.randint(0, n, (2, 30), generator=g), torch.arange(n).repeat(2, 1)], 1)
    bias = torch.randn(1, 4, n, n, generator=g)
    one = core(q, k, v, bias, ei, "sparse")
    two = core(q, k, v, bias, [ei, ei], "sparse")
    assert torch.allclose(one, two, atol=1e-5)
    assert not torch.allclose(one, core(q, k, v, None, ei, "sparse"), atol=1e-4)


def test_two_phase_sparse_attention_equals_one_pass():
    m, _ = _model("graphormer", ["--num_global_node", "0"])
    core = next(iter(m.core_attention_modules()))
    n = 14
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(1, n, 4, 8, generator=g) for _ in range(3))
    ei = torch.cat([torch.randint(0, n, (2, 50), generator=g), torch.arange(n - 2).repeat(2, 1)], 1)   # two queries without edges
    ctx = core.sparse_score_phase(q, k, ei)
    two = core.sparse_aggregate_phase(ctx, v).reshape(1, n, -1)
    one = core(q, k, v, None, ei, "sparse")
    assert torch.allclose(one, two, atol=1e-5)
