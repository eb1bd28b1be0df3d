import math

import pytest
import torch

from budgetformer_b200.config import build_fullgraph_parser, parse_fullgraph_args
from budgetformer_b200.graph.engine import resolve_budget_state
from budgetformer_b200.utils.lr import build_lr_scheduler, cosine_with_warmup_value, polynomial_decay_value, schedule_epochs


def test_reference_flags_and_defaults():
    a = parse_fullgraph_args([])
    assert a.peak_lr == 1e-3 and a.warmup_updates == 5 and a.sequence_parallel_size == 1 and a.num_global_node == 1
    assert a.dataset == "ogbn-arxiv" and a.to_bidirected is True            # arxiv forces bidirected
    assert a.model == "graphormer" and a.hidden_dim == 64 and a.ffn_dim == 256 and a.n_layers == 4
    assert a.walk_length == 4 and a.walks_per_node == 2 and a.distributed_backend == "nccl"
    names = {x.dest for x in build_fullgraph_parser()._actions}
    for flag in ("dataset_dir split_id hops pe_dim expander_degree attn_bias_dim tot_updates lr_ref_batch_size end_lr "
                 "lr_schedule save_model model_dir rw_edge_mode fanout edge_build_device rank local_rank world_size "
                 "distributed_timeout_minutes force_random_split node_sample_ratio activation_checkpoint_mode amp_dtype "
                 "activation_cpu_offload profile_sp_comm multi_tier_gpu_memory_limit_mib force_multi_tier_plan "
                 "disable_edge_prefetch random_edge_blocks max_total_edges_per_query adaptive_edge_budget "
                 "adaptive_edge_budget_probe_size adaptive_edge_budget_block_size adaptive_edge_budget_warmup_epochs "
                 "adaptive_edge_budget_patience adaptive_edge_budget_static_seed_epochs include_real_edges to_bidirected "
                 "force_edge_broadcast fixed_real_edges_per_query fixed_rw_edges_per_query fixed_walk_length seq_len "
                 "multi_tier_probe_cpu_broadcast").split():
        assert flag in names, flag


def test_normalisation_rules():
    a = parse_fullgraph_args(["--model", "gt", "--attn_type", "full", "--dataset", "x"])
    assert a.attn_type == "sparse" and a.num_global_node == 0
    a = parse_fullgraph_args(["--model", "graphgps", "--attn_type", "full", "--dataset", "x"])
    assert a.attn_type == "full"
    with pytest.raises(ValueError):
        parse_fullgraph_args(["--fixed_real_edges_per_query", "4"])
    with pytest.raises(ValueError):
        parse_fullgraph_args(["--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "2", "--walks_per_node", "0"])
    with pytest.raises(ValueError):
        parse_fullgraph_args(["--adaptive_edge_budget", "--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "2"])
    with pytest.raises(ValueError):
        parse_fullgraph_args(["--node_sample_ratio", "0"])
    with pytest.raises(ValueError):
        parse_fullgraph_args(["--num_global_node", "2"])
    with pytest.raises(SystemExit):
        parse_fullgraph_args(["--activation_checkpoint_mode", "bogus"])


def test_budget_decision_table():
    a = parse_fullgraph_args(["--dataset", "x"])
    s = resolve_budget_state(a)
    assert (s.use_real, s.use_rw, s.b_real, s.b_rw) == (False, True, None, None)
    a = parse_fullgraph_args(["--dataset", "x", "--include_real_edges", "1", "--walks_per_node", "0"])
    s = resolve_budget_state(a)
    assert (s.use_real, s.use_rw) == (True, False)
    a = parse_fullgraph_args(["--dataset", "x", "--random_edge_blocks", "--max_total_edges_per_query", "9"])
    s = resolve_budget_state(a)
    assert (s.b_real, s.b_rw) == (5, 4)
    a = parse_fullgraph_args(["--dataset", "x", "--random_edge_blocks", "--max_total_edges_per_query", "9", "--walks_per_node", "0"])
    assert resolve_budget_state(a).b_real == 9 and not resolve_budget_state(a).use_rw
    s = resolve_budget_state(a, {"real_edges_per_query": 0, "rw_edges_per_query": 6})
    assert not s.use_real


def test_lr_schedules():
    assert polynomial_decay_value(1, 5, 100, 1e-3, 1e-9, 1.0) == pytest.approx(2e-4)
    assert polynomial_decay_value(5, 5, 100, 1e-3, 1e-9, 1.0) == pytest.approx(1e-3)
    assert polynomial_decay_value(100, 5, 100, 1e-3, 1e-9, 1.0) == 1e-9
    mid = polynomial_decay_value(52, 5, 100, 1e-3, 1e-9, 1.0)
    assert mid == pytest.approx((1e-3 - 1e-9) * (1 - 47 / 95) + 1e-9)
    assert cosine_with_warmup_value(3, 6, 60, 1.0) == pytest.approx(0.5)
    assert cosine_with_warmup_value(33, 6, 60, 1.0) == pytest.approx(0.5 * (1 + math.cos(math.pi * 0.5)))
    a = parse_fullgraph_args(["--dataset", "x", "--tot_updates", "1000", "--warmup_updates", "100", "--lr_ref_batch_size", "1000"])
    assert schedule_epochs(a, n_train=10_000) == (10, 100)
    opt = torch.optim.AdamW([torch.nn.Parameter(torch.zeros(1))], lr=1e-3)
    a = parse_fullgraph_args(["--dataset", "x", "--epochs", "10", "--warmup_updates", "2"])
    sch = build_lr_scheduler(a, opt)
    lrs = []
    for _ in range(4):
        lrs.append(opt.param_groups[0]["lr"])
        opt.step(); sch.step()
    assert lrs[0] == pytest.approx(5e-4) and lrs[1] == pytest.approx(1e-3) and lrs[2] < lrs[1]
