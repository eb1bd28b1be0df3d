"""Command-line surface.

Every flag of the reference's ``main_node_fullgraph_sp.py`` / ``main_node_sp.py`` is accepted with
the same name, type, default and choices (utils/parser_node_level.py:4-405, driver-level default
overrides main_node_fullgraph_sp.py:188-206) and the same post-parse normalisation
(:408-477).  Flags are declared in tables; additive flags of this framework are grouped at the end.
"""
from __future__ import annotations

import argparse
from typing import Dict, Iterable, Optional

_STORE_TRUE = object()

# (flags, type, default, extra kwargs)
_COMMON = [
    (("--dataset_dir",), str, "./dataset/", {}),
    (("--dataset",), str, "ogbn-arxiv", {}),
    (("--split_id",), int, 0, {"help": "split index for datasets that ship several fixed splits"}),
    (("--model",), str, "graphormer", {"choices": ["graphormer", "gt", "exphormer", "graphgps", "nagphormer"]}),
    (("--hops",), int, 0, {"help": "K-hop feature pre-aggregation (0 = off); NAGphormer needs >= 1"}),
    (("--pe_dim",), int, 0, {"help": "Laplacian positional-encoding dimension (0 = off)"}),
    (("--expander_degree",), int, 0, {"help": "[Exphormer] degree of the random expander graph (0 = off)"}),
    (("--n_layers",), int, 4, {}),
    (("--num_heads",), int, 8, {}),
    (("--hidden_dim",), int, 64, {}),
    (("--ffn_dim",), int, 256, {}),
    (("--attn_bias_dim",), int, 1, {}),
    (("--dropout_rate",), float, 0.3, {}),
    (("--input_dropout_rate",), float, 0.1, {}),
    (("--attention_dropout_rate",), float, 0.5, {}),
    (("--num_global_node",), int, 1, {}),
    (("--attn_type",), str, "sparse", {"help": "sparse/full/flash/performer"}),
    (("--weight_decay",), float, 0.01, {}),
    (("--warmup_updates",), int, 10, {}),
    (("--tot_updates",), int, 0, {"help": "total LR-schedule steps in mini-batch units; 0 = epochs"}),
    (("--lr_ref_batch_size",), int, 1000, {}),
    (("--epochs",), int, 300, {}),
    (("--eval_every",), int, 5, {}),
    (("--peak_lr",), float, 2e-4, {}),
    (("--end_lr",), float, 1e-9, {}),
    (("--lr_schedule",), str, "polynomial", {"choices": ["polynomial", "cosine_with_warmup"]}),
    (("--seed",), int, 42, {}),
    (("--save_model",), _STORE_TRUE, False, {}),
    (("--model_dir",), str, "./model_ckpt/", {}),
    (("--walk_length",), int, 4, {}),
    (("--walks_per_node",), int, 2, {}),
    (("--rw_edge_mode",), str, "random_walk", {"choices": ["random_walk", "dgl_neighbor"]}),
    (("--fanout",), str, "10,5", {"help": "per-hop fanout for --rw_edge_mode dgl_neighbor"}),
    (("--edge_build_device",), str, "gpu", {"help": "gpu|cpu|cuda|cuda:N ('same' = gpu)"}),
    (("--rank",), int, None, {}),
    (("--local-rank", "--local_rank"), int, None, {}),
    (("--world-size",), int, None, {}),
    (("--distributed-backend",), str, "nccl", {"choices": ["nccl", "gloo", "ccl"]}),
    (("--distributed-timeout-minutes",), int, 10, {}),
    (("--sequence-parallel-size",), int, 4, {}),
]

_BATCH_SP = [
    (("--batch_subgraph_mode",), str, "induced", {"choices": ["induced", "seed_rw"]}),
    (("--batch_reorder_parts",), int, 0, {}),
    (("--seed_batch_size",), int, None, {}),
    (("--seq_len",), int, 256000, {}),
    (("--full_attn_hop_stats",), _STORE_TRUE, False, {}),
    (("--full_attn_hop_mass",), float, 0.95, {}),
    (("--full_attn_hop_max_queries",), int, 64, {}),
    (("--full_attn_hop_query_sampling",), str, "random", {"choices": ["random", "prefix"]}),
    (("--full_attn_hop_max_batches",), int, 1, {}),
    (("--full_attn_hop_max_hop",), int, 64, {}),
    (("--full_attn_hop_stats_dir",), str, "./plot/hop_stats", {}),
    (("--full_attn_hop_stats_tag",), str, "", {}),
    (("--attn_bias_mode",), str, "none", {"choices": ["none", "local_spd"]}),
    (("--attn_bias_max_dist",), int, 5, {}),
]

_FULLGRAPH = [
    (("--force_random_split",), _STORE_TRUE, False, {}),
    (("--node_sample_ratio",), float, 1.0, {}),
    (("--activation_checkpoint_mode",), str, None, {"choices": ["all", "ffn_only", "adaptive", "multi_tier"]}),
    (("--amp_dtype",), str, "none", {"choices": ["none", "bf16", "fp16"]}),
    (("--activation_cpu_offload",), _STORE_TRUE, False, {}),
    (("--profile_sp_comm",), _STORE_TRUE, False, {}),
    (("--multi_tier_gpu_memory_limit_mib",), int, 0, {}),
    (("--force_multi_tier_plan",), str, "", {}),
    (("--disable_edge_prefetch",), _STORE_TRUE, False, {}),
    (("--random_edge_blocks",), _STORE_TRUE, False, {}),
    (("--max_total_edges_per_query",), int, 0, {}),
    (("--adaptive_edge_budget",), _STORE_TRUE, False, {}),
    (("--adaptive_edge_budget_probe_size",), int, 0, {}),
    (("--adaptive_edge_budget_block_size",), int, 0, {}),
    (("--adaptive_edge_budget_warmup_epochs",), int, -1, {}),
    (("--adaptive_edge_budget_patience",), int, 0, {}),
    (("--adaptive_edge_budget_static_seed_epochs",), int, 0, {}),
    (("--include_real_edges",), int, 0, {}),
    (("--to_bidirected",), _STORE_TRUE, False, {}),
    (("--force_edge_broadcast",), _STORE_TRUE, False, {}),
    (("--fixed_real_edges_per_query",), int, None, {}),
    (("--fixed_rw_edges_per_query",), int, None, {}),
    (("--fixed_walk_length",), int, None, {}),
    (("--seq_len",), int, 0, {"help": "compat arg for shared launch scripts"}),
    (("--multi_tier_probe_cpu_broadcast",), _STORE_TRUE, False, {"help": "deprecated no-op"}),
]

# Additive flags (not in the reference).
_EXTRA = [
    (("--resume",), str, "", {"help": "path of a *.train_state.pt sidecar to resume from"}),
    (("--device",), str, "", {"help": "override the training device (e.g. cpu)"}),
    (("--multilabel",), _STORE_TRUE, False, {"help": "y is [N, C] multi-hot; train with BCE-with-logits"}),
    (("--fused_sp",), str, "auto", {"choices": ["auto", "on", "off"],
                                     "help": "fused projection + all-to-all kernels over symmetric memory"}),
    (("--sync_batchnorm",), _STORE_TRUE, False, {"help": "all-reduce BatchNorm statistics over SP ranks"}),
    (("--metrics_jsonl",), str, "", {"help": "write one JSON line per epoch (device-timed)"}),
    (("--fault_inject",), str, "", {"help": "host-side fault injection spec, <kind>@<phase>:<epoch>[:rank<k>], e.g. oom@fwd:3 or exit@step:7:rank1"}),
    (("--watchdog_seconds",), float, 0.0, {"help": "heartbeat watchdog: abort all ranks cleanly when a peer leaves or stays "
                                                   "silent for this many seconds (0 = off, NCCL's timeout only)"}),
    (("--watchdog_step_seconds",), float, 0.0, {"help": "with --watchdog_seconds: also abort when this rank itself has "
                                                        "not reached a step boundary for this long (a collective or "
                                                        "kernel over its deadline; 0 = off)"}),
    (("--locality_reorder_parts",), int, 0, {"help": "relabel nodes at load time into this many locality clusters "
                                                     "(multilevel partition; 0 = keep the dataset's order)"}),
    (("--edge_build_threads",), int, 0, {"help": "OpenMP threads of a host-side edge build (0 = usable cores / ranks "
                                                 "on this node)"}),
    (("--shard_cpu_edge_build",), _STORE_TRUE, False, {"help": "cpu_rank_local_prefetch policy: each rank builds the rows "
                                                             "of its own queries and the shards are all-gathered"}),
    (("--replicate_gpu_edge_build",), _STORE_TRUE, False, {"help": "GPU edge policies on several ranks: every rank builds the "
                                                                 "whole attention graph itself instead of building the rows of "
                                                                 "its own queries and fetching the other shards over NVLink"}),
    (("--nvtx",), _STORE_TRUE, False, {"help": "emit NVTX ranges for step phases and profiled calls"}),
    (("--debug_checks",), _STORE_TRUE, False, {"help": "validate every attention graph, poison reusable symmetric "
                                               "buffers after use and check losses/gradients for NaN (also BF_DEBUG=1)"}),
    (("--cuda_graph",), _STORE_TRUE, False, {"help": "capture the optimizer step in a CUDA graph"}),
]


def _add(parser: argparse.ArgumentParser, table, defaults: Optional[Dict] = None) -> None:
    defaults = defaults or {}
    for flags, typ, default, extra in table:
        dest = flags[0].lstrip("-").replace("-", "_")
        dflt = defaults.get(dest, default)
        if typ is _STORE_TRUE:
            parser.add_argument(*flags, action="store_true", default=dflt, **extra)
        else:
            parser.add_argument(*flags, type=typ, default=dflt, **extra)


def add_node_common_args(parser, defaults=None):
    _add(parser, _COMMON, defaults)


def add_node_batch_sp_args(parser, defaults=None):
    _add(parser, _BATCH_SP, defaults)


def add_node_fullgraph_sp_args(parser, defaults=None):
    _add(parser, _FULLGRAPH, defaults)
    _add(parser, _EXTRA, defaults)


FULLGRAPH_DEFAULTS = {"peak_lr": 1e-3, "warmup_updates": 5, "sequence_parallel_size": 1, "num_global_node": 1}


def build_fullgraph_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Full-graph sequence-parallel Graph Transformer training (B200)")
    add_node_common_args(p, FULLGRAPH_DEFAULTS)
    add_node_fullgraph_sp_args(p, FULLGRAPH_DEFAULTS)
    return p


def build_batch_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Mini-batch sequence-parallel training (legacy mode)")
    add_node_common_args(p, {})
    add_node_batch_sp_args(p, {})
    _add(p, [t for t in _FULLGRAPH if t[0][0] in ("--activation_checkpoint_mode", "--amp_dtype",
                                                  "--force_random_split", "--to_bidirected")], {})
    _add(p, [t for t in _EXTRA if t[0][0] in ("--device",)], {})
    return p


def _normalize_checkpoint_args(args) -> None:
    mode = getattr(args, "activation_checkpoint_mode", None)
    if mode is None:
        return
    mode = str(mode).lower()
    if mode not in {"all", "ffn_only", "adaptive", "multi_tier"}:
        raise ValueError(f"Unsupported activation_checkpoint_mode: {mode}")
    args.activation_checkpoint_mode = mode


def _normalize_fixed_edge_budget_args(args) -> None:
    real = getattr(args, "fixed_real_edges_per_query", None)
    rw = getattr(args, "fixed_rw_edges_per_query", None)
    walk = getattr(args, "fixed_walk_length", None)
    if real is None and rw is None:
        if walk is not None:
            raise ValueError("--fixed_walk_length requires --fixed_real_edges_per_query and --fixed_rw_edges_per_query.")
        return
    if real is None or rw is None:
        raise ValueError("--fixed_real_edges_per_query and --fixed_rw_edges_per_query must be set together.")
    if int(real) < 0 or int(rw) < 0:
        raise ValueError("Fixed edge budgets must be >= 0.")
    args.fixed_real_edges_per_query, args.fixed_rw_edges_per_query = int(real), int(rw)
    if args.fixed_rw_edges_per_query > 0 and int(getattr(args, "walks_per_node", 0)) <= 0:
        raise ValueError("--fixed_rw_edges_per_query > 0 requires --walks_per_node > 0.")
    if walk is not None:
        if int(walk) <= 0:
            raise ValueError("--fixed_walk_length must be > 0 when provided.")
        args.fixed_walk_length = int(walk)


def normalize_main_node_sp_args(args):
    _normalize_checkpoint_args(args)
    if str(getattr(args, "model", "")).lower() == "gt":
        args.attn_type = "sparse"
    return args


def normalize_main_node_fullgraph_sp_args(args):
    _normalize_checkpoint_args(args)
    _normalize_fixed_edge_budget_args(args)
    args.multi_tier_gpu_memory_limit_mib = max(0, int(getattr(args, "multi_tier_gpu_memory_limit_mib", 0) or 0))
    ratio = float(getattr(args, "node_sample_ratio", 1.0))
    if not (0.0 < ratio <= 1.0):
        raise ValueError("--node_sample_ratio must be in (0, 1].")
    args.node_sample_ratio = ratio
    model = str(getattr(args, "model", "")).lower()
    if model in ("gt", "exphormer"):
        args.attn_type = "sparse"
    if model == "graphgps" and not getattr(args, "attn_type", None):
        args.attn_type = "sparse"
    if args.model != "graphormer":
        args.num_global_node = 0
    elif args.num_global_node not in (0, 1):
        raise ValueError("main_node_fullgraph_sp.py supports at most one Graphormer-style virtual node.")
    if args.model in ("graphormer", "gt") and int(getattr(args, "hops", 0)) < 0:
        raise ValueError("--hops must be >= 0 for Graphormer/GT (0 = disabled).")
    if args.model == "nagphormer" and int(getattr(args, "hops", 0)) < 1:
        raise ValueError("--hops must be >= 1 for NAGphormer.")
    if str(getattr(args, "dataset", "")).lower() == "ogbn-arxiv":
        args.to_bidirected = True
    if getattr(args, "adaptive_edge_budget", False) and getattr(args, "fixed_real_edges_per_query", None) is not None:
        raise ValueError("--adaptive_edge_budget and --fixed_*_edges_per_query are mutually exclusive.")
    return args


def parse_fullgraph_args(argv: Optional[Iterable[str]] = None):
    args = build_fullgraph_parser().parse_args(list(argv) if argv is not None else None)
    return normalize_main_node_fullgraph_sp_args(args)
