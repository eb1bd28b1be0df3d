"""Rank-0 console output in the reference's line formats (utils/fullgraph_sp_runtime.py:44-137,
890-1079): header block, communication-profile table, final summary with average epoch time
(first epoch excluded), data-preparation time, inference throughput and per-rank peak memory."""
from __future__ import annotations

import subprocess
from typing import Dict

import torch
import torch.distributed as dist

from ..utils.misc import process_peak_rss_mib


def print_git_version(log) -> None:
    try:
        rev = subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5)
        if rev.returncode == 0:
            log(f"[git] {rev.stdout.strip()}")
    except Exception:
        pass


def print_training_header(t) -> None:
    a = t.args
    st = t.budget_state()
    t.log("=" * 88)
    t.log(f"Full-graph SP training | model={a.model} dataset={a.dataset} nodes={t.data.num_nodes:,} "
          f"(padded {t.num_nodes:,}) edges={t.data.edge_index.size(1):,}")
    t.log(f"  layers={a.n_layers} hidden={a.hidden_dim} heads={a.num_heads} ffn={a.ffn_dim} classes={t.data.output_dim} "
          f"amp={a.amp_dtype} ckpt={a.activation_checkpoint_mode}")
    backend = dist.get_backend() if dist.is_initialized() else "none (single process)"
    t.log(f"  sp_world={t.sp_world} nodes/rank={t.nodes_per_rank:,} device={t.device} backend={backend} "
          f"fused_sp={'on' if t.fused_sp else 'off'}")
    t.log(f"  edges: policy={t.edge_engine.policy} real={st.b_real if st.use_real else 0} "
          f"rw={st.b_rw if st.use_rw else 0} walk_length={st.walk_length} walks_per_node={a.walks_per_node} "
          f"adaptive={bool(t.budget_cfg.enabled)} prefetch={t.edge_engine.uses_prefetch()}")
    if t.budget_cfg.enabled and not t.controller.frozen:
        t.log("  budget search active: synchronous CPU-side baseline policy and all-recompute tiers until it freezes")
    t.log("=" * 88)


def format_comm_profile(summary: Dict, step_s: float) -> str:
    lines = ["  comm profile:"]
    for name, s in summary.items():
        if name == "scalars":
            continue
        share = 100.0 * s["total_s"] / step_s if step_s > 0 else 0.0
        lines.append(f"    {name:<22} total={s['total_s'] * 1e3:9.3f} ms avg={s['avg_s'] * 1e3:8.3f} ms "
                     f"count={s['count']:<4d} share={share:5.1f}% payload={s['bytes'] / 2 ** 20:9.2f} MiB")
    sc = summary.get("scalars", {})
    if sc:
        lines.append("    edge cardinality: " + " ".join(f"{k}={int(v):,}" for k, v in sorted(sc.items())))
    return "\n".join(lines)


def aggregate_comm_profile(summary: Dict, group=None) -> Dict:
    """Keep the profile of the rank with the largest total (utils/fullgraph_sp_runtime.py:91-137)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return summary
    objs = [None] * dist.get_world_size(group)
    dist.all_gather_object(objs, summary, group=group)
    tot = lambda s: sum(v["total_s"] for k, v in s.items() if k != "scalars")
    return max(objs, key=tot)


def print_training_summary(t) -> None:
    times = t.epoch_times[1:] if len(t.epoch_times) > 1 else t.epoch_times
    prep = t.prep_times[1:] if len(t.prep_times) > 1 else t.prep_times
    if t.rank == 0:
        b = t.best
        t.log(f"Best by validation: epoch={b['epoch']} train={b['train']:.4f} valid={b['valid']:.4f} test={b['test']:.4f}")
        if times:
            avg = sum(times) / len(times)
            t.log(f"Avg epoch wall time (excluding epoch 1): {avg:.4f}s | throughput={t.data.num_nodes / avg:,.0f} nodes/s")
        if prep:
            t.log(f"Avg data prep time: {sum(prep) / len(prep):.4f}s")
        if t.eval_times:
            avg = sum(t.eval_times) / len(t.eval_times)
            t.log(f"Avg inference time per eval: {avg:.4f}s throughput={t.data.num_nodes / avg:,.0f} nodes/s")
    peak = torch.cuda.max_memory_allocated(t.device) / 2 ** 20 if t.device.type == "cuda" else 0.0
    vals = [peak, process_peak_rss_mib()]
    if dist.is_initialized() and t.sp_world > 1:
        objs = [None] * t.sp_world
        dist.all_gather_object(objs, vals, group=t.sp_group)
    else:
        objs = [vals]
    if t.rank == 0:
        t.log("Peak GPU memory per rank (MiB): " + " ".join(f"r{i}={v[0]:.0f}" for i, v in enumerate(objs)))
        t.log("Peak CPU RSS per rank (MiB): " + " ".join(f"r{i}={v[1]:.0f}" for i, v in enumerate(objs)))
