"""Headline benchmark: full-graph training epoch time / nodes per second.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Configuration: GT, 4 layers, hidden 128, 8 heads, bf16, sequence parallel over N GPUs, on a synthetic
citation-like DAG with 2,923,922 nodes / ~13.98 M edges, 269-d N(0,1) features, 5 classes, per-query
budget B = 8 (4 real + 4 random-walk, walk length 4, 2 walks per node), random-init weights.  One step
is one epoch: attention-graph construction + forward + backward + gradient reduction + clip + AdamW.
Total work is fixed as N grows (strong scaling).  Rank 0 prints one JSON line.

``--impl reference`` runs the unmodified reference (installed under ``baseline/_ref``) on the same graph
and model configuration through its own command-line driver.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
MODEL_NAMES = {"gt": "GT", "graphormer": "Graphormer", "graphgps": "GraphGPS", "exphormer": "Exphormer"}
GRAPH_DESC = {"dag": "citation-like DAG (power-law out-degree)", "chung_lu_directed": "Chung-Lu power-law directed graph",
              "chung_lu_undirected": "Chung-Lu power-law undirected graph", "sbm": "stochastic block model"}
sys.path.insert(0, REPO)

# Epoch time of the reference arm (unmodified reference + pure-PyTorch stand-ins for its native wheels, its own NCCL
# and cuBLAS path), measured on this pool's B200s with this file's `--impl reference`: ms per epoch by number of GPUs
# (patents_like: 20 timed epochs per GPU count; arxiv_like: 3 timed epochs on one GPU).  The reference publishes no
# numbers of its own, so `vs_baseline` is this arm's epoch time over ours at the same GPU count.
REFERENCE_EPOCH_MS = {"patents_like": {1: 5089.0, 2: 3388.5, 4: 1707.0, 8: 1455.5}, "arxiv_like": {1: 3156.7}}


def config_record(name, cfg, n_nodes, n_edges, feat_dim, world, ckpt, scale):
    """The `config` object of the JSON line; both arms emit exactly these keys."""
    b = int(cfg["budget"])
    return {"name": name,
            "model": f"{MODEL_NAMES.get(cfg['model'], cfg['model'])} L{cfg['n_layers']} h{cfg['hidden_dim']} H{cfg['num_heads']}",
            "nodes": int(n_nodes), "edges": int(n_edges), "global_batch": int(n_nodes), "seq_len": int(n_nodes),
            "feat_dim": int(feat_dim),
            "budget": f"{(b + 1) // 2} real + {b // 2} random-walk per query (B={b} ceiling of the adaptive search), "
                      f"rebuilt every epoch",
            "parallelism": f"sp{world}", "activation_checkpoint": ckpt or "none (retain)", "scale": scale,
            "l2": "working set per step (>= 750 MB activations per layer) exceeds the 126 MB L2; no flush needed"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="patents_like")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the graph (tests only; <1 is not the named config)")
    ap.add_argument("--fused_sp", default="auto")
    ap.add_argument("--ckpt", default="", help="activation checkpoint mode (default none = retain everything)")
    ap.add_argument("--no_e2e", action="store_true")
    ap.add_argument("--fit_epochs", type=int, default=0,
                    help="instead of the timed steps: run FullGraphTrainer.fit for this many epochs on the named configuration "
                         "(adaptive budget search, planner and evaluation included), log on stderr, one JSON summary line")
    ap.add_argument("--fit_flags", default="",
                    help="extra command-line flags of the training driver for --fit_epochs, e.g. "
                         "'--adaptive_edge_budget --max_total_edges_per_query 8 --activation_checkpoint_mode multi_tier'")
    ap.add_argument("--kernel_events", type=int, default=0,
                    help="after the timed loops run this many extra steps with CUDA events around every call into the "
                         "extension and print rank 0's per-kernel device times (a breakdown, not a benchmark value)")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of this process's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        super().__init__(daemon=True)
        self.gpu = gpu_index
        self.samples = []
        self._stop = threading.Event()
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                if self._stop.is_set():
                    break
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 7:
                    self.samples.append((time.time(), parts))
        except Exception:
            pass

    def stop(self):
        self._stop.set()
        if self.proc is not None:
            try:
                self.proc.terminate()
            except Exception:
                pass

    def summary(self, t0=None, t1=None):
        """Median SM clock and the throttle reasons seen between host times ``t0`` and ``t1`` (the timed region); when
        no sample fell inside (a very short region) the samples closest after ``t0`` are used."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [p for (t, p) in self.samples if (t0 is None or t >= t0) and (t1 is None or t <= t1 + 0.25)]
        if not rows and self.samples:
            rows = [p for (t, p) in self.samples if t0 is None or t >= t0 - 0.5][:3] or [self.samples[-1][1]]
        for p in rows:
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for n, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def bench_args(cfg: dict, ns, extra=()):
    from budgetformer_b200.config import parse_fullgraph_args

    b = int(cfg["budget"])
    argv = ["--model", cfg["model"], "--dataset", ns.config, "--n_layers", str(cfg["n_layers"]),
            "--hidden_dim", str(cfg["hidden_dim"]), "--num_heads", str(cfg["num_heads"]), "--ffn_dim", str(2 * cfg["hidden_dim"]),
            "--amp_dtype", "bf16", "--walk_length", str(cfg["walk_length"]), "--walks_per_node", str(cfg["walks_per_node"]),
            "--force_random_split", "--fused_sp", ns.fused_sp]
    if "--adaptive_edge_budget" in extra:
        argv += ["--max_total_edges_per_query", str(b)]
    else:
        argv += ["--fixed_real_edges_per_query", str((b + 1) // 2), "--fixed_rw_edges_per_query", str(b // 2)]
    argv += ["--epochs", str(ns.fit_epochs) if ns.fit_epochs > 0 else "100000"]
    if cfg.get("multilabel"):
        argv.append("--multilabel")
    if ns.ckpt:
        argv += ["--activation_checkpoint_mode", ns.ckpt]
    return parse_fullgraph_args(argv + list(extra))


def _plan_record(planner):
    if planner is None or not hasattr(planner, "modes"):
        return None
    return {"state": planner.state_name(), "active": bool(planner.is_active()), "tiers": list(planner.modes()),
            "edge_policy": planner.edge_policy if planner.is_active() else None}


def run_fit(ns):
    """The training loop a user runs (``FullGraphTrainer.fit``: budget search with its probe steps, execution planner,
    evaluation) on a named configuration; the trainer's own log goes to stderr."""
    import shlex

    import torch

    from budgetformer_b200.graph.synthetic import make_bench_graph
    from budgetformer_b200.train.data import GraphData, random_split_idx
    from budgetformer_b200.train.engine import FullGraphTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
    x, y, ei, cfg = make_bench_graph(ns.config, seed=42, scale=ns.scale)
    n = x.size(0)
    data = GraphData(x, y, ei, random_split_idx(n, 42), n, int(cfg["classes"]), bool(cfg.get("multilabel")))
    extra = shlex.split(ns.fit_flags)
    log = (lambda *a, **k: print(*a, file=sys.stderr, flush=True)) if rank == 0 else (lambda *a, **k: None)
    trainer = FullGraphTrainer(bench_args(cfg, ns, extra), data=data, log=log)
    t0 = time.time()
    best = trainer.fit()
    if trainer.device.type == "cuda":
        torch.cuda.synchronize(trainer.device)
    wall = time.time() - t0
    if rank == 0:
        c = trainer.controller
        times = list(trainer.epoch_times)
        tail = times[len(times) // 2:] or times
        rec = {"mode": "fit", "impl": "ours", "n_gpus": world, "epochs": ns.fit_epochs, "wall_s": wall,
               "epoch_ms_median_second_half": 1e3 * sorted(tail)[len(tail) // 2] if tail else None,
               "epoch_ms_first": [round(1e3 * t, 1) for t in times[:12]],
               "budget": {"real": c.real_budget, "rw": c.rw_budget, "frozen": bool(c.frozen)},
               "plan": _plan_record(getattr(trainer, "planner", None)),
               "edge_policy": getattr(trainer.edge_engine, "policy", None),
               "peak_hbm_mib": (torch.cuda.max_memory_allocated(trainer.device) / 2 ** 20 if trainer.device.type == "cuda" else 0.0),
               "best": best, "fit_flags": ns.fit_flags,
               "config": config_record(ns.config, cfg, n, int(ei.size(1)), int(x.size(1)), world, ns.ckpt, ns.scale)}
        print(json.dumps(rec, default=str), flush=True)
    if world > 1:
        from budgetformer_b200.parallel.initialize import destroy_distributed
        destroy_distributed()


def run_ours(ns):
    import torch
    import torch.distributed as dist

    from budgetformer_b200.graph.synthetic import make_bench_graph
    from budgetformer_b200.ops import _ext
    from budgetformer_b200.train.data import GraphData, random_split_idx
    from budgetformer_b200.train.engine import FullGraphTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != ns.gpus:
        raise SystemExit(f"--gpus {ns.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N>1")
    # The clock sampler (an nvidia-smi child) starts first: its start-up was measured to stall the GPU for about 0.1 s,
    # so it must be over long before the timed region; samples are filtered by time afterwards, and the GPU never
    # idles between warm-up and measurement.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank % torch.cuda.device_count())     # large graphs are generated on this rank's GPU
    x, y, ei, cfg = make_bench_graph(ns.config, seed=42, scale=ns.scale)
    n = x.size(0)
    data = GraphData(x, y, ei, random_split_idx(n, 42), n, int(cfg["classes"]), bool(cfg.get("multilabel")))
    args = bench_args(cfg, ns)
    trainer = FullGraphTrainer(args, data=data, log=lambda *a, **k: None)
    dev = trainer.device
    assert dev.type == "cuda", "bench.py measures on GPUs"
    _ext.load()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    epoch = 0
    for _ in range(max(3, ns.warmup)):
        epoch += 1
        trainer.train_step(epoch, read_loss=False)
    sync()
    torch.cuda.reset_peak_memory_stats(dev)
    _ext.reset_launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    t_begin = time.time()
    start.record()
    for _ in range(ns.steps):
        epoch += 1
        trainer.train_step(epoch, read_loss=False)
    end.record()
    sync()
    t_end = time.time()
    launches = _ext.launch_count()
    ms = start.elapsed_time(end)
    # end-to-end: input features copied host->device from pinned memory and the loss read back, every step
    e2e_ms = None
    if not ns.no_e2e:
        for _ in range(2):                             # untimed: allocates the double buffer and primes the upload pipeline
            epoch += 1
            trainer.train_step(epoch, x_host=trainer.x_host, read_loss="async")
        sync()
        start.record()
        for _ in range(ns.steps):
            epoch += 1
            out = trainer.train_step(epoch, x_host=trainer.x_host, read_loss="async")
        last_loss = trainer.flush_loss()               # the final step's loss read is inside the timed region too
        end.record()
        sync()
        assert last_loss == last_loss, "end-to-end loop produced a NaN loss"
        e2e_ms = start.elapsed_time(end)
    if rank == 0:
        sampler.stop()
    if ns.kernel_events > 0:
        _kernel_breakdown(ns, trainer, epoch, sync, rank, world)
        epoch += ns.kernel_events
    peak = torch.cuda.max_memory_allocated(dev) / 2 ** 20
    vals = torch.tensor([ms, e2e_ms or 0.0, peak], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, e2e_ms_max, peak = (float(v) for v in vals.tolist())
    if rank == 0:
        ms_step = ms / ns.steps
        rec = {
            "metric": "fullgraph_train_nodes_per_s", "value": n / (ms_step / 1e3), "unit": "nodes/s",
            "n_gpus": world, "steps": ns.steps, "warmup": max(3, ns.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": f"synthetic {GRAPH_DESC.get(cfg['graph'], cfg['graph'])}, N(0,1) features, random-init weights",
            "impl": "ours", "fused_sp": bool(trainer.fused_sp),
            "config": config_record(ns.config, cfg, n, int(ei.size(1)), int(x.size(1)), world, ns.ckpt, ns.scale),
            "epoch_ms": ms_step, "peak_hbm_mib_per_gpu": peak, "gpu_launches": launches,
            "clocks": sampler.summary(t_begin, t_end),
        }
        ref_ms = REFERENCE_EPOCH_MS.get(ns.config, {}).get(world) if ns.scale == 1.0 else None
        if ref_ms:
            rec["vs_baseline"] = ref_ms / ms_step
            rec["baseline_source"] = (f"reference arm of this file (unmodified reference + stand-ins for its native wheels) "
                                      f"at {world} GPU(s): {ref_ms} ms per epoch; the reference publishes no numbers")
        if e2e_ms is not None:
            e_step = e2e_ms_max / ns.steps
            rec["e2e"] = {"value": n / (e_step / 1e3), "unit": "nodes/s", "ms_per_step": e_step,
                          # whole job: every rank uploads its slice of the features and reads its loss back
                          "h2d_bytes_per_step": int(trainer.x_host.numel() * trainer.x_host.element_size()) * world,
                          "d2h_bytes_per_step": 4 * world}
        print(json.dumps(rec), flush=True)
    trainer.edge_engine.shutdown()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _kernel_breakdown(ns, trainer, epoch, sync, rank, world):
    """Per-entry-point device time of ``ns.kernel_events`` steps on rank 0 (CUDA-event pairs around every call into
    the extension; the device barriers' time is the wait for the slowest rank).  Written to stderr."""
    import torch

    from budgetformer_b200.ops import _ext
    _ext.enable_kernel_events(True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    t0 = time.perf_counter()
    start.record()
    host_s = 0.0
    for _ in range(ns.kernel_events):
        epoch += 1
        h0 = time.perf_counter()
        trainer.train_step(epoch, read_loss=False)
        host_s += time.perf_counter() - h0
    end.record()
    sync()
    wall_ms = (time.perf_counter() - t0) * 1e3
    table = _ext.kernel_event_summary()
    _ext.enable_kernel_events(False)
    if rank != 0:
        return
    k = ns.kernel_events
    step_ms = start.elapsed_time(end) / k
    rows = sorted(table.items(), key=lambda kv: -kv[1][1])
    total = sum(ms for _c, ms in table.values()) / k
    print(f"[kernel_events] world={world} step={step_ms:.3f} ms (events on), host time in train_step={host_s / k * 1e3:.3f} ms, "
          f"wall={wall_ms / k:.3f} ms, sum of bracketed calls={total:.3f} ms (side-stream graph build included)",
          file=sys.stderr)
    print("[kernel_events] | share of step | ms/step | calls/step | entry point |", file=sys.stderr)
    for name, (calls, ms) in rows:
        print(f"[kernel_events] | {ms / k / step_ms:6.1%} | {ms / k:8.3f} | {calls / k:6.1f} | {name} |", file=sys.stderr)
    sys.stderr.flush()


def run_reference(ns):
    try:
        from baseline.run_reference import run
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"baseline harness not importable: {type(e).__name__}: {e}"}))
        return
    run(ns, config_record)


if __name__ == "__main__":
    ns = parse()
    if ns.impl == "reference":
        run_reference(ns)
    else:
        from budgetformer_b200.utils.rank_main import run_rank_main
        run_rank_main(run_fit if ns.fit_epochs > 0 else run_ours, ns)
