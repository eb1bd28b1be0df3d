"""Reference arm of bench.py: runs the unmodified reference driver (``baseline/_ref``, installed by
``baseline/install_reference.sh``) on the benchmark graph and model configuration.

The reference is pure Python on top of torch-scatter / torch-sparse / torch-cluster / PyG / DGL, none of which
can be installed offline for this PyTorch build; ``baseline/shims`` provides thin pure-PyTorch stand-ins for the
few entry points the reference calls, so the arm is reported as "reference + shims".  Nothing of the product
(models, kernels, engine) is on this path.  Timing: the reference's own per-epoch timer (``t=`` in its log line:
host wall clock around the epoch, which includes a device sync through ``loss.item()``), taken over the K epochs
after W warm-up epochs, max over ranks by construction of that log line."""
from __future__ import annotations

import contextlib
import io
import json
import os
import re
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIMS = os.path.join(HERE, "shims")


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


class _Tee(io.TextIOBase):
    def __init__(self, lines):
        self.lines, self._buf = lines, ""

    def write(self, s):
        self._buf += s
        while "\n" in self._buf:
            line, self._buf = self._buf.split("\n", 1)
            self.lines.append(line)
        return len(s)


def _patch_torch_compat() -> None:
    """The reference targets torch 2.1: its schedulers pass ``verbose`` positionally to ``_LRScheduler.__init__``
    (utils/lr.py:12,34), an argument that current PyTorch removed.  Accept and drop it so that the unmodified
    sources run; nothing else is patched."""
    from torch.optim import lr_scheduler as _ls

    base = _ls.LRScheduler
    if getattr(base, "_bf_compat", False):
        return
    orig = base.__init__

    def init(self, optimizer, last_epoch=-1, *ignored, **kw):
        kw.pop("verbose", None)
        return orig(self, optimizer, last_epoch)

    base.__init__ = init
    base._bf_compat = True


def run(ns, config_record) -> None:
    """``config_record`` builds the JSON line's ``config`` object (bench.py's, so that both arms print the same keys)."""
    if not os.path.isdir(os.path.join(REF, "gt_sp")):
        return _unavailable("baseline/_ref is missing: run baseline/install_reference.sh")
    import torch
    if not torch.cuda.is_available():
        return _unavailable("no CUDA device: the reference asserts GPUs for multi-process runs and is benchmarked on GPUs")
    sys.path.insert(0, os.path.dirname(HERE))
    from budgetformer_b200.graph.synthetic import make_bench_graph, write_dataset   # graph generator only

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    root = f"/tmp/bf_bench_ds_{ns.config}_{ns.scale}"
    marker = os.path.join(root, ns.config, ".done")
    if rank == 0 and not os.path.exists(marker):
        x, y, ei, cfg = make_bench_graph(ns.config, seed=42, scale=ns.scale)
        if y.dim() == 2:                       # the reference has no multi-label loss: collapse to the first positive
            y = y.argmax(1)
        write_dataset(root, ns.config, x, y, ei)
        open(marker, "w").close()
    t0 = time.time()
    while not os.path.exists(marker):
        if time.time() - t0 > 1800:
            return _unavailable("timed out waiting for rank 0 to write the synthetic dataset")
        time.sleep(1.0)
    from budgetformer_b200.graph.synthetic import BENCH_CONFIGS
    cfg = BENCH_CONFIGS[ns.config]
    n_nodes = torch.load(os.path.join(root, ns.config, "y.pt")).numel()
    n_edges = torch.load(os.path.join(root, ns.config, "edge_index.pt"), mmap=True).size(1)
    b = int(cfg["budget"])
    warm, steps = max(3, ns.warmup), ns.steps
    argv = ["--dataset_dir", root + "/", "--dataset", ns.config, "--model", cfg["model"], "--n_layers", str(cfg["n_layers"]),
            "--hidden_dim", str(cfg["hidden_dim"]), "--num_heads", str(cfg["num_heads"]), "--ffn_dim", str(2 * cfg["hidden_dim"]),
            "--amp_dtype", "bf16", "--walk_length", str(cfg["walk_length"]), "--walks_per_node", str(cfg["walks_per_node"]),
            "--fixed_real_edges_per_query", str((b + 1) // 2), "--fixed_rw_edges_per_query", str(b // 2),
            "--epochs", str(warm + steps), "--eval_every", "1000000", "--force_random_split"]
    if ns.ckpt:
        argv += ["--activation_checkpoint_mode", ns.ckpt]
    # the reference and its stand-in dependencies come first on the path; the product package is not imported below
    sys.path.insert(0, SHIMS)
    sys.path.insert(0, REF)
    for m in [k for k in sys.modules if k.split(".")[0] in ("utils", "models", "gt_sp")]:
        del sys.modules[m]
    _patch_torch_compat()
    lines = []
    old_argv = sys.argv
    sys.argv = ["main_node_fullgraph_sp.py"] + argv
    try:
        import main_node_fullgraph_sp as ref_main
        with contextlib.redirect_stdout(_Tee(lines)):
            ref_main.main()
    except SystemExit:
        pass
    except Exception as e:  # the reference failed on this box: report, do not crash the harness
        tail = " | ".join(lines[-3:])
        return _unavailable(f"reference run failed: {type(e).__name__}: {str(e)[:200]} ; last log: {tail[:200]}")
    finally:
        sys.argv = old_argv
    if rank != 0:
        return
    times, phases = {}, {}
    for ln in lines:
        m = re.search(r"Epoch\s+(\d+)\s*\|.*?\bt=([0-9.]+)s", ln)
        if m:
            times[int(m.group(1))] = float(m.group(2))
            # the same line carries the reference's own split of the epoch: rw= (graph construction, the phase the
            # stand-ins for torch_cluster / torch_sparse / PyG serve), fwd=, bwd= (torch_scatter stand-in), opt=
            phases[int(m.group(1))] = {k: float(v) for k, v in re.findall(r"\b(rw|fwd|bwd|opt|adj|prefetch_wait)=([0-9.]+)", ln)}
    timed_epochs = [e for e in sorted(times) if e > warm][:steps]
    timed = [times[e] for e in timed_epochs]
    if len(timed) < steps:
        return _unavailable(f"reference printed {len(timed)} timed epochs, expected {steps}; last log: {' | '.join(lines[-2:])[:300]}")
    ms = 1e3 * sum(timed) / len(timed)
    split = {}
    for key in ("rw", "fwd", "bwd", "opt", "adj", "prefetch_wait"):
        vals = [phases[e][key] for e in timed_epochs if key in phases.get(e, {})]
        if vals:
            split[key + "_ms"] = 1e3 * sum(vals) / len(vals)
    peak = torch.cuda.max_memory_allocated() / 2 ** 20
    feat_dim = torch.load(os.path.join(root, ns.config, "x.pt"), mmap=True).size(1)
    rec = {"metric": "fullgraph_train_nodes_per_s", "value": n_nodes / (ms / 1e3), "unit": "nodes/s", "n_gpus": world,
           "steps": steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "bf16", "data": f"synthetic {cfg['graph']} graph, N(0,1) features, random-init weights",
           "impl": "reference", "impl_note": "unmodified reference sources + pure-PyTorch stand-ins for torch_scatter/"
           "torch_sparse/torch_cluster/PyG/DGL; timed by the reference's own epoch timer (host clock incl. device sync)",
           "config": config_record(ns.config, cfg, n_nodes, n_edges, feat_dim, world, ns.ckpt, ns.scale),
           "phase_split": split,
           "phase_note": "the reference's own synchronised timers per epoch: rw = attention-graph construction (served by the "
                         "stand-ins for torch_cluster / torch_sparse / PyG), bwd includes the torch_scatter stand-in",
           "epoch_ms": ms, "peak_hbm_mib_per_gpu": peak, "gpu_launches": 0,
           "e2e": {"value": n_nodes / (ms / 1e3), "unit": "nodes/s", "note": "the reference keeps its inputs resident; "
                   "its epoch timer already includes the loss read-back"}}
    print(json.dumps(rec), flush=True)
