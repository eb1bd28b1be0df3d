"""Full-graph sequence-parallel trainer: the public training API.

``FullGraphTrainer(args)`` performs what the reference's ``main()`` does between argument parsing
and the epoch loop (main_node_fullgraph_sp.py:212-456): distributed bootstrap, data load / pad /
slice, edge engine, budget controller, model construction and parameter sync, gradient reducer,
optimizer bundle.  ``train_step(epoch)`` is one epoch (= one optimizer step, :646-1310);
``evaluate`` restates ``_eval_sp`` (utils/fullgraph_sp_support.py:3379-3477);
``maybe_update_edge_budget`` restates the probe loop (:2475-2928); ``fit`` is the epoch loop with
logging, checkpointing and the planner hooks.
"""
from __future__ import annotations

import gc
import json
import os
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..control.budget import (BudgetSearch, decide_budget_move, fixed_budget_controller,
                              resolve_adaptive_edge_budget_config)
from ..control.multi_tier import parse_force_multi_tier_plan, TIER_FROM_ID, TIER_IDS, EDGE_POLICY_ORDER
from ..graph.attn_graph import AttnGraph
from ..graph.engine import BudgetState, EdgeEngine, edge_seed_for_epoch, resolve_budget_state
from ..models import MODEL_REGISTRY
from ..parallel import comm
from ..parallel.initialize import (get_sequence_parallel_group, get_sequence_parallel_rank,
                                   get_sequence_parallel_src_rank, get_sequence_parallel_world_size,
                                   initialize_distributed, set_global_token_indices)
from ..parallel.reducer import build_gradient_reducer, sync_params_and_buffers
from ..utils import comm_profiler, debug
from ..utils.fault import FaultInjector
from ..utils.lr import build_lr_scheduler
from ..utils.misc import (StepTimer, autocast_context, process_peak_rss_mib, process_rss_mib, resolve_amp_dtype,
                          set_seed)
from .data import (GraphData, generate_expander_edges, load_data, pad_to_sequence_parallel_world,
                   preprocess_hop_features)

MAX_STEP_RETRIES = 3
MAX_CONSECUTIVE_DROPPED = 5


class StepDropped(RuntimeError):
    """The step was abandoned symmetrically on all ranks (OOM after backward had started)."""


def build_model(args, input_dim: int, output_dim: int) -> torch.nn.Module:
    """Model factory (utils/fullgraph_sp_support.py:718-806)."""
    name = str(args.model).lower()
    if name == "nagphormer":
        hops = int(args.hops)
        return MODEL_REGISTRY[name](hops=hops, n_class=output_dim, input_dim=input_dim // (hops + 1),
                                    n_layers=args.n_layers, num_heads=args.num_heads, hidden_dim=args.hidden_dim,
                                    ffn_dim=args.ffn_dim, dropout_rate=args.dropout_rate,
                                    attention_dropout_rate=args.attention_dropout_rate)
    kwargs = dict(n_layers=args.n_layers, num_heads=args.num_heads, input_dim=input_dim, hidden_dim=args.hidden_dim,
                  output_dim=output_dim, attn_bias_dim=args.attn_bias_dim, dropout_rate=args.dropout_rate,
                  input_dropout_rate=args.input_dropout_rate, attention_dropout_rate=args.attention_dropout_rate,
                  ffn_dim=args.ffn_dim, num_global_node=args.num_global_node)
    if name == "graphgps":
        kwargs["attn_type"] = getattr(args, "attn_type", "sparse") or "sparse"
    return MODEL_REGISTRY[name](**kwargs)


class FullGraphTrainer:
    def __init__(self, args, data: Optional[GraphData] = None, log=print):
        self.args = args
        self._log_fn = log
        self._guard_rank_departure(args)
        initialize_distributed(args)
        self.rank = int(args.rank)
        self.device = torch.device(args.device)
        self.sp_group = get_sequence_parallel_group()
        self.sp_world = get_sequence_parallel_world_size()
        self.sp_rank = get_sequence_parallel_rank()
        self.sp_src = get_sequence_parallel_src_rank()
        if args.num_heads % self.sp_world != 0:
            raise ValueError(f"num_heads={args.num_heads} must be divisible by the SP world size {self.sp_world}")
        self.amp_dtype = resolve_amp_dtype(getattr(args, "amp_dtype", "none"), self.device)
        set_seed(int(args.seed))
        comm_profiler.enable_comm_profiler(bool(getattr(args, "profile_sp_comm", False)))
        comm_profiler.enable_nvtx(bool(getattr(args, "nvtx", False)))
        if bool(getattr(args, "debug_checks", False)):
            debug.enable(True)
        self.fault = FaultInjector(getattr(args, "fault_inject", "") or "", self.rank)
        from ..utils.watchdog import build_watchdog
        self.watchdog = build_watchdog(args, self.rank, self.sp_world)
        if self.watchdog is not None:
            self.fault.on_exit = self._depart

        # ---- data -------------------------------------------------------------------------------
        if data is None:
            data = load_data(args, dist if dist.is_initialized() else None)
        data = pad_to_sequence_parallel_world(data, self.sp_world)
        data = preprocess_hop_features(args, data, self.rank)
        self.data = data
        self.multilabel = bool(data.multilabel)
        self.num_nodes = int(data.x.size(0))                      # padded
        self.nodes_per_rank = self.num_nodes // self.sp_world
        self.rank_start = self.sp_rank * self.nodes_per_rank
        self.rank_end = self.rank_start + self.nodes_per_rank
        split = data.split_idx
        self.local_idx = {k: self._localize(v) for k, v in split.items()}
        self.n_train_global = int(split["train"].numel())
        y_local = data.y[self.rank_start:self.rank_end]
        self.local_y = y_local.to(self.device)
        self.x_host = data.x[self.rank_start:self.rank_end].float().contiguous()
        if self.device.type == "cuda":
            if self.amp_dtype is not None:
                # under mixed precision the first layer consumes the features in the compute dtype anyway: keep the
                # host copy (and every upload) in that dtype instead of casting on the device every step
                self.x_host = self.x_host.to(self.amp_dtype)
                pad = (-self.x_host.size(1)) % 8
                if pad and args.model in ("gt", "graphormer", "graphgps", "exphormer"):
                    # 16-byte aligned feature rows (e.g. 269 -> 272 columns): the encoder pads its weight to match
                    self.x_host = torch.nn.functional.pad(self.x_host, (0, pad))
            self.x_host = self.x_host.pin_memory()
        self.x_local = self.x_host.to(self.device, non_blocking=True)
        if args.model == "graphormer" and args.num_global_node > 0:
            s = self.nodes_per_rank + 1
            set_global_token_indices([r * s for r in range(self.sp_world)])
        else:
            set_global_token_indices(None)

        # ---- edges / budget ---------------------------------------------------------------------
        expander = None
        if args.model == "exphormer" and int(getattr(args, "expander_degree", 0)) > 0:
            expander = generate_expander_edges(data.num_nodes, int(args.expander_degree), seed=int(args.seed))
        self.edge_engine = EdgeEngine(args, data.edge_index, self.num_nodes, self.device,
                                      nodes_per_rank=self.nodes_per_rank, sp_group=self.sp_group, sp_rank=self.sp_rank,
                                      sp_src_rank=self.sp_src, sp_world=self.sp_world, expander_edges=expander)
        self.budget_cfg = resolve_adaptive_edge_budget_config(args)
        if getattr(args, "fixed_real_edges_per_query", None) is not None:
            self.controller = fixed_budget_controller(args.fixed_real_edges_per_query, args.fixed_rw_edges_per_query,
                                                      getattr(args, "fixed_walk_length", None))
            self._controller_drives_budget = True
        elif self.budget_cfg.enabled:
            self.controller = BudgetSearch(self.budget_cfg)
            self._controller_drives_budget = True
        else:
            self.controller = BudgetSearch(self.budget_cfg)   # disabled => frozen
            self._controller_drives_budget = False
        self.probe_local_idx = self._select_probe_nodes()
        self._static_seed_epochs = self._resolve_static_seed_epochs()

        # ---- model / optimizer ------------------------------------------------------------------
        self.model = build_model(args, int(data.x.size(1)), int(data.output_dim)).to(self.device)
        ckpt_mode = getattr(args, "activation_checkpoint_mode", None)
        budget_moving = self.budget_cfg.enabled and not self.controller.frozen
        self.model.set_activation_checkpoint(ckpt_mode is not None, ckpt_mode, deferred=budget_moving)
        self.planner = self.model._comm_ckpt if ckpt_mode == "multi_tier" else None
        if self.planner is not None:
            self.planner.active_edge_policy_fn = lambda: self.edge_engine.policy
        self._configure_fused_sp()
        if self.planner is not None and self.sp_world > 1 and self.device.type == "cuda":
            from ..parallel import symm
            self.planner.probe.extra_bytes_fn = symm.symmetric_bytes   # peer-mapped buffers live outside the allocator
        sync_params_and_buffers(self.model, self.sp_group, self.sp_src)
        self.reducer = build_gradient_reducer(self.model, self.sp_group, 25.0, self.sp_world)
        self.scaler = torch.amp.GradScaler("cuda", enabled=(self.amp_dtype == torch.float16 and self.device.type == "cuda"))
        self.flat_optimizer = False
        if self.device.type == "cuda" and not self.scaler.is_enabled() and all(
                b.flat.dtype == torch.float32 for b in self.reducer.buckets):
            from ..ops.optim import FlatAdamW
            self.optimizer = FlatAdamW(self.reducer.buckets, lr=args.peak_lr, weight_decay=args.weight_decay, max_grad_norm=1.0,
                                       cuda_graph=bool(getattr(args, "cuda_graph", False)))
            self.flat_optimizer = True
        else:
            self.optimizer = torch.optim.AdamW(self.model.parameters(), lr=args.peak_lr, weight_decay=args.weight_decay)
        self.lr_scheduler = build_lr_scheduler(args, self.optimizer, self.n_train_global)
        self._apply_memory_limit()
        self._apply_forced_plan()

        # ---- bookkeeping ------------------------------------------------------------------------
        self.epoch = 0
        self.loss_ema: Optional[float] = None
        self.best = {"valid": -1.0, "test": -1.0, "train": -1.0, "epoch": 0}
        self.epoch_times: List[float] = []
        self.prep_times: List[float] = []
        self.eval_times: List[float] = []
        self.consecutive_dropped = 0
        self._budget_frozen_notified = not budget_moving
        self._metrics_fh = open(args.metrics_jsonl, "a") if (getattr(args, "metrics_jsonl", "") and self.rank == 0) else None
        self.kernel_launches = 0
        if getattr(args, "resume", ""):
            from .checkpoint import load_train_state
            load_train_state(self, args.resume)

    # ------------------------------------------------------------------------------------------ helpers
    @staticmethod
    def _guard_rank_departure(args) -> None:
        """A run in which a rank may leave or freeze on purpose (the heartbeat watchdog ends the process; ``exit`` /
        ``stall`` faults are injected) must not have its buffers bound to an NVSwitch multicast object: a rank that dies
        while bound raises NVLink faults on the other ranks' GPUs.  So, before the process group and the symmetric
        buffers exist, in-switch reduction is turned off for NCCL and for this package's own all-reduce (which then
        uses plain peer loads and stores)."""
        spec = str(getattr(args, "fault_inject", "") or os.environ.get("BF_FAULT", ""))
        wd = float(getattr(args, "watchdog_seconds", 0) or 0) > 0 or float(getattr(args, "watchdog_step_seconds", 0) or 0) > 0
        if wd or "exit@" in spec or "stall@" in spec:
            os.environ["NCCL_NVLS_ENABLE"] = "0"
            os.environ["BF_DISABLE_MULTIMEM"] = "1"
            os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"     # symmetric allocations are not bound to a multicast object
            if int(os.environ.get("RANK", "0")) == 0:
                print("[init] watchdog / departure faults requested: NVLS and multimem are off for this run", flush=True)

    def _depart(self) -> None:
        """Orderly departure of this rank between steps: let every kernel it has queued finish first (its peers' kernels
        of the same step wait for flags that only those kernels raise), then tell the others through the store."""
        self.edge_engine.shutdown()                  # the look-ahead worker has queued all of its build (or never will)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.watchdog.leave("injected exit")

    def log(self, msg: str) -> None:
        if self.rank == 0:
            self._log_fn(msg, flush=True)

    def _localize(self, idx: torch.Tensor) -> torch.Tensor:
        m = (idx >= self.rank_start) & (idx < self.rank_end)
        return (idx[m] - self.rank_start).to(self.device)

    def _select_probe_nodes(self) -> Optional[torch.Tensor]:
        """Validation nodes of this rank, optionally sub-sampled to ``--adaptive_edge_budget_probe_size`` globally
        (utils/fullgraph_sp_support.py:2245-2262)."""
        if not self.budget_cfg.enabled:
            return None
        valid = self.data.split_idx["valid"]
        k = int(self.budget_cfg.probe_size)
        if 0 < k < valid.numel():
            g = torch.Generator().manual_seed(int(self.args.seed) + 7)
            valid = valid[torch.randperm(valid.numel(), generator=g)[:k]]
        return self._localize(valid)

    def _resolve_static_seed_epochs(self) -> int:
        v = int(self.budget_cfg.static_seed_epochs)
        if v < 0:
            return 0
        if v == 0 and self.budget_cfg.enabled:
            return int(self.args.warmup_updates)
        return v

    def _configure_fused_sp(self) -> None:
        """Switch the models to the fused projection + all-to-all kernels when running on GPUs."""
        if bool(getattr(self.args, "sync_batchnorm", False)) and self.sp_world > 1:
            # every rank holds N/P rows of the same "batch": sum the BatchNorm statistics over the SP group
            for m in self.model.modules():
                if isinstance(m, torch.nn.BatchNorm1d):
                    m._bf_sync_group = self.sp_group
        mode = str(getattr(self.args, "fused_sp", "auto"))
        self.fused_sp = False
        if mode == "off" or self.device.type != "cuda":
            return
        try:
            from ..ops import fused_sp
            self.fused_sp = fused_sp.enable_for_model(self.model, self.args, self.sp_group, self.sp_world,
                                                      self.nodes_per_rank, self.amp_dtype)
        except ImportError:
            if mode == "on":
                raise

    def _apply_memory_limit(self) -> None:
        """``--multi_tier_gpu_memory_limit_mib``: cap the allocator and tell the planner
        (utils/fullgraph_sp_runtime.py:167-195)."""
        from ..graph.device_budget import BUDGET
        limit = int(getattr(self.args, "multi_tier_gpu_memory_limit_mib", 0) or 0)
        BUDGET.reset()                                  # process-wide state: a new trainer starts a new run
        if limit <= 0 or self.device.type != "cuda":
            return
        total = torch.cuda.get_device_properties(self.device).total_memory
        frac = min(1.0, limit * 2 ** 20 / total)
        torch.cuda.set_per_process_memory_fraction(frac, self.device)
        BUDGET.set_gpu_memory_cap(limit * 2 ** 20)      # the driver's free-memory figure does not know about the cap
        if self.planner is not None:
            self.planner.set_gpu_memory_limit_bytes(limit * 2 ** 20)
        self.log(f"[gpu-cap] per-process GPU memory limited to {limit} MiB ({frac:.1%} of device)")

    def _apply_forced_plan(self) -> None:
        spec = getattr(self.args, "force_multi_tier_plan", "") or ""
        if not spec or self.planner is None:
            return
        policy, tiers = parse_force_multi_tier_plan(spec, self.args.n_layers)
        self.planner.override_active_plan(policy, tiers)
        self.edge_engine.set_policy(policy, lock=True)

    # ------------------------------------------------------------------------------------------ budget state
    def budget_state(self, controller_state: Optional[dict] = None) -> BudgetState:
        if controller_state is None and self._controller_drives_budget:
            controller_state = self.controller.current_state()
        return resolve_budget_state(self.args, controller_state)

    def edge_seed(self, epoch: int) -> int:
        return edge_seed_for_epoch(self.args, epoch, self._static_seed_epochs)

    # ------------------------------------------------------------------------------------------ step
    def _loss(self, graph: AttnGraph, idx: torch.Tensor, x_local: Optional[torch.Tensor] = None):
        """Mean loss over this rank's nodes in ``idx`` (main_node_fullgraph_sp.py:1214-1240): NLL of the
        log-softmax output, or BCE-with-logits for multi-label targets.  A rank without such nodes
        contributes ``out.sum() * 0`` so that every collective still runs."""
        x = self.x_local if x_local is None else x_local
        attn_type = getattr(self.args, "attn_type", "sparse")
        with autocast_context(self.device, self.amp_dtype):
            if self.multilabel:
                out = self.model.forward_logits(x, None, graph, attn_type=attn_type)
                if idx.numel() == 0:
                    return out.sum() * 0, out
                return F.binary_cross_entropy_with_logits(out[idx].float(), self.local_y[idx].float()), out
            if self.device.type == "cuda" and hasattr(self.model, "forward_logits"):
                # fused log-softmax + NLL (+ gradient) over this rank's rows of `idx`; `out` are logits, whose argmax
                # equals the argmax of the log-probabilities the model would return
                from ..ops.loss import masked_nll
                out = self.model.forward_logits(x, None, graph, attn_type=attn_type)
                if idx.numel() == 0:
                    return out.sum() * 0, out
                return masked_nll(out, self.local_y, idx, self._loss_mask(idx)), out
            out = self.model(x, None, graph, attn_type=attn_type)
            if idx.numel() == 0:
                return out.sum() * 0, out
            return F.nll_loss(out[idx].float(), self.local_y[idx]), out

    def _loss_mask(self, idx: torch.Tensor) -> torch.Tensor:
        """uint8 row mask of ``idx`` (cached per index tensor: the train / probe sets are fixed)."""
        cache = self.__dict__.setdefault("_mask_cache", {})
        key = (idx.data_ptr(), int(idx.numel()))
        m = cache.get(key)
        if m is None:
            m = torch.zeros(self.nodes_per_rank, dtype=torch.uint8, device=self.device)
            m[idx] = 1
            cache[key] = m
        return m

    def _any_rank(self, flag: bool) -> bool:
        """MAX-vote over SP ranks (``_sp_any_oom``, main_node_fullgraph_sp.py:1313-1318)."""
        if self.sp_world == 1:
            return bool(flag)
        dev = comm.comm_device(self.sp_group, self.device)
        return comm.all_reduce_scalar(1.0 if flag else 0.0, "max", self.sp_group, dev) > 0.5

    def _cleanup_after_oom(self) -> None:
        for p in self.model.parameters():
            if p.grad is not None:
                p.grad.zero_()
        gc.collect()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            torch.cuda.empty_cache()
        gc.collect()

    def _fwd_bwd(self, graph: AttnGraph, epoch: int, x_local, timers: Dict[str, float], sync_timers: bool):
        """Forward, backward and gradient reduction of one step; everything that can fail on one rank only."""
        self.model.train()
        stage = {"bwd_started": False}
        if debug.enabled():
            debug.validate_graph(graph)
        sp_ctx = getattr(self.model, "_fused_sp_context", None)
        if sp_ctx is not None:
            sp_ctx.step_seed = (int(self.args.seed) * 1000003 + int(epoch)) & 0x7FFFFFFF     # identical on every rank
        with StepTimer(self.device, sync_timers) as t_fwd, comm_profiler.nvtx_range("forward"):
            self.fault.check("fwd", epoch)
            ctx = torch.autograd.graph.save_on_cpu(pin_memory=True) if (
                getattr(self.args, "activation_cpu_offload", False) and self.planner is None
                and self.device.type == "cuda") else _null()
            with ctx:
                loss, _ = self._loss(graph, self.local_idx["train"], x_local)
        with StepTimer(self.device, sync_timers) as t_bwd, comm_profiler.nvtx_range("backward"):
            self.reducer.prepare_backward()
            stage["bwd_started"] = True
            self._stage = stage
            self.fault.check("bwd", epoch)
            if self.scaler.is_enabled():
                self.scaler.scale(loss).backward()
            else:
                loss.backward()
            self.reducer.finalize_backward()
        if debug.enabled():
            debug.assert_finite(f"the loss of epoch {epoch}", loss.detach())
            debug.assert_finite(f"the gradients of epoch {epoch}", *[p.grad for p in self.model.parameters()])
        self.fault.check("opt", epoch)          # last point at which a one-rank failure can still be voted on
        timers.update(fwd=t_fwd.elapsed, bwd=t_bwd.elapsed)
        return loss

    def _optimizer_step(self, timers: Dict[str, float], sync_timers: bool) -> None:
        """Clip + AdamW + schedule.  Runs only after every rank voted that its forward and backward went through, so a
        rank can never apply an update that the others drop."""
        with StepTimer(self.device, sync_timers) as t_opt, comm_profiler.nvtx_range("optimizer"):
            if self.scaler.is_enabled():
                self.scaler.unscale_(self.optimizer)
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
                self.scaler.step(self.optimizer)
                self.scaler.update()
            elif self.flat_optimizer:
                self.optimizer.step()                      # clipping is fused into the step
            else:
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
                self.optimizer.step()
            self.lr_scheduler.step()
        timers.update(opt=t_opt.elapsed)

    def _step_with_oom_recovery(self, graph, epoch, x_local, timers, sync_timers):
        """Voted OOM protocol (main_node_fullgraph_sp.py:1320-1507).  Every attempt ends with one packed MAX vote
        (failed here?, had backward started?, did a device-side wait expire?) taken after the gradient reduction has
        been launched and before the optimizer: on a failure all ranks clean up and then either demote one activation
        tier (plan ACTIVE), mark the tier under calibration infeasible, or abort; a failure after backward started
        drops the step.  The vote travels over the host-side group, so it does not drain the GPU queue."""
        from torch.utils.checkpoint import CheckpointError
        attempt = 0
        while True:
            attempt += 1
            failed, err = False, None
            self._stage = {"bwd_started": False}
            loss = None
            try:
                loss = self._fwd_bwd(graph, epoch, x_local, timers, sync_timers)
            except (torch.cuda.OutOfMemoryError, CheckpointError) as e:
                failed, err = True, e
            expired = self._take_device_status()
            any_failed, bwd_started, any_expired = self._vote(failed, self._stage.get("bwd_started", False), expired != 0)
            if any_expired:
                self._abort_on_expired_wait(expired)
            if not any_failed:
                self._optimizer_step(timers, sync_timers)
                self.consecutive_dropped = 0
                return loss
            del loss
            self._cleanup_after_oom()
            self._resync_device_barriers()
            self.log(f"[oom] step failed on some rank (attempt {attempt}, bwd_started={bwd_started}): "
                     f"{type(err).__name__ if err else 'remote'}")
            if self.planner is None:
                raise RuntimeError("out of memory in the training step and no multi_tier planner to adapt") from err
            if self.planner.is_active():
                if not self.planner.apply_oom_fallback(self.device, self.sp_group, self.sp_world):
                    raise RuntimeError("out of memory with every layer already recomputed") from err
            elif not self.planner.mark_current_calibration_infeasible(self.device):
                # warm-up (every layer recomputed) does not fit.  What can still be given back is the memory of a GPU
                # edge policy - the resident topology and the build's working set: GPU policies leave the planner's
                # search, the graph build moves to the CPU with prefetch and the step is retried from the next epoch
                # (the reference marks gpu_persist infeasible at this point too, main_node_fullgraph_sp.py:1431-1444)
                if self.edge_engine.policy.startswith("gpu") and not self.edge_engine.policy_locked \
                        and self.planner.report_runtime_edge_gpu_infeasible(self.device):
                    self.edge_engine.set_policy("cpu_rank_local_prefetch")
                    self._cleanup_after_oom()
                    self.log("[multi_tier] out of memory during warm-up under a GPU edge policy: "
                             "edge build moved to cpu_rank_local_prefetch, step dropped")
                    self.consecutive_dropped += 1
                    raise StepDropped() from err
                raise RuntimeError("out of memory during warm-up with every layer recomputed") from err
            if bwd_started or attempt >= MAX_STEP_RETRIES:
                self.consecutive_dropped += 1
                if self.consecutive_dropped >= MAX_CONSECUTIVE_DROPPED:
                    raise RuntimeError(f"{MAX_CONSECUTIVE_DROPPED} consecutive steps dropped after OOM") from err
                raise StepDropped()

    def _vote(self, *flags: bool):
        """Element-wise OR over the SP ranks of several flags in one collective."""
        if self.sp_world == 1:
            return tuple(bool(f) for f in flags)
        dev = comm.comm_device(self.sp_group, self.device)
        vals = comm.all_reduce_scalars([1.0 if f else 0.0 for f in flags], "max", self.sp_group, dev)
        return tuple(v > 0.5 for v in vals)

    # ---- device-side status word ----------------------------------------------------------------------------
    # Kernels with bounded waits (the peer barrier, the GEMM's mbarrier waits) report an expired wait by writing a
    # status word and returning; what they computed after that is invalid.  The word is copied to pinned host memory
    # at the end of every step without stalling the launch queue and examined once that copy has landed, which the
    # run-ahead bound of two steps guarantees before the step after next is launched.
    def _queue_device_status_read(self) -> None:
        if self.device.type != "cuda" or not self.fused_sp:
            return
        from ..ops.gemm import status_tensor
        pipe = self.__dict__.setdefault("_status_pipe", {"host": torch.zeros(2, 4, dtype=torch.int32).pin_memory(),
                                                         "events": [None, None], "slot": 0})
        slot = pipe["slot"]
        pipe["host"][slot].copy_(status_tensor(self.device), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        pipe["events"][slot] = ev
        pipe["slot"] = slot ^ 1

    def _take_device_status(self) -> int:
        """Status word of the most recent step whose copy has completed (0 = healthy)."""
        pipe = self.__dict__.get("_status_pipe")
        if pipe is None:
            return 0
        code = 0
        for slot in (0, 1):
            ev = pipe["events"][slot]
            if ev is not None and ev.query():
                code = code or int(pipe["host"][slot][0])
                pipe["events"][slot] = None
        return code

    def _abort_on_expired_wait(self, local_code: int) -> None:
        """Some rank saw a bounded device-side wait give up: the steps launched since then computed on data a peer had
        not finished writing.  The reference's NCCL collectives would have blocked until their time-out and ended the
        job; so does this - on every rank, after the same vote."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        raise RuntimeError(
            f"a device-side bounded wait expired on {'this rank' if local_code else 'another rank'} "
            f"(status {local_code}): a peer did not reach a barrier in time, results since then are invalid")

    def _resync_device_barriers(self) -> None:
        """After a step that failed on the host of some rank the ranks have issued different numbers of device
        barriers; bring the epoch counters back together before anything is launched again."""
        if self.fused_sp and self.sp_world > 1 and self.device.type == "cuda":
            from ..parallel import symm
            symm.get_world(self.sp_group, self.device).resync()

    def build_edges(self, epoch: int) -> AttnGraph:
        """Build (or fetch the prefetched) attention graph of ``epoch`` with a voted retry on failure
        (main_node_fullgraph_sp.py:1097-1163)."""
        seed, state = self.edge_seed(epoch), self.budget_state()
        failed, err, g = False, None, None
        try:
            self.fault.check("edge", epoch)
            g = self.edge_engine.build(seed, state)
        except torch.cuda.OutOfMemoryError as e:
            failed, err = True, e
        if self._any_rank(failed or self.edge_engine.gpu_build_failed):
            self._cleanup_after_oom()
            self.edge_engine.gpu_build_failed = False
            if self.planner is not None:
                self.planner.report_runtime_edge_gpu_infeasible(self.device)
                self.sync_active_plan()
            if not self.edge_engine.policy.startswith("cpu"):
                self.edge_engine.set_policy("cpu_rank_local_prefetch")
            self.log("[edge-cache] GPU edge build failed on some rank; rebuilding with a CPU policy")
            if failed or g is None:
                g = self.edge_engine.build(seed, state)
        return g

    def train_step(self, epoch: int, x_host: Optional[torch.Tensor] = None, read_loss: bool = True) -> Dict[str, float]:
        """One epoch = edge build + forward + backward + gradient reduction + optimizer step.

        ``x_host`` (pinned ``[N/P, d]``) makes the step copy its input features host -> device inside the step
        (the end-to-end measurement path); otherwise the resident device copy is used.  With ``read_loss``
        the loss is read back to the host (one 4-byte device -> host copy)."""
        self.epoch = epoch
        if self.device.type == "cuda":
            # bound the host's run-ahead to two steps: deeper queues only grow the caching allocator (blocks shared with
            # the look-ahead stream are recycled late) and make its growth calls land inside later steps
            pending = self.__dict__.setdefault("_step_done", [])
            if len(pending) >= 2:
                pending.pop(0).synchronize()
        sync_timers = bool(getattr(self.args, "profile_sp_comm", False)) or (
            self.planner is not None and self.planner.needs_precise_timing())
        timers: Dict[str, float] = {"rw": 0.0, "fwd": 0.0, "bwd": 0.0, "opt": 0.0, "prefetch_wait": 0.0}
        t0 = time.perf_counter()
        x_local = None
        if x_host is not None:
            x_local = self._stage_input(x_host)
        with StepTimer(self.device, sync_timers) as t_rw, comm_profiler.nvtx_range("edge_build"):
            graph = self.build_edges(epoch)
        timers["rw"] = t_rw.elapsed
        timers["prefetch_wait"] = self.edge_engine.last_prefetch_wait_s
        if self._next_budget_known():
            self.edge_engine.submit_prefetch(self.edge_seed(epoch + 1), self.budget_state())
        self.last_graph = graph
        out: Dict[str, float] = {"dropped": 0.0}
        try:
            loss = self._step_with_oom_recovery(graph, epoch, x_local, timers, sync_timers)
            if read_loss == "async":
                # device -> host copy of this step's loss into pinned memory without stalling the launch queue; the
                # value returned is the previous step's (its copy has completed by now), the last one via flush_loss()
                out["loss"] = self._read_loss_async(loss.detach())
            elif read_loss:
                out["loss"] = float(loss.item())
                self.loss_ema = out["loss"] if self.loss_ema is None else 0.9 * self.loss_ema + 0.1 * out["loss"]
            else:
                out["loss_tensor"] = loss.detach()
        except StepDropped:
            out["dropped"], out["loss"] = 1.0, float("nan")
            comm.barrier(self.sp_group)
        if not out["dropped"] and (self.planner is not None or getattr(self.model, "_comm_ckpt", None) is not None):
            # a dropped step measured nothing the planner may use (its peak is the failed allocation's)
            self.model.comm_aware_notify_step_end(self.device, t_bwd=timers["bwd"], t_fwd=timers["fwd"])
        if self.device.type == "cuda":
            self._queue_device_status_read()
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream(self.device))
            self._step_done.append(done)
        timers["total"] = time.perf_counter() - t0
        out.update({f"t_{k}": v for k, v in timers.items()})
        out["edges"] = float(graph.num_edges)
        return out

    def _read_loss_async(self, loss: torch.Tensor) -> float:
        if self.device.type != "cuda":
            return float(loss)
        st = self.__dict__.setdefault("_loss_pipe", {"buf": torch.zeros(2, dtype=torch.float32).pin_memory(),
                                                     "events": [None, None], "slot": 0})
        slot = st["slot"]
        prev = float("nan")
        other = slot ^ 1
        if st["events"][other] is not None:
            st["events"][other].synchronize()
            prev = float(st["buf"][other])
        st["buf"][slot:slot + 1].copy_(loss.reshape(1).float(), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        st["events"][slot] = ev
        st["slot"] = other
        return prev

    def flush_loss(self) -> float:
        """Value of the most recent asynchronous loss read (waits for its copy)."""
        st = self.__dict__.get("_loss_pipe")
        if st is None:
            return float("nan")
        last = st["slot"] ^ 1
        if st["events"][last] is None:
            return float("nan")
        st["events"][last].synchronize()
        return float(st["buf"][last])

    def _stage_input(self, x_host: torch.Tensor) -> torch.Tensor:
        """Host -> device input pipeline: this step's features were uploaded from pinned memory on a copy stream while
        the previous step computed (double buffer); the upload for the next step is started before returning.  Every
        step therefore consumes exactly one full host -> device copy, overlapped with compute."""
        if self.device.type != "cuda":
            return x_host.to(self.device)
        st = getattr(self, "_input_pipe", None)
        if st is None or st["shape"] != tuple(x_host.shape):
            st = {"shape": tuple(x_host.shape), "stream": torch.cuda.Stream(self.device), "bufs": [
                torch.empty(x_host.shape, dtype=x_host.dtype, device=self.device) for _ in range(2)],
                "events": [None, None], "src": [None, None], "next": 0}
            self._input_pipe = st
        cur_stream = torch.cuda.current_stream(self.device)

        def upload(slot):
            st["stream"].wait_stream(cur_stream)            # the buffer's previous consumer has been enqueued before
            with torch.cuda.stream(st["stream"]):
                st["bufs"][slot].copy_(x_host, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(st["stream"])
            st["events"][slot], st["src"][slot] = ev, x_host.data_ptr()

        slot = st["next"]
        if st["events"][slot] is None or st["src"][slot] != x_host.data_ptr():
            upload(slot)                                     # first step (or a new host tensor): nothing prefetched yet
        cur_stream.wait_event(st["events"][slot])
        x = st["bufs"][slot]
        st["events"][slot] = None
        st["next"] = slot ^ 1
        upload(slot ^ 1)                                     # prefetch for the next step
        return x

    def _align_ranks(self) -> None:
        """Stream-ordered NCCL rendezvous before a fused forward outside the training step (evaluation, budget
        probes).  The in-kernel barriers of the fused path use bounded spins (a few seconds); this keeps host-side
        skew between ranks (metrics on rank 0, logging) out of those spins.  The training step needs none: the
        host-side vote on the graph build, taken by every rank right before it launches the step, already is a
        rendezvous of the hosts, and it queues nothing on the GPU."""
        if self.fused_sp and self.sp_world > 1:
            if not hasattr(self, "_align_buf"):
                self._align_buf = torch.zeros(1, device=self.device)
            dist.all_reduce(self._align_buf, group=self.sp_group)

    def _next_budget_known(self) -> bool:
        """Prefetch only when the next epoch's budget cannot change (main_node_fullgraph_sp.py:545-555)."""
        return (not self.budget_cfg.enabled) or self.controller.frozen or self.epoch <= int(self.args.warmup_updates)

    # ------------------------------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def evaluate(self, epoch: int) -> Optional[Dict[str, float]]:
        """No-grad forward on the local slice, predictions gathered to rank 0, metrics on CPU
        (utils/fullgraph_sp_support.py:3379-3477).  The graph is the epoch's training graph (same seed and
        budget => cache hit)."""
        t0 = time.perf_counter()
        self.model.eval()
        graph = getattr(self, "last_graph", None)
        if graph is None:
            graph = self.build_edges(epoch)
        self._align_ranks()
        attn_type = getattr(self.args, "attn_type", "sparse")
        with autocast_context(self.device, self.amp_dtype):
            if self.multilabel:
                out = self.model.forward_logits(self.x_local, None, graph, attn_type=attn_type)
                pred = (out > 0).to(torch.uint8)
            else:
                out = self.model(self.x_local, None, graph, attn_type=attn_type)
                if str(self.args.dataset).lower() == "genius":
                    pred = out.float().exp()[:, 1]
                else:
                    pred = out.argmax(dim=1)
        if self.sp_world > 1:
            parts = [torch.empty_like(pred) for _ in range(self.sp_world)]
            dist.all_gather(parts, pred.contiguous(), group=self.sp_group)
            pred = torch.cat(parts, 0)
        self.model.train()
        res = None
        if self.rank == 0:
            pred = pred.cpu()
            y = self.data.y
            res = {}
            for name, idx in self.data.split_idx.items():
                if idx.numel() == 0:
                    res[name] = 0.0
                elif self.multilabel:
                    res[name] = float((pred[idx] == y[idx].to(torch.uint8)).float().mean())
                elif str(self.args.dataset).lower() == "genius":
                    from sklearn.metrics import roc_auc_score
                    res[name] = float(roc_auc_score(y[idx].numpy(), pred[idx].float().numpy()))
                else:
                    res[name] = float((pred[idx] == y[idx]).float().mean())
        self.eval_times.append(time.perf_counter() - t0)
        return res

    # ------------------------------------------------------------------------------------------ budget probe
    @torch.no_grad()
    def _probe_loss(self, state: dict, seed: int):
        """Loss / accuracy of the current weights on the probe nodes under budget ``state``
        (``_probe_loss_sp``, utils/fullgraph_sp_support.py:2318-2358): three SUM reductions packed into one."""
        graph = self.edge_engine.build(seed, resolve_budget_state(self.args, state), record=False)
        self._align_ranks()
        idx = self.probe_local_idx
        was_training = self.model.training
        self.model.eval()
        loss, out = self._loss(graph, idx)
        self.model.train(was_training)
        n = float(idx.numel())
        if n > 0 and not self.multilabel:
            correct = float((out[idx].argmax(1) == self.local_y[idx]).sum())
        elif n > 0:
            correct = float(((out[idx] > 0) == (self.local_y[idx] > 0.5)).float().mean(1).sum())
        else:
            correct = 0.0
        vals = [float(loss) * n, correct, n]
        if self.sp_world > 1:
            vals = comm.all_reduce_scalars(vals, "sum", self.sp_group, comm.comm_device(self.sp_group, self.device))
        tot = max(vals[2], 1.0)
        return vals[0] / tot, vals[1] / tot, graph.num_edges

    def maybe_update_edge_budget(self, epoch: int) -> None:
        c = self.controller
        if (not c.enabled) or c.frozen or epoch <= int(self.args.warmup_updates) or (
                c.warmup_epochs is not None and epoch > c.warmup_epochs):
            return
        n_probe = float(self.probe_local_idx.numel()) if self.probe_local_idx is not None else 0.0
        if self.sp_world > 1:
            n_probe = comm.all_reduce_scalar(n_probe, "sum", self.sp_group, comm.comm_device(self.sp_group, self.device))
        if n_probe <= 0:
            c.frozen = True
            return
        if c.over_limit:
            ns = c.force_shrink() or c.current_state()
            self.log(f"  ↳ BudgetCtrl shrink epoch={epoch} (peak over GPU limit) "
                     f"new_budget=({ns['real_edges_per_query']},{ns['rw_edges_per_query']})")
            return
        seed = self.edge_seed(epoch)      # common random numbers: candidate edge sets are nested in the budget
        rows = []
        base = c.current_state()
        for kind, state in [("current", base)] + list(c.candidate_states().items()):
            failed = False
            try:
                self.fault.check("probe", epoch)
                loss, acc, edges = self._probe_loss(state, seed)
            except torch.cuda.OutOfMemoryError:
                failed = True
                loss, acc, edges = float("inf"), 0.0, 0
            if self._any_rank(failed):
                self._cleanup_after_oom()
                loss, acc, edges = float("inf"), 0.0, 0
                if kind == "current":
                    return
            rows.append({"kind": kind, "state": state, "loss": loss, "acc": acc, "edges": edges})
        decide_budget_move(c, rows, epoch, self.log)
        self.edge_engine.clear_cache()

    # ------------------------------------------------------------------------------------------ planner hooks
    def observe_memory_for_budget(self) -> None:
        if self.device.type != "cuda" or not self.budget_cfg.enabled or self.controller.frozen:
            return
        peak = torch.cuda.max_memory_allocated(self.device) / 2 ** 20
        if self.sp_world > 1:
            peak = comm.all_reduce_scalar(peak, "max", self.sp_group, comm.comm_device(self.sp_group, self.device))
        self.controller.observe_peak(peak)

    def notify_budget_frozen_if_needed(self) -> None:
        """When the controller freezes, the planner leaves DEFERRED (main_node_fullgraph_sp.py:1587-1622)."""
        if self._budget_frozen_notified or not self.controller.frozen:
            return
        self._budget_frozen_notified = True
        self._release_probe_memory()
        self.model.comm_aware_notify_budget_frozen(reuse_deferred_baseline=True)
        if self.planner is not None and not self.edge_engine.policy_locked:
            self.profile_edge_policies()

    def _release_probe_memory(self) -> None:
        """The budget search is over: drop the host-side graphs it left in the cache and hand freed heap pages back to
        the system, so that the resident set the planner calibrates against is the steady-state one
        (``_release_probe_caches_on_freeze``, utils/fullgraph_sp_support.py:3142-3168)."""
        import gc
        from ..utils.misc import glibc_malloc_trim
        self.edge_engine.clear_cache()
        gc.collect()
        glibc_malloc_trim()

    def profile_edge_policies(self) -> None:
        """Measure each placement policy once (cold + warm build with a bumped seed) and hand the profiles to
        the planner (``_profile_multi_tier_edge_policy``, utils/fullgraph_sp_runtime.py:251-546)."""
        if self.planner is None:
            return
        from ..control.profile import profile_edge_policies
        profile_edge_policies(self)

    def sync_active_plan(self) -> None:
        """Cross-rank consensus on the ACTIVE plan: MAX-reduce the policy id and MIN-reduce the tier ids in one
        packed collective, then lock the runtime policy (``_apply_multi_tier_active_plan``,
        utils/fullgraph_sp_runtime.py:618-816)."""
        p = self.planner
        if p is None or not p.is_active() or self.edge_engine.policy_locked and getattr(self, "_plan_applied", False):
            return
        pol_id = EDGE_POLICY_ORDER.index(p.edge_policy)
        tiers = [TIER_IDS[m] for m in p.modes()]
        if self.sp_world > 1:
            dev = comm.comm_device(self.sp_group, self.device)
            vals = comm.all_reduce_scalars([float(pol_id)] + [-float(t) for t in tiers], "max", self.sp_group, dev)
            pol_id, tiers = int(vals[0]), [int(-v) for v in vals[1:]]
        policy = EDGE_POLICY_ORDER[pol_id]
        p.override_active_plan(policy, [TIER_FROM_ID[t] for t in tiers])
        self.edge_engine.set_policy(policy, lock=True)
        from ..graph.device_budget import BUDGET
        BUDGET.set_force_gpu_build(policy.startswith("gpu") and p.rw_on_gpu)   # set on every (re-)plan, never stale
        self._plan_applied = True

    # ------------------------------------------------------------------------------------------ loop
    def fit(self) -> Dict[str, float]:
        from .checkpoint import save_best_model, save_train_state
        from .report import print_training_header, print_training_summary
        args = self.args
        print_training_header(self)
        if (self.planner is not None and self.controller.frozen and not self.edge_engine.policy_locked
                and not self.planner.is_active() and not self.planner.edge_costs):
            # the budget never moves (fixed split, or a resumed run whose search is over): the placement policies are
            # measured once before the first step, as the reference does at its first epoch with a frozen budget
            # (main_node_fullgraph_sp.py:665-988)
            self.profile_edge_policies()
        start_epoch = self.epoch + 1
        for epoch in range(start_epoch, int(args.epochs) + 1):
            if self.device.type == "cuda":
                torch.cuda.reset_peak_memory_stats(self.device)
            self.fault.check("step", epoch)
            if self.watchdog is not None:
                # between steps, nothing of this rank in flight: post the heartbeat and learn of a lost peer on the
                # host before the next launch (raises PeerLost on every surviving rank)
                self.watchdog.beat(epoch)
                self.watchdog.check()
            if self.planner is not None and self.planner.is_active() and not getattr(self, "_plan_applied", False):
                self.sync_active_plan()
            t_ep = time.time()
            stats = self.train_step(epoch)
            self.observe_memory_for_budget()
            t_adj0 = time.perf_counter()
            self.maybe_update_edge_budget(epoch)
            self.notify_budget_frozen_if_needed()
            t_adj = time.perf_counter() - t_adj0
            comm.barrier(self.sp_group)
            wall = time.time() - t_ep
            if self.sp_world > 1:
                dev = comm.comm_device(self.sp_group, self.device)
                wall, prep, wait = comm.all_reduce_scalars([wall, stats["t_rw"], stats["t_prefetch_wait"]], "max",
                                                           self.sp_group, dev)
            else:
                prep, wait = stats["t_rw"], stats["t_prefetch_wait"]
            self.epoch_times.append(wall)
            self.prep_times.append(prep)
            if self.planner is not None and self.planner.is_active():
                self.planner.reconsider_with_actual_timing(self.device, stats["t_fwd"] + stats["t_bwd"], wait)
            ema = self.loss_ema if self.loss_ema is not None else float("nan")
            self.log(f"Epoch {epoch:04d} | loss={stats['loss']:.4f} (ema={ema:.4f}) | t={wall:.3f}s "
                     f"(rw={stats['t_rw']:.3f} fwd={stats['t_fwd']:.3f} bwd={stats['t_bwd']:.3f} "
                     f"opt={stats['t_opt']:.3f} adj={t_adj:.3f} prefetch_wait={wait:.3f}) | "
                     f"cpu_rss={process_rss_mib():.0f}/{process_peak_rss_mib():.0f} MiB")
            if getattr(args, "profile_sp_comm", False):
                from .report import format_comm_profile
                self.log(format_comm_profile(comm_profiler.get_comm_profile_summary(reset=True), wall))
            if self._metrics_fh is not None:
                rec = {"epoch": epoch, "loss": stats["loss"], "epoch_s": wall, "nodes_per_s": self.data.num_nodes / wall,
                       "edges": stats["edges"], "peak_hbm_mib": (torch.cuda.max_memory_allocated(self.device) / 2 ** 20
                                                                  if self.device.type == "cuda" else 0.0)}
                self._metrics_fh.write(json.dumps(rec) + "\n")
                self._metrics_fh.flush()
            if epoch % max(1, int(args.eval_every)) == 0 or epoch == int(args.epochs):
                res = self.evaluate(epoch)
                if self.rank == 0 and res is not None:
                    self.log(f"  eval epoch {epoch:04d} | train={res['train']:.4f} valid={res['valid']:.4f} "
                             f"test={res['test']:.4f}")
                    if res["valid"] > self.best["valid"]:
                        self.best = {**res, "epoch": epoch}
                        if getattr(args, "save_model", False):
                            path = save_best_model(self)
                            self.log(f"  saved best model to {path}")
                if getattr(args, "save_model", False):
                    save_train_state(self)
        self.edge_engine.shutdown()
        if self.watchdog is not None:
            self.watchdog.stop()
        print_training_summary(self)
        if self._metrics_fh is not None:
            self._metrics_fh.close()
        return dict(self.best)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
