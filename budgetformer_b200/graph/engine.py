"""Edge construction engine: budget resolution, placement policies, prefetch and caching.

One ``EdgeEngine`` per rank owns the raw ``Topology`` (host copy in pinned memory, optional device
copy) and produces the epoch's ``AttnGraph`` on the training device.  Placement policies are the
reference's (utils/fullgraph_sp_support.py:394-402, gt_sp/multi_tier.py:1210-1223):

=========================  ====================================================================
``gpu_persist``            topology resident in HBM, sample + walk on the GPU every epoch
``gpu_ephemeral``          topology uploaded from pinned memory each epoch, built on GPU, freed
``cpu_rank_local_prefetch``  every rank builds on CPU (C++/OpenMP) in a background thread and
                           uploads the compact CSR (int32, ``4*(N+1+E_m)`` bytes) asynchronously
``cpu_broadcast_prefetch`` the source rank builds on CPU in the background and broadcasts
``cpu_broadcast``          same, synchronously (baseline while the budget is still moving)
=========================  ====================================================================

Because the builders are counter-based and bit-identical on CPU and GPU, the rank-local policies
need no communication; broadcast exists for parity and for ``--force_edge_broadcast``.
"""
from __future__ import annotations

import os
import threading
import time
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..utils.comm_profiler import profile_call, record_scalar
from .device_budget import BUDGET
from .attn_graph import AttnGraph, Topology, add_virtual_node
from .builder import ShardedDeviceBuild, build_attn_graph, build_attn_graph_shard, graph_totals, native_supported

EDGE_POLICY_CHOICES = ("gpu_persist", "gpu_ephemeral", "cpu_rank_local_prefetch", "cpu_broadcast_prefetch",
                       "cpu_broadcast")
_CPU_POLICIES = ("cpu_rank_local_prefetch", "cpu_broadcast_prefetch", "cpu_broadcast")


@dataclass(frozen=True)
class BudgetState:
    """Resolved per-query budgets for one build.  ``None`` = unsampled (all candidates)."""
    use_real: bool
    use_rw: bool
    b_real: Optional[int]
    b_rw: Optional[int]
    walk_length: int

    def key(self) -> tuple:
        return (self.use_real, self.use_rw, self.b_real, self.b_rw, self.walk_length)


def resolve_budget_state(args, controller_state: Optional[dict] = None) -> BudgetState:
    """Decision table of utils/fullgraph_sp_support.py:830-915.

    * fixed / adaptive state given  -> that split (0 drops a side);
    * ``--random_edge_blocks --max_total_edges_per_query B`` -> ``(B+1)//2`` real, ``B//2`` walk
      (all ``B`` to real when ``walks_per_node == 0``);
    * otherwise -> all real edges iff ``--include_real_edges 1``, the full walk pool iff ``walks_per_node > 0``.

    ``--rw_edge_mode dgl_neighbor`` builds its pool from the fan-out, so ``walks_per_node`` does not gate the walk
    side there (:905-915)."""
    wl = int(getattr(args, "walk_length", 4))
    wpn = int(getattr(args, "walks_per_node", 0))
    walks_on = wpn > 0 or str(getattr(args, "rw_edge_mode", "random_walk")) == "dgl_neighbor"
    if controller_state is not None:
        r = int(controller_state.get("real_edges_per_query", 0))
        w = int(controller_state.get("rw_edges_per_query", 0))
        wl = int(controller_state.get("walk_length", getattr(args, "fixed_walk_length", None) or wl))
        return BudgetState(r > 0, w > 0 and walks_on, r, w, wl)
    total = int(getattr(args, "max_total_edges_per_query", 0) or 0)
    if getattr(args, "random_edge_blocks", False) and total > 0:
        if wpn <= 0:
            return BudgetState(True, False, total, 0, wl)
        return BudgetState(True, True, (total + 1) // 2, total // 2, wl)
    return BudgetState(bool(int(getattr(args, "include_real_edges", 0))), walks_on, None, None, wl)


def edge_seed_for_epoch(args, epoch: int, static_seed_epochs: int = 0) -> int:
    """``seed`` while ``epoch <= static_seed_epochs`` else ``seed + epoch`` (utils/fullgraph_sp_runtime.py:221-226)."""
    return int(args.seed) if epoch <= int(static_seed_epochs) else int(args.seed) + int(epoch)


class EdgeEngine:
    def __init__(self, args, edge_index_global: torch.Tensor, num_nodes: int, device, *, nodes_per_rank: int,
                 sp_group=None, sp_rank: int = 0, sp_src_rank: int = 0, sp_world: int = 1,
                 expander_edges: Optional[torch.Tensor] = None):
        self.args = args
        self.device = torch.device(device)
        self.num_nodes = int(num_nodes)                 # padded node count
        self.nodes_per_rank = int(nodes_per_rank)
        self.group, self.rank, self.src_rank, self.world = sp_group, int(sp_rank), int(sp_src_rank), int(sp_world)
        self.model = str(getattr(args, "model", "gt"))
        self.virtual_node = self.model == "graphormer" and int(getattr(args, "num_global_node", 0)) > 0
        self.exphormer = self.model == "exphormer"
        self.expander_edges = expander_edges
        self.fanout = None
        if str(getattr(args, "rw_edge_mode", "random_walk")) == "dgl_neighbor":
            from .builder_spec import parse_fanout
            self.fanout = parse_fanout(getattr(args, "fanout", "10,5"))
        t0 = time.perf_counter()
        if self.device.type == "cuda" and edge_index_global.size(1) >= 20_000_000:
            # the two CSR forms need a sort and a unique over all edges: seconds on the GPU, minutes on the host
            try:
                self.topo_cpu = Topology.from_edge_index(edge_index_global.to(self.device), self.num_nodes).to("cpu")
                torch.cuda.empty_cache()
            except torch.cuda.OutOfMemoryError:
                torch.cuda.empty_cache()
                self.topo_cpu = Topology.from_edge_index(edge_index_global.cpu(), self.num_nodes)
        else:
            self.topo_cpu = Topology.from_edge_index(edge_index_global.cpu(), self.num_nodes)
        if self.device.type == "cuda":
            try:
                self.topo_cpu = self.topo_cpu.pin_memory()
            except RuntimeError:
                pass
        self.t_topology_build = time.perf_counter() - t0
        self.topo_gpu: Optional[Topology] = None
        self.policy = self._initial_policy()
        self.policy_locked = False
        self.force_broadcast = bool(getattr(args, "force_edge_broadcast", False))
        self._cache: Dict[tuple, AttnGraph] = {}        # up to 2 finished host-side builds (prefetch hand-off)
        self._cache_lock = threading.Lock()
        self._pool: Optional[ThreadPoolExecutor] = None
        self._future: Optional[Tuple[tuple, Future]] = None
        self._copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self._build_stream = None                        # side stream of the device-side look-ahead build
        self._dev_future: Optional[Tuple[tuple, Future]] = None
        self.last_build_s = 0.0
        self.last_prefetch_wait_s = 0.0
        self.last_graph_bytes = 0
        self.gpu_build_failed = False
        self.build_threads = self._resolve_build_threads()
        # device builds split over the ranks: one instance (and barrier channel) per host thread that builds
        self._shard_builds = {}

    def _resolve_build_threads(self) -> int:
        """OpenMP threads of a host-side build: ``--edge_build_threads`` or the cores this process may use divided by
        the ranks on this node.  Launchers export OMP_NUM_THREADS=1 for multi-process jobs, which would otherwise
        make every host build single-threaded."""
        n = int(getattr(self.args, "edge_build_threads", 0) or 0)
        if n > 0:
            return n
        try:
            cores = len(os.sched_getaffinity(0))
        except (AttributeError, OSError):
            cores = os.cpu_count() or 1
        local = int(os.environ.get("LOCAL_WORLD_SIZE", "0") or 0) or max(1, self.world)
        return max(1, cores // max(1, local))

    # ------------------------------------------------------------------ policy
    def _initial_policy(self) -> str:
        dev = str(getattr(self.args, "edge_build_device", "gpu")).lower()
        if self.device.type != "cuda" or dev == "cpu" or self.fanout:
            return "cpu_rank_local_prefetch"      # fan-out graphs are built by the C++ builder: prefetch hides it
        return "gpu_persist"

    def set_policy(self, policy: str, lock: bool = False) -> None:
        if policy not in EDGE_POLICY_CHOICES:
            raise ValueError(f"unknown edge policy {policy!r}")
        if (self.device.type != "cuda" or self.fanout) and policy.startswith("gpu"):
            policy = "cpu_rank_local_prefetch"
        if policy != self.policy:
            self.clear_cache()
        self.policy = policy
        self.policy_locked = bool(lock)
        if policy != "gpu_persist":
            self.topo_gpu = None

    def build_devices(self) -> Tuple[str, str]:
        """(final device, walk device) of the active policy (utils/fullgraph_sp_support.py:394-402)."""
        if self.policy in ("cpu_broadcast", "cpu_broadcast_prefetch"):
            return "cpu", "cpu"
        if self.policy == "cpu_rank_local_prefetch":
            return str(self.device), "cpu"
        return str(self.device), str(self.device)

    def uses_prefetch(self) -> bool:
        return (self.policy in ("cpu_rank_local_prefetch", "cpu_broadcast_prefetch")
                and not getattr(self.args, "disable_edge_prefetch", False)
                and not getattr(self.args, "profile_sp_comm", False))

    # ------------------------------------------------------------------ cache / prefetch
    @staticmethod
    def _key(seed: int, state: BudgetState) -> tuple:
        return (int(seed),) + state.key()

    def clear_cache(self) -> None:
        with self._cache_lock:
            self._cache.clear()

    def _store(self, key: tuple, g: AttnGraph) -> None:
        with self._cache_lock:
            if len(self._cache) >= 2:
                self._cache.pop(next(iter(self._cache)))
            self._cache[key] = g

    def uses_device_prefetch(self) -> bool:
        """GPU policies: the next epoch's graph (construction, transposition, backward work list) is built one epoch
        ahead on a side stream, driven by a worker thread, so that the host-side size reads of the build never stall
        the thread that launches the training step."""
        return (self.device.type == "cuda" and self.policy in ("gpu_persist", "gpu_ephemeral") and not self.fanout
                and not self.force_broadcast
                and not getattr(self.args, "disable_edge_prefetch", False)
                and not getattr(self.args, "profile_sp_comm", False))

    def _build_device_ahead(self, seed: int, state: BudgetState):
        if self._gpu_build_ruled_out(state):
            return None                                   # decided and reported by the synchronous path of build()
        try:
            torch.cuda.set_device(self.device)
            if self._build_stream is None:
                self._build_stream = torch.cuda.Stream(self.device)
            with torch.cuda.stream(self._build_stream):
                g = self._finalize(self._build_device(seed, state, who="ahead"))
                g.ensure_transpose()
                done = torch.cuda.Event()
                done.record(self._build_stream)
            return g, done
        except torch.cuda.OutOfMemoryError:
            return None                                   # the step builds synchronously and reports the failure

    def _take_device_prefetch(self, key: tuple) -> Optional[AttnGraph]:
        if self._dev_future is None:
            return None
        fkey, fut = self._dev_future
        self._dev_future = None
        t0 = time.perf_counter()
        res = fut.result()
        self.last_prefetch_wait_s = time.perf_counter() - t0
        if res is None or fkey != key:
            return None
        g, done = res
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(done)
        g.record_stream(cur)                              # allocated on the side stream, consumed on this one
        return g

    def submit_prefetch(self, seed: int, state: BudgetState) -> bool:
        """Start building the next epoch's graph on a worker thread (main_node_fullgraph_sp.py:512-636): on the CPU
        for the offload policies, on a side stream of the GPU for the device policies."""
        if self.uses_device_prefetch():
            key = self._key(seed, state)
            if self._dev_future is not None and self._dev_future[0] == key:
                return True
            self._prepare_sharded(state)
            if self._pool is None:
                self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="bf-edge-prefetch")
            self._dev_future = (key, self._pool.submit(self._build_device_ahead, seed, state))
            return True
        if not self.uses_prefetch():
            return False
        if self.policy == "cpu_broadcast_prefetch" and self.world > 1 and self.rank != 0:
            return False
        key = self._key(seed, state)
        if self._future is not None and self._future[0] == key:
            return True
        if self._pool is None:
            self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="bf-edge-prefetch")
        self._future = (key, self._pool.submit(self._build_host, seed, state))
        return True

    def _wait_prefetch(self, key: tuple) -> Optional[AttnGraph]:
        if self._future is None:
            return None
        fkey, fut = self._future
        t0 = time.perf_counter()
        g = fut.result()
        self.last_prefetch_wait_s = time.perf_counter() - t0
        self._future = None
        self._store(fkey, g)
        return g if fkey == key else None

    def shutdown(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None
        self._future = None
        self._dev_future = None

    # ------------------------------------------------------------------ builds
    def sharded_host_build(self) -> bool:
        """``--shard_cpu_edge_build`` under the rank-local CPU policy: every rank builds only the rows of its own
        queries (1/P of the work, and the ranks of a node stop competing for the same cores) and the shards are
        all-gathered on the training device.  Rows do not depend on one another, so the result is the same graph."""
        return (bool(getattr(self.args, "shard_cpu_edge_build", False)) and self.world > 1
                and self.policy == "cpu_rank_local_prefetch" and not self.force_broadcast
                and self.num_nodes % self.world == 0)

    def _build_host(self, seed: int, state: BudgetState) -> AttnGraph:
        kw = dict(use_real=state.use_real, use_rw=state.use_rw, exphormer=self.exphormer and self.expander_edges is None,
                  fanout=self.fanout, num_threads=self.build_threads)
        walks = int(getattr(self.args, "walks_per_node", 0))
        if self.sharded_host_build():
            per = self.num_nodes // self.world
            rows = (self.rank * per, (self.rank + 1) * per)
            g = build_attn_graph_shard(self.topo_cpu, rows, state.b_real, state.b_rw, walks, state.walk_length, seed, **kw)
            g.shard_rows = rows
        else:
            g = build_attn_graph(self.topo_cpu, state.b_real, state.b_rw, walks, state.walk_length, seed, **kw)
        graph_totals(g)
        if self.device.type == "cuda":
            for name in ("rowptr", "col", "etype"):
                t = getattr(g, name)
                if t is not None and not t.is_pinned():
                    try:
                        setattr(g, name, t.pin_memory())
                    except RuntimeError:
                        pass
        return g

    def _topology_on_device(self) -> Topology:
        if self.topo_gpu is not None:
            return self.topo_gpu
        nbytes = self.topo_cpu.nbytes()
        topo = profile_call("edge_full_h2d", lambda: self.topo_cpu.to(self.device, non_blocking=True),
                            device=self.device, payload_bytes=nbytes)
        if self.policy == "gpu_persist":
            self.topo_gpu = topo
        return topo

    SHARD_CHANNELS = {"step": 3, "ahead": 2}          # barrier channels of the sharded device build, per building thread

    def _device_budgets(self, state: BudgetState):
        walks = int(getattr(self.args, "walks_per_node", 0))
        br = 0 if not state.use_real else state.b_real
        bw = 0 if (not state.use_rw or walks <= 0 or state.walk_length <= 0) else state.b_rw
        return br, bw

    def sharded_device_build(self, state: BudgetState) -> bool:
        """GPU policies on several ranks: each rank selects the rows of its own queries and fetches the others' over
        NVLink (``graph/builder.py::ShardedDeviceBuild``) unless ``--replicate_gpu_edge_build`` asks for local builds."""
        if (self.world <= 1 or self.device.type != "cuda" or self.fanout or self.force_broadcast
                or bool(getattr(self.args, "replicate_gpu_edge_build", False)) or self.policy not in ("gpu_persist", "gpu_ephemeral")):
            return False
        br, bw = self._device_budgets(state)
        if not native_supported(br, bw, state.walk_length):
            return False
        return self.num_nodes % self.world == 0

    def _prepare_sharded(self, state: BudgetState) -> None:
        """Size the shard buffers of both building threads (a collective allocation: main thread only)."""
        if not self.sharded_device_build(state):
            return
        from ..parallel import symm
        br, bw = self._device_budgets(state)
        cap = max(int(br) + int(bw) + (1 if self.exphormer and self.expander_edges is None else 0), 1)
        rows = self.num_nodes // self.world
        for who, channel in self.SHARD_CHANNELS.items():
            sb = self._shard_builds.get(who)
            if sb is None:
                sb = self._shard_builds[who] = ShardedDeviceBuild(symm.get_world(self.group, self.device), channel)
            sb.ensure(rows, cap)

    def _build_device(self, seed: int, state: BudgetState, who: str = "step") -> AttnGraph:
        walks = int(getattr(self.args, "walks_per_node", 0))
        br, bw = self._device_budgets(state)
        if self.fanout or not native_supported(br, bw, state.walk_length):
            # fan-out sampling, sides without budget and budgets beyond the fixed-width kernels are built by the general
            # C++ builder from the host copy of the topology (no topology transfer in either direction)
            return self._upload(self._build_host(seed, state))
        topo = self._topology_on_device()
        typed = self.exphormer and self.expander_edges is None
        sb = self._shard_builds.get(who)
        if sb is not None and self.sharded_device_build(state):
            cap = max(int(br) + int(bw) + (1 if typed else 0), 1)
            if sb.ready(self.num_nodes // self.world, cap):
                return sb.build(topo, br, bw, walks, state.walk_length, seed, typed)
        return build_attn_graph(topo, state.b_real, state.b_rw, int(getattr(self.args, "walks_per_node", 0)),
                                state.walk_length, seed, use_real=state.use_real, use_rw=state.use_rw,
                                exphormer=self.exphormer and self.expander_edges is None)

    def _upload(self, g: AttnGraph) -> AttnGraph:
        if self.device.type != "cuda":
            return g
        if self._copy_stream is not None:
            cur = torch.cuda.current_stream(self.device)
            with torch.cuda.stream(self._copy_stream):
                out = g.to(self.device, non_blocking=True)
            cur.wait_stream(self._copy_stream)
            for t in (out.rowptr, out.col, out.etype):
                if t is not None:
                    t.record_stream(cur)
            return out
        return g.to(self.device)

    def _broadcast(self, g: Optional[AttnGraph]) -> AttnGraph:
        """Source rank ships (sizes, rowptr, col[, etype]) to the others (utils/fullgraph_sp_support.py:3318-3332)."""
        nccl = dist.get_backend(self.group) == "nccl"
        dev = self.device if nccl else torch.device("cpu")
        is_src = self.rank == 0
        meta = torch.zeros(4, dtype=torch.int64, device=dev)
        if is_src:
            meta = torch.tensor([g.num_rows, g.num_edges, 1 if g.etype is not None else 0,
                                 -1 if g.max_degree is None else g.max_degree], dtype=torch.int64, device=dev)
        dist.broadcast(meta, src=self.src_rank, group=self.group)
        n_rows, n_edges, has_type, maxdeg = (int(v) for v in meta.tolist())
        def _bc(t, shape, dtype):
            buf = t.to(dev) if is_src else torch.empty(shape, dtype=dtype, device=dev)
            dist.broadcast(buf, src=self.src_rank, group=self.group)
            return buf
        rowptr = _bc(g.rowptr if is_src else None, (n_rows + 1,), torch.int32)
        col = _bc(g.col if is_src else None, (n_edges,), torch.int32)
        etype = _bc(g.etype if is_src else None, (n_edges,), torch.uint8) if has_type else None
        return AttnGraph(n_rows, rowptr, col, etype, max_degree=None if maxdeg < 0 else maxdeg)

    def _gather_shards(self, shard: AttnGraph) -> AttnGraph:
        """All ranks hold the rows of their own queries; concatenate them in rank order on the collective's device
        (sizes first, then row offsets, keys and types padded to the longest shard)."""
        nccl = dist.get_backend(self.group) == "nccl"
        dev = self.device if nccl else torch.device("cpu")
        local = self._upload(shard) if dev.type == "cuda" else shard
        p = self.world
        sizes = torch.tensor([local.num_edges, max(local.n_real, 0), max(local.n_rw, 0),
                              -1 if local.max_degree is None else local.max_degree], dtype=torch.int64, device=dev)
        all_sizes = [torch.empty_like(sizes) for _ in range(p)]
        dist.all_gather(all_sizes, sizes, group=self.group)
        all_sizes = torch.stack(all_sizes).cpu()
        edges = [int(v) for v in all_sizes[:, 0].tolist()]
        longest = max(max(edges), 1)

        def gather(t: torch.Tensor, length: int) -> list:
            buf = torch.zeros(length, dtype=t.dtype, device=dev)
            buf[: t.numel()] = t.to(dev)
            out = [torch.empty_like(buf) for _ in range(p)]
            dist.all_gather(out, buf, group=self.group)
            return out

        rowptrs = gather(local.rowptr, local.num_rows + 1)
        cols = gather(local.col, longest)
        types = gather(local.etype, longest) if local.etype is not None else None
        offsets, total = [], 0
        for e in edges:
            offsets.append(total)
            total += e
        rowptr = torch.cat([rp[:-1] + off for rp, off in zip(rowptrs, offsets)]
                           + [torch.tensor([total], dtype=torch.int32, device=dev)]).to(torch.int32)
        col = torch.cat([c[:e] for c, e in zip(cols, edges)])
        etype = torch.cat([t[:e] for t, e in zip(types, edges)]) if types is not None else None
        degs = all_sizes[:, 3]
        g = AttnGraph(self.num_nodes, rowptr, col, etype, n_real=int(all_sizes[:, 1].sum()), n_rw=int(all_sizes[:, 2].sum()),
                      max_degree=None if bool((degs < 0).any()) else int(degs.max()))
        return g if g.device == self.device else self._upload(g)

    def _finalize(self, g: AttnGraph) -> AttnGraph:
        """Model-specific assembly on the final device."""
        if self.exphormer and self.expander_edges is not None:
            # sampled + self loops are type 0, expander edges type 1 (main_node_fullgraph_sp.py:1170-1185)
            ei = g.edge_index()[:2]
            self_ids = torch.arange(self.num_nodes, device=ei.device)
            exp = self.expander_edges.to(ei.device)
            allei = torch.cat([ei, torch.stack([self_ids, self_ids]), exp], dim=1)
            typ = torch.cat([torch.zeros(ei.size(1) + self.num_nodes, dtype=torch.long, device=ei.device),
                             torch.ones(exp.size(1), dtype=torch.long, device=ei.device)])
            g = AttnGraph.from_edge_index(torch.cat([allei, typ.unsqueeze(0)], 0), self.num_nodes)
        if self.virtual_node:
            g = add_virtual_node(g, self.num_nodes, self.nodes_per_rank)
        return g

    def build(self, seed: int, state: BudgetState, record: bool = True) -> AttnGraph:
        """The epoch's attention graph on the training device (utils/fullgraph_sp_support.py:3171-3362)."""
        t0 = time.perf_counter()
        self.last_prefetch_wait_s = 0.0
        key = self._key(seed, state)
        self._prepare_sharded(state)
        broadcast = self.world > 1 and (self.force_broadcast or self.policy in ("cpu_broadcast", "cpu_broadcast_prefetch"))
        g: Optional[AttnGraph] = None
        ahead = self._take_device_prefetch(key)
        if ahead is not None:
            self.last_build_s = time.perf_counter() - t0
            self.last_graph_bytes = ahead.nbytes()
            if record:
                record_scalar("edge_merged_edges", ahead.num_edges, reduce="max")
            return ahead
        with self._cache_lock:
            host = self._cache.get(key)
        if host is None and self._future is not None:
            host = self._wait_prefetch(key)
        if broadcast:
            if self.rank == 0 and host is None:
                host = profile_call("edge_build_local", lambda: self._build_host(seed, state), device="cpu")
                self._store(key, host)
            g = profile_call("edge_broadcast", lambda: self._broadcast(host), device=self.device)
            if g.device != self.device:
                g = self._upload(g)
        elif self.policy in _CPU_POLICIES or self.device.type != "cuda":
            if host is None or (getattr(host, "shard_rows", None) is not None) != self.sharded_host_build():
                host = profile_call("edge_build_local", lambda: self._build_host(seed, state), device="cpu")
                self._store(key, host)
            if getattr(host, "shard_rows", None) is not None:
                g = profile_call("edge_shard_gather", lambda: self._gather_shards(host), device=self.device)
            else:
                g = self._upload(host)
        elif self._gpu_build_ruled_out(state):
            # proactive CPU build: the estimate does not fit under the registered memory cap, or the GPU build already
            # failed in this run; the caller reports it to the planner like a run-time failure
            self.gpu_build_failed = True
            self.topo_gpu = None
            g = self._upload(profile_call("edge_build_local", lambda: self._build_host(seed, state), device="cpu"))
        else:
            try:
                g = profile_call("edge_build_local", lambda: self._build_device(seed, state), device=self.device)
            except torch.cuda.OutOfMemoryError:
                # sticky CPU fallback, reported to the planner by the caller (utils/fullgraph_sp_support.py:1334-1491)
                self.gpu_build_failed = True
                self.topo_gpu = None
                BUDGET.mark_infeasible(self.device, self.topo_cpu.num_edges)
                torch.cuda.empty_cache()
                host = self._build_host(seed, state)
                g = self._upload(host)
        g = profile_call("edge_merge", lambda: self._finalize(g), device=self.device)
        self.last_build_s = time.perf_counter() - t0
        self.last_graph_bytes = g.nbytes()
        if record:
            record_scalar("edge_merged_edges", g.num_edges, reduce="max")
        return g

    def _gpu_build_ruled_out(self, state: BudgetState) -> bool:
        """Checked only when a per-process memory cap is registered or a GPU build failed before: without either the
        build is simply tried (its out-of-memory error is caught), so the common path makes no driver query."""
        if self.device.type != "cuda" or (BUDGET.cap_bytes <= 0 and not BUDGET.any_infeasible()):
            return False
        dev = BUDGET.safe_build_device(self.device, self.estimate_working_set_bytes(state), self.topo_cpu.num_edges,
                                       log=print if self.rank == 0 else None)
        return dev.type != "cuda"

    def estimate_working_set_bytes(self, state: BudgetState) -> int:
        """First-principles GPU footprint of one device build: topology + fixed-width rows + CSR
        (the analogue of ``_estimate_rw_working_set_bytes``, gt_sp/utils.py:160-236, for this builder)."""
        cap = (state.b_real or 0) + (state.b_rw or 0) + 1
        topo = self.topo_cpu.nbytes()
        rows = self.num_nodes * cap * 5 + self.num_nodes * 12
        return int(topo + 2 * rows)
