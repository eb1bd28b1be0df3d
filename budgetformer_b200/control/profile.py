"""Edge-policy profiling for the execution planner.

Each placement policy is built twice with bumped seeds (cold, then warm) and the warm build is
recorded as ``prep/serial/overlap`` seconds, GPU peak, CPU delta and resident bytes, MAX-reduced
over ranks; policies that are provably dominated on one node are skipped
(``_profile_multi_tier_edge_policy``, utils/fullgraph_sp_runtime.py:251-546 and
main_node_fullgraph_sp.py:665-988).  With the counter-based builders the GPU policies cost
milliseconds, so on an uncapped B200 the planner normally lands on ``gpu_persist``; under a tight
``--multi_tier_gpu_memory_limit_mib`` the resident topology no longer fits and a CPU policy wins."""
from __future__ import annotations

import time

import torch

from ..parallel import comm
from ..utils.misc import process_rss_mib


def _measure(trainer, policy: str, seed: int):
    eng = trainer.edge_engine
    dev = trainer.device
    state = trainer.budget_state()
    old_policy, old_lock, old_topo = eng.policy, eng.policy_locked, eng.topo_gpu
    eng.set_policy(policy)
    rss0 = process_rss_mib()
    res = None
    try:
        for rep in range(2):                       # cold, then warm
            eng.clear_cache()
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
                torch.cuda.reset_peak_memory_stats(dev)
            t0 = time.perf_counter()
            g = eng.build(seed + rep, state, record=False)
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            dt = time.perf_counter() - t0
            peak = torch.cuda.max_memory_allocated(dev) if dev.type == "cuda" else 0
            live = eng.topo_gpu.nbytes() if eng.topo_gpu is not None else 0
            res = (dt, peak, max(0.0, process_rss_mib() - rss0) * 2 ** 20, live, g.nbytes())
            del g
        ok = not eng.gpu_build_failed
    except torch.cuda.OutOfMemoryError:
        ok = False
    eng.gpu_build_failed = False
    eng.topo_gpu = old_topo if old_policy == "gpu_persist" else None
    eng.policy, eng.policy_locked = old_policy, old_lock
    eng.clear_cache()
    return ok, res


def profile_edge_policies(trainer) -> None:
    planner = trainer.planner
    dev = trainer.device
    cdev = comm.comm_device(trainer.sp_group, dev)
    base_seed = int(trainer.args.seed) + 900_000
    policies = ["cpu_rank_local_prefetch"]
    if dev.type == "cuda":
        policies = ["gpu_persist", "gpu_ephemeral", "cpu_rank_local_prefetch"]
    if trainer.sp_world > 1:
        policies.append("cpu_broadcast_prefetch")
    state = trainer.budget_state()
    for i, policy in enumerate(policies):
        ok, res = _measure(trainer, policy, base_seed + 10 * i)
        ok_all = comm.all_reduce_scalar(1.0 if ok else 0.0, "min", trainer.sp_group, cdev) > 0.5
        if not ok_all or res is None:
            planner.set_edge_policy_profile(policy, 0, 0, 0, enabled=False)
            trainer.log(f"[MultiTierManager] edge policy {policy}: infeasible on some rank, excluded")
            continue
        dt, peak, cpu_delta, live, gbytes = comm.all_reduce_scalars(list(res), "max", trainer.sp_group, cdev)
        prefetch = policy.endswith("_prefetch") and not getattr(trainer.args, "disable_edge_prefetch", False)
        # a prefetched build overlaps the model step; only the upload is serial
        serial = 0.0 if prefetch else dt
        overlap = dt if prefetch else 0.0
        planner.set_edge_policy_profile(
            policy, prep_time_s=dt, gpu_peak_bytes=int(peak), cpu_delta_bytes=int(cpu_delta),
            live_edge_bytes=int(live), serial_time_s=serial, overlap_time_s=overlap,
            rw_gpu_extra_bytes=trainer.edge_engine.estimate_working_set_bytes(state) if policy == "gpu_persist" else 0)
        trainer.log(f"[MultiTierManager] edge policy {policy}: build={dt * 1e3:.1f} ms gpu_peak={peak / 2 ** 20:.0f} MiB "
                    f"resident={live / 2 ** 20:.0f} MiB cpu_delta={cpu_delta / 2 ** 20:.0f} MiB")
    planner.set_edge_info(trainer.edge_engine.topo_cpu.nbytes(), 0.0)
