"""Process-group bootstrap and the sequence-parallel (SP) group registry.

Same public surface as the reference's ``gt_sp/initialize.py`` (``initialize_distributed``
:24-91, ``initialize_sequence_parallel`` :94-134, the getters :137-172 and the Graphormer
global-token registry :189-227) with two differences: multi-process runs work on a CPU-only
machine (gloo), and state lives in one ``_State`` object instead of loose module globals.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class _State:
    group: Optional[object] = None
    world_size: int = 1
    rank: int = 0
    src_rank: int = 0
    seq_len: int = 0
    initialized: bool = False
    global_token_indices: Optional[List[int]] = None
    last_batch_global_token_indices: Optional[List[int]] = None
    last_batch_flag: bool = False
    owns_process_group: bool = False


_STATE = _State()


def initialize_distributed(args) -> None:
    """Set ``args.rank / world_size / local_rank / device`` and create the process group.

    Single-process fallback when ``RANK``/``WORLD_SIZE`` are absent or the world is 1
    (reference :32-51).  With more ranks: NCCL binds rank -> GPU ``rank % device_count``; gloo needs
    no GPU.  The SP group always spans the whole world (reference :88-91)."""
    rank = int(os.getenv("RANK", getattr(args, "rank", None) or 0))
    world = int(os.getenv("WORLD_SIZE", getattr(args, "world_size", None) or 1))
    args.rank, args.world_size = rank, world
    backend = getattr(args, "distributed_backend", "nccl")
    n_gpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    want_cpu = str(getattr(args, "device", "") or "").startswith("cpu") or backend == "gloo" and n_gpu == 0
    if world <= 1:
        args.sequence_parallel_size = 1
        args.local_rank = 0
        if n_gpu > 0 and not want_cpu:
            args.device = f"cuda:{int(os.getenv('LOCAL_RANK', 0)) % n_gpu}"
            torch.cuda.set_device(args.device)
        else:
            args.device = "cpu"
        initialize_sequence_parallel(getattr(args, "seq_len", 0), 1, 1, 1)
        return
    if backend == "nccl":
        if n_gpu == 0:
            raise RuntimeError("distributed backend 'nccl' needs GPUs; use --distributed-backend gloo on CPU")
        local = int(os.getenv("LOCAL_RANK", rank % n_gpu))
        args.local_rank = local
        args.device = f"cuda:{local % n_gpu}"
        torch.cuda.set_device(args.device)
    else:
        args.local_rank = int(os.getenv("LOCAL_RANK", rank))
        if n_gpu > 0 and not want_cpu:
            args.device = f"cuda:{args.local_rank % n_gpu}"
            torch.cuda.set_device(args.device)
        else:
            args.device = "cpu"
    timeout = datetime.timedelta(minutes=int(getattr(args, "distributed_timeout_minutes", 10)))
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device(args.device)
        dist.init_process_group(backend=backend, world_size=world, rank=rank, timeout=timeout, **kwargs)
        _STATE.owns_process_group = True
    args.sequence_parallel_size = world
    initialize_sequence_parallel(getattr(args, "seq_len", 0), 1, 1, world)
    if backend == "nccl" and os.getenv("BF_HOST_CONTROL_PLANE", "1") != "0":
        _create_control_group(timeout)


def _create_control_group(timeout) -> None:
    """Host-side (gloo) twin of the SP group for control scalars.  The reference sends every vote through NCCL and
    reads it with ``.item()`` (e.g. main_node_fullgraph_sp.py:1313-1318), which empties the GPU queue each time; with
    the twin the training stream is never synchronised by the control plane.  Creation is collective; when gloo cannot
    come up on this host every rank sees the same failure and the votes stay on NCCL."""
    from . import comm
    if _STATE.group is None or comm.control_group(_STATE.group) is not None:
        return
    try:
        if os.environ.get("MASTER_ADDR", "") in ("127.0.0.1", "localhost"):
            os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
        kw = {"timeout": timeout} if timeout is not None else {}
        twin = dist.new_group(backend="gloo", **kw)
        probe = torch.zeros(1)
        dist.all_reduce(probe, group=twin)
        comm.register_control_group(_STATE.group, twin)
    except Exception as e:  # pragma: no cover - depends on the host's network setup
        if dist.get_rank() == 0:
            print(f"[init] host-side control group unavailable ({type(e).__name__}: {e}); votes use the device group",
                  flush=True)


def initialize_sequence_parallel(seq_len: int = 0, tensor_model_parallel_size: int = 1,
                                 pipeline_model_parallel_size: int = 1, sequence_parallel_size: int = 1) -> None:
    """Create contiguous-rank SP groups of ``sequence_parallel_size`` (tensor/pipeline sizes are accepted
    and ignored, as in the reference :96-97)."""
    sp = int(sequence_parallel_size)
    _STATE.seq_len = int(seq_len or 0)
    if not dist.is_initialized() or dist.get_world_size() == 1 or sp <= 1:
        _STATE.group, _STATE.world_size, _STATE.rank, _STATE.src_rank = None, 1, 0, 0
        _STATE.initialized = True
        return
    world = dist.get_world_size()
    rank = dist.get_rank()
    if world % sp != 0:
        raise ValueError(f"world size {world} is not divisible by sequence_parallel_size {sp}")
    for g in range(world // sp):
        ranks = list(range(g * sp, (g + 1) * sp))
        grp = dist.group.WORLD if (sp == world) else dist.new_group(ranks)
        if rank in ranks:
            _STATE.group = grp
            _STATE.world_size = sp
            _STATE.rank = rank - g * sp
            _STATE.src_rank = g * sp
    _STATE.initialized = True


def destroy_distributed() -> None:
    if dist.is_initialized():
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()
    reset_state()


def reset_state() -> None:
    global _STATE
    from . import comm
    comm._CONTROL_TWIN.clear()
    _STATE.__init__()


def sequence_parallel_is_initialized() -> bool:
    return _STATE.initialized and _STATE.world_size > 1


def get_sequence_parallel_group():
    return _STATE.group


def get_sequence_parallel_world_size() -> int:
    return _STATE.world_size


def get_sequence_parallel_rank() -> int:
    return _STATE.rank


def get_sequence_parallel_src_rank() -> int:
    return _STATE.src_rank


def get_sequence_length() -> int:
    return _STATE.seq_len


# ---- Graphormer global-token registry (reference :189-227) ---------------------------------------
def set_global_token_indices(indices) -> None:
    _STATE.global_token_indices = list(indices) if indices is not None else None


def get_global_token_indices(last_batch: bool = False):
    if last_batch and _STATE.last_batch_global_token_indices is not None:
        return _STATE.last_batch_global_token_indices
    return _STATE.global_token_indices


def set_last_batch_global_token_indices(indices) -> None:
    _STATE.last_batch_global_token_indices = list(indices) if indices is not None else None


def last_batch_flag(flag: bool) -> None:
    _STATE.last_batch_flag = bool(flag)


def get_last_batch_flag() -> bool:
    return _STATE.last_batch_flag
