"""Checkpointing.

The model file keeps the reference's name and key layout — rank 0 writes
``<model_dir>/<dataset>_fg_sp.pkl`` = ``torch.save(model.state_dict())`` whenever validation
improves (main_node_fullgraph_sp.py:1859-1865).  The reference has no resume path; here a sidecar
``<dataset>_fg_sp.train_state.pt`` additionally stores optimizer, scheduler, scaler, epoch, budget
controller, planner plan, RNG state and best metrics, and ``--resume`` restores them.  Since weights
are replicated, rank 0 writes and every rank loads, checking a checksum of the weights."""
from __future__ import annotations

import hashlib
import os
from typing import Dict

import torch

_CORE_PREFIX = "dist_attn.local_attn."


def model_path(args) -> str:
    return os.path.join(args.model_dir, f"{args.dataset}_fg_sp.pkl")


def train_state_path(args) -> str:
    return os.path.join(args.model_dir, f"{args.dataset}_fg_sp.train_state.pt")


def normalize_state_dict_keys(sd: Dict[str, torch.Tensor], model: torch.nn.Module) -> Dict[str, torch.Tensor]:
    """Accept both key forms: single-process reference runs store the core attention at ``...dist_attn.X``,
    SP runs at ``...dist_attn.local_attn.X``.  This framework always emits the SP form."""
    want = set(model.state_dict().keys())
    out = {}
    for k, v in sd.items():
        if k in want:
            out[k] = v
            continue
        alt = k.replace("dist_attn.", _CORE_PREFIX) if (_CORE_PREFIX not in k and "dist_attn." in k) else k
        out[alt if alt in want else k] = v
    return out


def weights_checksum(model: torch.nn.Module) -> str:
    h = hashlib.sha256()
    for k, v in sorted(model.state_dict().items()):
        h.update(k.encode())
        h.update(v.detach().to("cpu", torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def save_best_model(trainer) -> str:
    os.makedirs(trainer.args.model_dir, exist_ok=True)
    path = model_path(trainer.args)
    if trainer.rank == 0:
        torch.save({k: v.detach().cpu() for k, v in trainer.model.state_dict().items()}, path)
    return path


def save_train_state(trainer) -> str:
    path = train_state_path(trainer.args)
    if trainer.rank != 0:
        return path
    os.makedirs(trainer.args.model_dir, exist_ok=True)
    planner = trainer.planner
    state = {
        "epoch": trainer.epoch,
        "model": {k: v.detach().cpu() for k, v in trainer.model.state_dict().items()},
        "checksum": weights_checksum(trainer.model),
        "optimizer": trainer.optimizer.state_dict(),
        "lr_scheduler": trainer.lr_scheduler.state_dict(),
        "scaler": trainer.scaler.state_dict(),
        "controller": trainer.controller.state_dict(),
        "planner": None if planner is None or not planner.is_active() else {
            "edge_policy": planner.edge_policy, "modes": planner.modes()},
        "best": dict(trainer.best),
        "loss_ema": trainer.loss_ema,
        "rng": {"torch": torch.get_rng_state(),
                "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None},
    }
    tmp = path + ".tmp"
    torch.save(state, tmp)
    os.replace(tmp, path)
    return path


def load_train_state(trainer, path: str) -> None:
    state = torch.load(path, map_location="cpu", weights_only=False)
    sd = normalize_state_dict_keys(state["model"], trainer.model)
    trainer.model.load_state_dict(sd)
    if state.get("checksum") and weights_checksum(trainer.model) != state["checksum"]:
        raise RuntimeError(f"weights restored from {path} do not match their recorded checksum")
    trainer.optimizer.load_state_dict(state["optimizer"])
    trainer.lr_scheduler.load_state_dict(state["lr_scheduler"])
    if state.get("scaler"):
        trainer.scaler.load_state_dict(state["scaler"])
    trainer.controller.load_state_dict(state["controller"])
    trainer.best = dict(state.get("best", trainer.best))
    trainer.loss_ema = state.get("loss_ema")
    trainer.epoch = int(state["epoch"])
    trainer._budget_frozen_notified = bool(trainer.controller.frozen)
    plan = state.get("planner")
    if plan and trainer.planner is not None:
        trainer.planner.override_active_plan(plan["edge_policy"], plan["modes"])
        trainer.edge_engine.set_policy(plan["edge_policy"], lock=True)
        trainer._plan_applied = True
    rng = state.get("rng") or {}
    if rng.get("torch") is not None:
        torch.set_rng_state(rng["torch"])
    if rng.get("cuda") is not None and torch.cuda.is_available() and len(rng["cuda"]) == torch.cuda.device_count():
        torch.cuda.set_rng_state_all(rng["cuda"])
    # gradient buckets were re-pointed by load_state_dict of nothing; parameters keep their .grad views
    trainer.log(f"[resume] restored epoch {trainer.epoch} from {path}")
