"""Small runtime helpers: seeding, AMP resolution, RSS readers, device-timed blocks."""
from __future__ import annotations

import contextlib
import os
import random
import resource
import time
from typing import Optional

import numpy as np
import torch


def set_seed(seed: int) -> None:
    """Seed python / numpy / torch (all devices) identically on every rank (utils/fullgraph_sp_support.py:446-451)."""
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def resolve_amp_dtype(name: str, device) -> Optional[torch.dtype]:
    """``none|bf16|fp16`` -> dtype; bf16 falls back to fp16 on GPUs without bf16 (utils/fullgraph_sp_support.py:354-359)."""
    name = str(name or "none").lower()
    if name == "none":
        return None
    dev = torch.device(device)
    if name == "bf16":
        if dev.type == "cuda" and not torch.cuda.is_bf16_supported():
            return torch.float16
        return torch.bfloat16
    if name == "fp16":
        return torch.float16 if dev.type == "cuda" else torch.bfloat16
    raise ValueError(f"unknown amp dtype {name!r}")


def autocast_context(device, amp_dtype: Optional[torch.dtype]):
    if amp_dtype is None:
        return contextlib.nullcontext()
    return torch.autocast(device_type=torch.device(device).type, dtype=amp_dtype)


def process_rss_mib() -> float:
    try:
        with open("/proc/self/statm") as fh:
            return int(fh.read().split()[1]) * os.sysconf("SC_PAGE_SIZE") / 2 ** 20
    except Exception:
        return 0.0


def process_peak_rss_mib() -> float:
    return resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024.0


def glibc_malloc_trim() -> bool:
    """Return freed heap pages to the OS after large CPU-side builds (utils/fullgraph_sp_support.py:3122-3139)."""
    try:
        import ctypes
        return bool(ctypes.CDLL("libc.so.6").malloc_trim(0))
    except Exception:
        return False


class StepTimer:
    """Host timer with optional device synchronisation on both sides (utils/fullgraph_sp_runtime.py:157-164)."""

    def __init__(self, device, sync: bool):
        self.device, self.sync = torch.device(device), bool(sync) and torch.device(device).type == "cuda"
        self.elapsed = 0.0

    def __enter__(self):
        if self.sync:
            torch.cuda.synchronize(self.device)
        self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.sync:
            torch.cuda.synchronize(self.device)
        self.elapsed = time.perf_counter() - self._t0
        return False


def clone_model_state_to_cpu(model) -> dict:
    """Detached CPU copy of every entry of ``model.state_dict()`` (a snapshot that later training does not touch)."""
    return {name: t.detach().cpu().clone() for name, t in model.state_dict().items()}


@contextlib.contextmanager
def dropout_disabled(model):
    """Every ``nn.Dropout`` of ``model`` in eval mode inside the block, its previous mode restored afterwards
    (``_set_dropout_eval`` / ``_restore_dropout``, utils/fullgraph_sp_support.py:3365-3376); BatchNorm and the rest of
    the model keep their mode."""
    saved = [(m, m.training) for m in model.modules() if isinstance(m, torch.nn.Dropout)]
    for m, _ in saved:
        m.eval()
    try:
        yield
    finally:
        for m, mode in saved:
            m.train(mode)
