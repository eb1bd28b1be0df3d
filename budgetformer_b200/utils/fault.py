"""Host-side fault injection for recovery tests.

A spec is a comma-separated list of ``<kind>@<phase>:<epoch>[:rank<k>]`` items, e.g.
``oom@fwd:3`` (raise an out-of-memory error in the forward of epoch 3 on every rank),
``oom@bwd:4:rank1``, ``raise@edge:2``, ``exit@step:7:rank1``, ``delay@step:5:rank0``, ``stall@step:3:rank1``
(the rank stops making progress without announcing it: sleeps until it is killed).
Faults are raised by the Python process at phase boundaries, never by a kernel: no GPU is
faulted, trapped or hung.  ``InjectedOOM`` derives from ``torch.cuda.OutOfMemoryError`` where that class can
be subclassed so that the regular recovery path handles it."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import List, Optional

import torch

try:
    class InjectedOOM(torch.cuda.OutOfMemoryError):  # type: ignore[misc]
        pass
except Exception:  # pragma: no cover
    class InjectedOOM(RuntimeError):  # type: ignore[no-redef]
        pass


class InjectedFailure(RuntimeError):
    pass


@dataclass
class _Fault:
    kind: str
    phase: str
    epoch: int
    rank: Optional[int]
    fired: bool = False


class FaultInjector:
    def __init__(self, spec: str = "", rank: int = 0):
        self.rank = int(rank)
        self.on_exit = None                       # optional callable run before an injected exit (orderly departure)
        self.faults: List[_Fault] = []
        spec = spec or os.environ.get("BF_FAULT", "")
        for item in filter(None, (s.strip() for s in spec.split(","))):
            self.faults.append(self._parse(item))

    GRAMMAR = "<kind>@<phase>:<epoch>[:rank<k>] with kind in oom|raise|exit|delay|stall, e.g. exit@step:7:rank1"

    @classmethod
    def _parse(cls, item: str) -> _Fault:
        try:
            kind, rest = item.split("@", 1)
            parts = rest.split(":")
            phase, epoch = parts[0], int(parts[1])
            rk = None
            if len(parts) > 2:
                if not parts[2].startswith("rank") or len(parts) > 3:
                    raise ValueError(parts[2])
                rk = int(parts[2][4:])
            if kind not in ("oom", "raise", "exit", "delay", "stall") or not phase:
                raise ValueError(kind)
        except (ValueError, IndexError) as e:
            raise ValueError(f"malformed fault spec {item!r}: expected {cls.GRAMMAR}") from e
        return _Fault(kind, phase, epoch, rk)

    def __bool__(self) -> bool:
        return bool(self.faults)

    def check(self, phase: str, epoch: int) -> None:
        for f in self.faults:
            if f.fired or f.phase != phase or f.epoch != epoch or (f.rank is not None and f.rank != self.rank):
                continue
            f.fired = True
            if f.kind == "oom":
                raise InjectedOOM(f"injected out-of-memory at {phase} epoch {epoch} rank {self.rank}")
            if f.kind == "raise":
                raise InjectedFailure(f"injected failure at {phase} epoch {epoch} rank {self.rank}")
            if f.kind == "delay":
                time.sleep(1.0)
            if f.kind == "stall":
                time.sleep(float(os.environ.get("BF_FAULT_STALL_SECONDS", "3600")))
            if f.kind == "exit":
                if self.on_exit is not None:
                    self.on_exit()
                os._exit(int(os.environ.get("BF_FAULT_EXIT_CODE", "17")))
