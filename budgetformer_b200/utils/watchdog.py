"""Host-side heartbeat watchdog: a lost or stalled rank becomes a clean, symmetric abort instead of a hang.

The reference relies on the NCCL timeout alone (``--distributed-timeout-minutes``, gt_sp/initialize.py:82-85).  Here
every rank posts a heartbeat to the job's key-value store at each step boundary and a daemon thread watches the peers:

* ``beat(step)``   called by the training loop between steps (no kernels or collectives of the step in flight yet);
* ``check()``      called right after ``beat``: a host-side rendezvous that returns once every peer has posted the same
                   step, and raises ``PeerLost`` when a peer announced that it left, when the abort flag is set, or
                   when a peer stays behind for ``deadline_s`` - i.e. the survivors learn of the loss on the host,
                   *before* their next launch;
* the thread       covers the case where this rank is already blocked inside a collective: when a peer stays silent
                   for ``deadline_s`` it sets the abort flag (so every other rank aborts too) and ends this process
                   with exit code ``EXIT_CODE`` after printing which rank was lost.  With ``step_deadline_s > 0`` it
                   also ends the job when this rank itself has not reached a step boundary for that long (a
                   collective or a kernel that exceeded its deadline while every rank sits in the same step).

Nothing here touches a GPU; the failure modes are exercised with gloo ranks on the CPU.
"""
from __future__ import annotations

import os
import sys
import threading
import time
from typing import Optional

EXIT_CODE = 75


class PeerLost(RuntimeError):
    """Raised on the surviving ranks between steps."""


class StepWatchdog:
    def __init__(self, store, rank: int, world: int, deadline_s: float = 120.0, poll_s: float = 0.5,
                 hard_exit: bool = True, startup_grace_s: float = 120.0, step_deadline_s: float = 0.0):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.deadline_s, self.poll_s, self.hard_exit = float(deadline_s), float(poll_s), bool(hard_exit)
        self.startup_grace_s = max(float(startup_grace_s), self.deadline_s)   # ranks reach their first step unevenly
        self.step_deadline_s = max(0.0, float(step_deadline_s))
        self._beats = 0
        self._beat_time = time.monotonic()
        self._step = -1
        self._last_seen = {r: (-1, time.monotonic()) for r in range(self.world)}
        self._stop = threading.Event()
        self._armed = False                       # peers are only timed once this rank has posted its first heartbeat
        self._lost: Optional[str] = None
        self._thread = threading.Thread(target=self._watch, name="bf-watchdog", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ API of the training loop
    def beat(self, step: int) -> None:
        self._step = int(step)
        self.store.set(f"hb/{self.rank}", str(self._step))
        self._beat_time = time.monotonic()
        self._beats += 1
        self._armed = True

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly departure (call between steps, then exit)."""
        self.store.set(f"left/{self.rank}", reason)
        self.stop()

    def check(self) -> None:
        """Step-boundary rendezvous on the host: wait until every peer has posted a heartbeat for this step (or a later
        one); a peer that announced its departure, an abort request or ``deadline_s`` of silence raises ``PeerLost``.
        Every rank reaches the same verdict here, before any kernel or collective of the step is launched."""
        t0 = time.monotonic()
        limit = self.deadline_s if self._beats > 1 else self.startup_grace_s
        while True:
            self._poll_once()
            if self._lost is not None:
                raise PeerLost(self._lost)
            behind = [r for r in range(self.world) if r != self.rank and self._last_seen[r][0] < self._step]
            if not behind:
                return
            if time.monotonic() - t0 > limit:
                self._lost = f"rank {behind[0]} did not reach step {self._step} within {limit:.0f} s"
                try:
                    self.store.set("abort", self._lost)
                except Exception:
                    pass
                raise PeerLost(self._lost)
            time.sleep(0.005)

    def stop(self) -> None:
        self._stop.set()

    # ------------------------------------------------------------------ internals
    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def _poll_once(self) -> None:
        now = time.monotonic()
        flag = self._get("abort")
        if flag is not None and self._lost is None:
            self._lost = f"abort requested: {flag}"
        for r in range(self.world):
            if r == self.rank:
                continue
            gone = self._get(f"left/{r}")
            if gone is not None and self._lost is None:
                self._lost = f"rank {r} left the job ({gone})"
            hb = self._get(f"hb/{r}")
            step = int(hb) if hb is not None else -1
            last_step, last_t = self._last_seen[r]
            if step != last_step:
                self._last_seen[r] = (step, now)
            elif (self._armed and step < self._step and self._lost is None
                  and now - last_t > (self.deadline_s if step >= 0 else self.startup_grace_s)):
                self._lost = f"rank {r} has been silent for {now - last_t:.1f} s at step {step} (this rank is at {self._step})"

    def _watch(self) -> None:
        waited_since: Optional[float] = None
        while not self._stop.wait(self.poll_s):
            try:
                self._poll_once()
            except Exception:
                continue
            if (self._lost is None and self._armed and self.step_deadline_s > 0
                    and time.monotonic() - self._beat_time > self.step_deadline_s):
                self._lost = (f"rank {self.rank} has not reached a step boundary for "
                              f"{time.monotonic() - self._beat_time:.0f} s (step {self._step}): a collective or a "
                              f"kernel exceeded its deadline")
            if self._lost is None:
                waited_since = None
                continue
            # give the main thread one deadline to notice at its next check(); if it is stuck in a collective, end the job
            if waited_since is None:
                waited_since = time.monotonic()
                # said at once: a launcher that notices the dead rank first may end this process before the grace is over
                print(f"[watchdog] rank {self.rank}: {self._lost}", file=sys.stderr, flush=True)
                try:
                    self.store.set("abort", self._lost)
                except Exception:
                    pass
            elif self.hard_exit and time.monotonic() - waited_since > min(self.deadline_s, 10.0):
                print(f"[watchdog] rank {self.rank}: {self._lost}; aborting", file=sys.stderr, flush=True)
                os._exit(EXIT_CODE)


def build_watchdog(args, rank: int, world: int):
    """``--watchdog_seconds S`` (> 0) on a multi-rank job: a watchdog on the default process group's store."""
    secs = float(getattr(args, "watchdog_seconds", 0) or 0)
    if secs <= 0 or world <= 1:
        return None
    import torch.distributed as dist
    from torch.distributed.distributed_c10d import _get_default_store
    store = dist.PrefixStore("bf_watchdog", _get_default_store())
    return StepWatchdog(store, rank, world, deadline_s=secs,
                        step_deadline_s=float(getattr(args, "watchdog_step_seconds", 0) or 0))
