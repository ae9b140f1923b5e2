"""Host-side failure detection: heartbeats through the rendezvous store and a watchdog thread.

The reference has only the process-group timeout, a SIGTERM handler and exit flags
(initialize.py:118-123, training.py:655-691).  Here every rank additionally publishes
``(iteration, wall time)`` to the ``torch.distributed`` store after each step; a daemon thread on
each rank reads its peers' beats and reports ranks whose beat is older than the timeout, so a stalled
or dead peer is noticed on the host before the next collective would block on it.  Nothing here
touches a GPU.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional

import torch.distributed as dist


class Heartbeat:
    def __init__(self, mesh, interval_s: float, timeout_s: float, store=None,
                 on_failure: Optional[Callable[[List[int]], None]] = None, clock: Callable[[], float] = time.time):
        self.mesh, self.interval, self.timeout, self.clock = mesh, interval_s, timeout_s, clock
        self.store = store
        if self.store is None and dist.is_initialized():
            self.store = dist.distributed_c10d._get_default_store()
        self.on_failure = on_failure
        self.failed: List[int] = []
        self._stop = threading.Event()
        self._thread = None
        self._started = clock()
        if self.store is not None and interval_s > 0:
            self._thread = threading.Thread(target=self._watch, daemon=True)
            self._thread.start()

    def _key(self, rank: int) -> str:
        return f"lmoe/heartbeat/{rank}"

    def beat(self, iteration: int):
        if self.store is not None:
            self.store.set(self._key(self.mesh.rank), f"{iteration}:{self.clock():.3f}")

    def check(self) -> List[int]:
        """Ranks whose last beat is older than the timeout (or that never beat within it)."""
        if self.store is None:
            return []
        now, stale = self.clock(), []
        for r in range(self.mesh.world_size):
            if r == self.mesh.rank:
                continue
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    last = self._started
                else:
                    last = float(self.store.get(self._key(r)).decode().split(":")[1])
            except Exception:
                last = self._started
            if now - last > self.timeout:
                stale.append(r)
        return stale

    def _watch(self):
        while not self._stop.wait(self.interval):
            stale = self.check()
            if stale and stale != self.failed:
                self.failed = stale
                msg = f"[watchdog] rank {self.mesh.rank}: no heartbeat from ranks {stale} for > {self.timeout}s"
                print(msg, flush=True)
                if self.on_failure is not None:
                    self.on_failure(stale)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)


class CommTimeout(RuntimeError):
    """Raised on the host when a fused communication kernel reports that a bounded wait ran out."""


def raise_on_comm_status(status_words, where: str = ""):
    """``status_words``: host-readable tensor written by the fused kernels: 0 = ok, otherwise
    ``(kernel_id << 24) | (peer << 16) | phase``."""
    bad = [int(x) for x in status_words.tolist() if int(x) != 0]
    if bad:
        w = bad[0]
        raise CommTimeout(f"{where}: bounded wait expired (kernel {w >> 24}, peer {(w >> 16) & 0xFF}, "
                          f"phase {w & 0xFFFF})")


# ---- scheduler-driven checkpoint-and-exit (``--adlr-autoresume``) ------------------------------------------------------
def _autoresume_service():
    """The cluster's auto-resume client (``userlib.auto_resume.AutoResume``, the library Megatron's
    ``check_adlr_autoresume_termination`` talks to; training.py:639-642), or None where it is not installed."""
    try:
        from userlib.auto_resume import AutoResume
    except ImportError:
        return None
    return AutoResume


def autoresume_termination_requested() -> bool:
    """True when the job should checkpoint and exit: the auto-resume service says so, or the file named by
    ``LMOE_AUTORESUME_FILE`` exists (a plain-file stand-in for clusters without the service: ``touch`` it to stop the job
    at its next check)."""
    import os
    svc = _autoresume_service()
    if svc is not None and svc.termination_requested():
        return True
    path = os.environ.get("LMOE_AUTORESUME_FILE")
    return bool(path) and os.path.exists(path)


def autoresume_request_resume():
    """Tell the service to queue the job again (called by rank 0 once the checkpoint is written)."""
    svc = _autoresume_service()
    if svc is not None:
        svc.request_resume()
