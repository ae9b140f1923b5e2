"""Named timers on the device clock.

Megatron ``Timers`` (names logged by the reference: training.py:420-444; flags
``--timing-log-level``, ``--barrier-with-L1-time``).  On CUDA a timer brackets its region with
events on the current stream and never synchronises in the hot path; elapsed times are read when the
log line is produced, and reduced as max over ranks.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class _Timer:
    def __init__(self, name: str, level: int, cuda: bool):
        self.name, self.level, self.cuda = name, level, cuda
        self._pairs: List = []
        self._start = None
        self._elapsed = 0.0

    def start(self, barrier: bool = False):
        if barrier and dist.is_initialized():
            dist.barrier()
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._start = ev
        else:
            self._start = time.perf_counter()

    def stop(self):
        if self._start is None:
            return
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pairs.append((self._start, ev))
        else:
            self._elapsed += time.perf_counter() - self._start
        self._start = None

    def elapsed(self, reset: bool = True) -> float:
        """Seconds accumulated since the last reset."""
        if self.cuda and self._pairs:
            self._pairs[-1][1].synchronize()
            self._elapsed += sum(a.elapsed_time(b) for a, b in self._pairs) / 1000.0
            self._pairs = []
        e = self._elapsed
        if reset:
            self._elapsed = 0.0
        return e


class _Null:
    def start(self, barrier: bool = False): pass
    def stop(self): pass


class Timers:
    def __init__(self, log_level: int = 0, cuda: Optional[bool] = None):
        self.log_level = log_level
        self.cuda = torch.cuda.is_available() if cuda is None else cuda
        self._timers: Dict[str, _Timer] = {}
        self._null = _Null()

    def __call__(self, name: str, log_level: int = 0):
        if log_level > self.log_level:
            return self._null
        if name not in self._timers:
            self._timers[name] = _Timer(name, log_level, self.cuda)
        return self._timers[name]

    def collect(self, names=None, reset: bool = True, reduce_max: bool = True) -> Dict[str, float]:
        names = list(self._timers) if names is None else [n for n in names if n in self._timers]
        vals = [self._timers[n].elapsed(reset) for n in names]
        if reduce_max and dist.is_initialized() and dist.get_world_size() > 1 and names:
            t = torch.tensor(vals, dtype=torch.float64,
                             device="cuda" if (self.cuda and dist.get_backend() == "nccl") else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            vals = t.tolist()
        return dict(zip(names, vals))

    def log_string(self, normalizer: float = 1.0) -> str:
        vals = self.collect()
        return " | ".join(f"{k}: {v * 1000.0 / normalizer:.2f}" for k, v in vals.items())
