"""Activation offload to pinned host memory for the first ``num_layers`` transformer blocks.

The reference wraps its layer loop in TransformerEngine's ``get_cpu_offload_context`` (linear_moe/model/qwen2/hybrid/
hybrid_transformer_block.py:120-139, 421-426; flags ``cpu_offloading``, ``cpu_offloading_num_layers``).  Here the same
capability is a ``torch.autograd.graph.saved_tensors_hooks`` pair around each offloaded block:

* **pack** (forward): a tensor saved for backward is copied to a pinned host buffer on a dedicated copy stream that
  waits for the producing stream; the device tensor is handed back to the caching allocator as soon as the copy has
  run (``record_stream``), so the block's activations leave HBM while later blocks compute.  Parameters, tiny tensors
  and CPU tensors are kept as they are.  A tensor saved by several operators of one block is copied once.
* **unpack** (backward): the first tensor asked for from block ``i`` also starts the host->device copies of everything
  block ``i - 1`` saved, on the copy stream, so those overlap block ``i``'s backward; a tensor whose copy was not
  prefetched is fetched on the spot.

Host buffers come from a size-keyed pool of pinned allocations that is reused every step (pinning is a slow,
synchronising call).  With 180 GB of HBM3e the feature is for very long sequences rather than for normal training, so
it is off by default."""
from __future__ import annotations

import contextlib
import weakref
from typing import Dict, List, Optional, Tuple

import torch

__all__ = ["ActivationOffload"]


class _Saved:
    """One offloaded tensor: host copy + how to bring it back."""
    __slots__ = ("host", "device", "ready", "dev", "dev_ready", "group", "nbytes", "uses")

    def __init__(self, host, device, ready, group, nbytes):
        self.host, self.device, self.ready, self.group, self.nbytes = host, device, ready, group, nbytes
        self.dev: Optional[torch.Tensor] = None
        self.dev_ready = None
        self.uses = 1                      # saved-tensor slots that will ask for this tensor in backward


class ActivationOffload:
    """``with offload.layer(i): block(...)`` offloads what block ``i`` saves for backward (``i < num_layers``)."""

    def __init__(self, num_layers: int, *, min_bytes: int = 1 << 20, offload_cpu_tensors: bool = False):
        self.num_layers = int(num_layers)
        self.min_bytes = int(min_bytes)
        self.offload_cpu_tensors = offload_cpu_tensors      # host->host copies; only for exercising the logic without a GPU
        self._stream: Optional[torch.cuda.Stream] = None
        self._pool: Dict[Tuple[int, torch.dtype], List[torch.Tensor]] = {}
        self._groups: Dict[int, List[_Saved]] = {}          # group = one (forward call, block); ids never repeat
        self._prev: Dict[int, int] = {}                     # group -> group of the block before it in the same forward
        self._next_group = 0
        self._last: Optional[Tuple[int, int]] = None        # (layer index, group) of the most recent ``layer()`` call
        self._dedupe: Dict[int, tuple] = {}                 # id(tensor) -> (weakref, version, _Saved)
        self._prefetched: set = set()
        self.stats = {"packed": 0, "deduped": 0, "kept": 0, "bytes": 0, "prefetched": 0, "fetched_late": 0}

    # ------------------------------------------------------------------ host buffers
    def _host_buffer(self, t: torch.Tensor) -> torch.Tensor:
        key = (t.numel(), t.dtype)
        free = self._pool.get(key)
        if free:
            return free.pop()
        return torch.empty(t.numel(), dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)

    def _release(self, s: _Saved):
        if s.host is not None:
            self._pool.setdefault((s.host.numel(), s.host.dtype), []).append(s.host)
            s.host = None

    def _copy_stream(self, device) -> "torch.cuda.Stream":
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=device)
        return self._stream

    # ------------------------------------------------------------------ hooks
    def _eligible(self, t: torch.Tensor) -> bool:
        if not isinstance(t, torch.Tensor) or isinstance(t, torch.nn.Parameter):
            return False
        if t._base is not None and isinstance(t._base, torch.nn.Parameter):       # a view of a weight (w.t())
            return False
        if t.numel() * t.element_size() < self.min_bytes or not t.is_contiguous():
            return False
        return t.is_cuda or self.offload_cpu_tensors

    def _pack(self, group: int, t):
        if not self._eligible(t):
            self.stats["kept"] += 1
            return t
        # the same tensor saved twice is copied once.  Identity is the live Python object (a weak reference): an address
        # is no identity here, since offloaded tensors are freed and their memory is handed to the next activation.
        hit = self._dedupe.get(id(t))
        if hit is not None and hit[0]() is t and hit[1] == t._version and hit[2].group == group and hit[2].host is not None:
            self.stats["deduped"] += 1
            hit[2].uses += 1
            return (hit[2], tuple(t.shape))
        host = self._host_buffer(t)
        ready = None
        if t.is_cuda:
            cur = torch.cuda.current_stream(t.device)
            side = self._copy_stream(t.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                host.copy_(t.reshape(-1), non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(side)
            t.record_stream(side)
        else:
            host.copy_(t.reshape(-1))
        s = _Saved(host, t.device, ready, group, t.numel() * t.element_size())
        self._dedupe[id(t)] = (weakref.ref(t), t._version, s)
        self._groups.setdefault(group, []).append(s)
        self.stats["packed"] += 1
        self.stats["bytes"] += s.nbytes
        return (s, tuple(t.shape))

    def _start_fetch(self, s: _Saved, *, on_side: bool):
        """Bring ``s`` back to its device; on the copy stream when prefetching, else on the consumer's stream.  The host
        buffer stays owned by ``s`` until ``step_done`` (the next step's device->host copies into it are ordered after
        this step's backward through ``wait_stream``)."""
        if s.dev is not None:
            return
        if s.device.type == "cuda":
            cur = torch.cuda.current_stream(s.device)
            stream = self._copy_stream(s.device) if on_side else cur
            with torch.cuda.stream(stream):
                if s.ready is not None:
                    stream.wait_event(s.ready)
                s.dev = torch.empty(s.host.numel(), dtype=s.host.dtype, device=s.device)
                s.dev.copy_(s.host, non_blocking=True)
                s.dev_ready = torch.cuda.Event()
                s.dev_ready.record(stream)
        else:
            s.dev = s.host.clone()

    def _unpack(self, obj):
        if not (isinstance(obj, tuple) and len(obj) == 2 and isinstance(obj[0], _Saved)):
            return obj
        s, shape = obj
        prev = self._prev.get(s.group)
        if prev is not None and prev in self._groups and prev not in self._prefetched:   # overlap the next block's copies
            self._prefetched.add(prev)
            for o in self._groups[prev]:
                if o.uses > 0:
                    self._start_fetch(o, on_side=True)
                    self.stats["prefetched"] += 1
        if s.dev is None:
            self.stats["fetched_late"] += 1
            self._start_fetch(s, on_side=False)
        if s.dev_ready is not None:
            torch.cuda.current_stream(s.device).wait_event(s.dev_ready)
            s.dev.record_stream(torch.cuda.current_stream(s.device))
        out = s.dev.view(shape)
        s.uses -= 1
        if s.uses <= 0:                    # the last consumer owns the device copy from here on
            s.dev, s.dev_ready = None, None
            grp = self._groups.get(s.group)
            if grp is not None and all(o.uses <= 0 for o in grp):          # block fully consumed: recycle its host buffers
                for o in grp:
                    self._release(o)
                del self._groups[s.group]
                self._prev.pop(s.group, None)
                self._prefetched.discard(s.group)
        return out

    # ------------------------------------------------------------------ public
    def layer(self, index: int):
        """Context for block ``index`` of this pipeline stage; a no-op past ``num_layers``.  Every call opens a new group,
        so interleaved micro-batches (1F1B) keep their tensors apart.  A graph built under it is backpropagated once
        (``retain_graph`` replays are not supported: the host copies are recycled after the first pass)."""
        if index >= self.num_layers:
            return contextlib.nullcontext()
        group = self._next_group
        self._next_group += 1
        if self._last is not None and self._last[0] == index - 1:
            self._prev[group] = self._last[1]
        self._last = (index, group)
        return torch.autograd.graph.saved_tensors_hooks(lambda t: self._pack(group, t), self._unpack)

    def step_done(self):
        """Safety net at the end of a step: recycles host buffers of forwards that never ran backward."""
        for group in self._groups.values():
            for s in group:
                self._release(s)
                s.dev, s.dev_ready = None, None
        self._groups.clear()
        self._prev.clear()
        self._dedupe.clear()
        self._prefetched.clear()
        self._last = None

    def pinned_bytes(self) -> int:
        """Bytes of pinned host memory currently in the pool (idle buffers)."""
        return sum(b.numel() * b.element_size() for bufs in self._pool.values() for b in bufs)
