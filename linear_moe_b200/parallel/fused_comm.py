"""Fused compute + communication paths over NVLink peer memory.

Workspaces are symmetric-memory allocations (``torch.distributed._symmetric_memory``: CUDA VMM allocation,
handle exchange, every peer's buffer mapped into every rank, optional NVLS multicast mapping).  The kernels
that read and write them are this framework's own (``csrc/lasp_comm.cu``, ``csrc/zero_comm.cu``): torch only
allocates and rendezvouses.  A workspace exists after :func:`init_workspaces` was called on a multi-GPU NCCL
mesh; until then every ``*_workspace`` query returns ``None`` and callers use ``dist.collectives``.

LASP workspace protocol
-----------------------
``data``   fp32 ``[NSLOT][W(src)][BH*D*D]`` — slot ``s`` of rank ``j`` receives the summary of every source rank.
``flags``  int32 ``[NSLOT][W(src)][nctas]``  — epoch numbers, written with release stores by the source.
Call ``i`` of a rank uses slot ``i % NSLOT`` with epoch ``i // NSLOT + 1``.  A rank can run ahead of a peer by
at most one direction of one step (forward waits on lower ranks, backward on higher ranks, and every optimizer
step synchronises all ranks), i.e. by ``2 x layers`` calls, which NSLOT must exceed.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist

_LASP: Dict[str, "LaspWorkspace"] = {}
_TP: Dict[str, object] = {}
_ZERO: Dict[str, object] = {}
STATUS: Optional[torch.Tensor] = None          # device status word shared by the fused kernels


def lasp_workspace(group) -> Optional["LaspWorkspace"]:
    return _LASP.get(group.name)


def tp_workspace(group):
    return _TP.get(group.name)


def zero_workspace(group):
    return _ZERO.get(group.name)


def _symm_empty(numel: int, dtype, device, group):
    import torch.distributed._symmetric_memory as symm
    name = group.pg.group_name if hasattr(group.pg, "group_name") else None
    if name is not None and hasattr(symm, "enable_symm_mem_for_group"):
        try:
            symm.enable_symm_mem_for_group(name)
        except Exception:
            pass                                   # newer torch enables every group implicitly
    t = symm.empty(numel, dtype=dtype, device=device)
    hdl = symm.rendezvous(t, name if name is not None else group.pg)
    return t, hdl


class _LaspArgs(ctypes.Structure):
    _fields_ = [("states", ctypes.c_void_p), ("final_out", ctypes.c_void_p), ("gconst", ctypes.c_void_p),
                ("peer_data", ctypes.c_void_p), ("peer_flags", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("data_off", ctypes.c_longlong), ("flag_off", ctypes.c_longlong), ("epoch", ctypes.c_int),
                ("rank", ctypes.c_int), ("world", ctypes.c_int), ("H", ctypes.c_int), ("G", ctypes.c_int),
                ("cpg", ctypes.c_int), ("T", ctypes.c_int), ("DD", ctypes.c_int), ("BH", ctypes.c_int),
                ("spin_limit", ctypes.c_longlong)]


class LaspWorkspace:
    NSLOT = 64

    def __init__(self, group, max_state_elems: int, device, spin_limit: int = 2_000_000):
        """``max_state_elems`` = B*H*D*D of the largest exchange."""
        self.group, self.device = group, device
        W = group.size
        self.W, self.rank = W, group.rank
        self.max_elems = max_state_elems
        self.max_ctas = (max_state_elems + 255) // 256 + 4096
        self.data, self.data_hdl = _symm_empty(self.NSLOT * W * max_state_elems, torch.float32, device, group)
        self.flags, self.flag_hdl = _symm_empty(self.NSLOT * W * self.max_ctas, torch.int32, device, group)
        self.flags.zero_()
        self.calls = 0
        self.spin_limit = spin_limit
        self.peer_data = torch.tensor(list(self.data_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        self.peer_flags = torch.tensor(list(self.flag_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        torch.cuda.synchronize()
        dist.barrier(group=group.pg)                 # every rank's flags are zero before anyone pushes

    def combine(self, rev: int, states, gconst, final_out, BH, H, G, cpg, T, D):
        from ..ops import cuda as K
        DD = D * D
        assert BH * DD <= self.max_elems, "LASP workspace too small for this state"
        nctas = ((DD + 255) // 256) * BH
        assert nctas <= self.max_ctas
        slot, epoch = self.calls % self.NSLOT, self.calls // self.NSLOT + 1
        self.calls += 1
        a = _LaspArgs()
        a.states = states.data_ptr()
        a.final_out = 0 if final_out is None else final_out.data_ptr()
        a.gconst = 0 if gconst is None else gconst.data_ptr()
        a.peer_data, a.peer_flags = self.peer_data.data_ptr(), self.peer_flags.data_ptr()
        a.status = status_word(self.device).data_ptr()
        a.data_off = slot * self.W * self.max_elems
        a.flag_off = slot * self.W * self.max_ctas
        a.epoch, a.rank, a.world = epoch, self.rank, self.W
        a.H, a.G, a.cpg, a.T, a.DD, a.BH = H, G, cpg, T, DD, BH
        a.spin_limit = self.spin_limit
        # slot layout inside the kernel is [W(src)][BH*DD] / [W(src)][nctas] with the *actual* BH*DD and nctas
        K._check(K.lib().lmoe_lasp_combine(ctypes.c_int(rev), ctypes.byref(a), K._st()), "lasp_combine")


def status_word(device) -> torch.Tensor:
    global STATUS
    if STATUS is None:
        STATUS = torch.zeros(4, dtype=torch.int32, device=device)
    return STATUS


def check_status(where: str = ""):
    """Raise ``CommTimeout`` if any fused kernel gave up on a bounded wait since the last check."""
    if STATUS is None:
        return
    from ..train.watchdog import raise_on_comm_status
    vals = STATUS[:1].cpu()
    if int(vals[0]) != 0:
        STATUS.zero_()
        raise_on_comm_status(vals, where)


def lasp2_scalar(q, k, v, g, scale, group):
    """Scalar-decay linear attention over a sequence split across ``group`` with the exchange fused into the
    combine kernel (forward and backward).  Returns ``(o, state after this rank's slice)``."""
    from ..ops import cuda as K
    ws = lasp_workspace(group)
    D = q.shape[-1]
    scale = D ** -0.5 if scale is None else scale
    K._LASP_CTX = ws
    try:
        base = K._fused_base(q, k, v)
        if base is not None:
            return K._LsmScalarFused.apply(base, g, scale, None)
        return K._LsmScalar.apply(q, k, v, g, scale, None)
    finally:
        K._LASP_CTX = None


def init_workspaces(mesh, cfg=None, tc=None):
    """Allocate the symmetric-memory workspaces of the fused paths for ``mesh`` (NCCL, >1 GPU)."""
    if not torch.cuda.is_available() or not dist.is_initialized() or dist.get_backend() != "nccl":
        return
    device = torch.device("cuda", torch.cuda.current_device())
    cp = mesh["cp"]
    if not cp.is_trivial and cfg is not None and cp.name not in _LASP:
        H = cfg.num_attention_heads // mesh.tp
        dk, dv = cfg.key_dim // cfg.num_attention_heads, cfg.value_dim // cfg.num_attention_heads
        mb = tc.micro_batch_size if tc is not None else 1
        _LASP[cp.name] = LaspWorkspace(cp, mb * H * dk * dv, device)


# ---------------------------------------------------------------------------------------------
# ZeRO-1: fused reduce-scatter + Adam + all-gather over NVLS (csrc/zero_comm.cu)
# ---------------------------------------------------------------------------------------------
class _ZeroArgs(ctypes.Structure):
    _fields_ = [("grads", ctypes.c_void_p), ("grads_mc", ctypes.c_void_p), ("peer_grads", ctypes.c_void_p),
                ("params", ctypes.c_void_p), ("params_mc", ctypes.c_void_p), ("peer_params", ctypes.c_void_p),
                ("peer_flags", ctypes.c_void_p), ("status", ctypes.c_void_p), ("sumsq", ctypes.c_void_p),
                ("done_ctr", ctypes.c_void_p), ("master", ctypes.c_void_p), ("exp_avg", ctypes.c_void_p),
                ("exp_avg_sq", ctypes.c_void_p), ("lo", ctypes.c_longlong), ("hi", ctypes.c_longlong),
                ("rank", ctypes.c_int), ("world", ctypes.c_int), ("epoch", ctypes.c_int), ("grad_scale", ctypes.c_float),
                ("lr", ctypes.c_float), ("b1", ctypes.c_float), ("b2", ctypes.c_float), ("eps", ctypes.c_float),
                ("wd", ctypes.c_float), ("bc1", ctypes.c_float), ("bc2", ctypes.c_float), ("gscale", ctypes.c_float),
                ("spin_limit", ctypes.c_longlong)]


class ZeroBufferWorkspace:
    """Symmetric parameter (bf16) and gradient (fp32) storage of one flat optimizer buffer plus the flags of its two
    barriers.  ``reduce`` and ``adam_broadcast`` are the two kernel launches of a fused ZeRO-1 step."""

    def __init__(self, group, numel: int, device, spin_limit: int = 4_000_000, use_multicast: bool = True):
        self.group, self.device, self.numel = group, device, numel
        self.W, self.rank = group.size, group.rank
        self.params, self.p_hdl = _symm_empty(numel, torch.bfloat16, device, group)
        self.grads, self.g_hdl = _symm_empty(numel, torch.float32, device, group)
        self.flags, self.f_hdl = _symm_empty(2 * self.W + 64, torch.int32, device, group)
        self.flags.zero_()
        mc_p = int(getattr(self.p_hdl, "multicast_ptr", 0) or 0)
        mc_g = int(getattr(self.g_hdl, "multicast_ptr", 0) or 0)
        self.mc_params, self.mc_grads = (mc_p, mc_g) if (use_multicast and mc_p and mc_g) else (0, 0)
        self.peer_params = torch.tensor(list(self.p_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        self.peer_grads = torch.tensor(list(self.g_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        self.peer_flags = torch.tensor(list(self.f_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        self.done_ctr = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.spin_limit = spin_limit
        torch.cuda.synchronize()
        dist.barrier(group=group.pg)

    def _args(self, shard) -> _ZeroArgs:
        a = _ZeroArgs()
        a.grads, a.grads_mc, a.peer_grads = self.grads.data_ptr(), self.mc_grads, self.peer_grads.data_ptr()
        a.params, a.params_mc, a.peer_params = self.params.data_ptr(), self.mc_params, self.peer_params.data_ptr()
        a.peer_flags, a.status = self.peer_flags.data_ptr(), status_word(self.device).data_ptr()
        a.sumsq, a.done_ctr = self.sumsq.data_ptr(), self.done_ctr.data_ptr()
        a.lo, a.hi = shard
        a.rank, a.world, a.epoch = self.rank, self.W, self.epoch
        a.spin_limit = self.spin_limit
        return a

    def reduce(self, shard, grad_scale: float):
        from ..ops import cuda as K
        self.epoch += 1
        self.sumsq.zero_()
        a = self._args(shard)
        a.grad_scale = grad_scale
        K._check(K.lib().lmoe_zero_reduce(ctypes.byref(a), ctypes.c_int(K.NUM_SMS * 4), K._st()), "zero_reduce")

    def adam_broadcast(self, shard, master, exp_avg, exp_avg_sq, lr, b1, b2, eps, wd, bc1, bc2, gscale):
        from ..ops import cuda as K
        a = self._args(shard)
        a.master, a.exp_avg, a.exp_avg_sq = master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr()
        a.lr, a.b1, a.b2, a.eps, a.wd, a.bc1, a.bc2, a.gscale = lr, b1, b2, eps, wd, bc1, bc2, gscale
        K._check(K.lib().lmoe_zero_adam_bcast(ctypes.byref(a), ctypes.c_int(K.NUM_SMS * 4), K._st()), "zero_adam_bcast")
