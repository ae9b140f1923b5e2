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
Call ``i`` of a rank uses slot ``i % NSLOT`` with epoch ``i // NSLOT + 1``.  The exchange itself does not bound how
far a rank runs ahead of a peer: in the forward direction rank 0 waits for nobody, in the backward direction the last
rank waits for nobody, so within one pass a rank can lead by every LSM layer of its stage, and a forward-only loop has no
other cross-rank dependency at all.  Slot reuse is therefore guarded on the host: ``NSLOT`` is sized from the layer count
(two passes of every layer), the trainer calls :func:`mark_step_sync` after each optimizer step (whose gradient
reduction waits for every rank), and a workspace that has issued ``NSLOT - 1`` exchanges since the last such point
enqueues a one-element all-reduce on the group first: it completes on a rank's stream only when every rank's stream
has reached it, i.e. when every earlier exchange of every rank has finished and all slots are free.
"""
from __future__ import annotations

import ctypes
import os
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
    # every peer-writable buffer ends in a guard region with a fixed byte pattern: a peer (or a local kernel) that writes
    # past the logical end of a workspace lands there, and `verify_canaries` (run from `check_status` with LMOE_CANARY=1)
    # reports which buffer was overrun
    t = symm.empty(numel + _CANARY_ELEMS, dtype=dtype, device=device)
    hdl = symm.rendezvous(t, name if name is not None else group.pg)
    t[numel:].view(torch.uint8).fill_(_CANARY_BYTE)
    _CANARIES.append((f"{group.name}:{dtype}:{numel}", t, numel))
    return t[:numel], hdl


_CANARY_ELEMS, _CANARY_BYTE = 256, 0xA5
_CANARIES: list = []


def verify_canaries():
    """Raise if the guard region behind any symmetric workspace of this rank no longer holds its pattern."""
    bad = [name for name, t, numel in _CANARIES if bool((t[numel:].view(torch.uint8) != _CANARY_BYTE).any())]
    if bad:
        raise RuntimeError(f"workspace overrun: the guard region of {bad} was overwritten")


class _LaspArgs(ctypes.Structure):
    _fields_ = [("states", ctypes.c_void_p), ("final_out", ctypes.c_void_p), ("gconst", ctypes.c_void_p),
                ("gdecay", ctypes.c_void_p), ("r_out", ctypes.c_void_p),
                ("peer_data", ctypes.c_void_p), ("peer_flags", ctypes.c_void_p), ("status", ctypes.c_void_p),
                ("data_off", ctypes.c_longlong), ("dec_off", ctypes.c_longlong), ("flag_off", ctypes.c_longlong),
                ("epoch", ctypes.c_int), ("rank", ctypes.c_int), ("world", ctypes.c_int), ("H", ctypes.c_int),
                ("G", ctypes.c_int), ("cpg", ctypes.c_int), ("T", ctypes.c_int), ("DD", ctypes.c_int), ("BH", ctypes.c_int),
                ("dmode", ctypes.c_int), ("D", ctypes.c_int), ("spin_limit", ctypes.c_longlong)]


class LaspWorkspace:
    def __init__(self, group, max_state_elems: int, device, spin_limit: Optional[int] = None, nslot: int = 64):
        """``max_state_elems`` = B*H*D*D of the largest exchange; ``nslot`` = exchanges that may be in flight between two
        points at which all ranks are known to have caught up."""
        self.group, self.device = group, device
        self.NSLOT = max(int(nslot), 4)
        self.since_sync = 0
        self.timing = None                           # a list: every exchange appends its (start, end) CUDA events
        self._sync_token = torch.zeros(1, dtype=torch.float32, device=device)
        W = group.size
        self.W, self.rank = W, group.rank
        self.max_elems = max_state_elems
        self.max_ctas = (max_state_elems + 255) // 256 + 4096
        self.max_dec = max(max_state_elems // 64, 1)             # summed log decay per state row (rows are >= 64 wide)
        self.data, self.data_hdl = _symm_empty(self.NSLOT * W * (max_state_elems + self.max_dec), torch.float32, device, group)
        self.flags, self.flag_hdl = _symm_empty(self.NSLOT * W * self.max_ctas, torch.int32, device, group)
        self.flags.zero_()
        self.calls = 0
        self.spin_limit = default_spin_limit() if spin_limit is None else spin_limit
        self.peer_data = torch.tensor(list(self.data_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        self.peer_flags = torch.tensor(list(self.flag_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        torch.cuda.synchronize()
        dist.barrier(group=group.pg)                 # every rank's flags are zero before anyone pushes

    def combine(self, rev: int, states, gconst, final_out, BH, H, G, cpg, T, D, gdecay=None, dmode: int = 0, r_out=None):
        """One exchange.  ``dmode`` 0: no decay or the constant per-head log decay ``gconst``; 1: ``gdecay`` ``[BH, G]``
        summed log decay per group (data-dependent scalar decay); 2: ``gdecay`` ``[BH, G, D]`` (per key channel).
        ``r_out`` ``[BH, D*D]`` receives the folded remote state."""
        from ..ops import cuda as K
        assert (dmode == 0) == (gdecay is None)
        DD = D * D
        assert BH * DD <= self.max_elems, "LASP workspace too small for this state"
        nctas = ((DD + 255) // 256) * BH
        assert nctas <= self.max_ctas
        if self.since_sync >= self.NSLOT - 1:
            dist.all_reduce(self._sync_token, group=self.group.pg)      # stream-ordered: all earlier exchanges are over
            self.since_sync = 0
        self.since_sync += 1
        slot, epoch = self.calls % self.NSLOT, self.calls // self.NSLOT + 1
        self.calls += 1
        a = _LaspArgs()
        a.states = states.data_ptr()
        a.final_out = 0 if final_out is None else final_out.data_ptr()
        a.gconst = 0 if gconst is None else gconst.data_ptr()
        a.gdecay = 0 if gdecay is None else gdecay.data_ptr()
        a.r_out = 0 if r_out is None else r_out.data_ptr()
        a.dmode, a.D = dmode, D
        a.dec_off = self.NSLOT * self.W * self.max_elems + slot * self.W * self.max_dec
        a.peer_data, a.peer_flags = self.peer_data.data_ptr(), self.peer_flags.data_ptr()
        a.status = status_word(self.device).data_ptr()
        a.data_off = slot * self.W * self.max_elems
        a.flag_off = slot * self.W * self.max_ctas
        a.epoch, a.rank, a.world = epoch, self.rank, self.W
        a.H, a.G, a.cpg, a.T, a.DD, a.BH = H, G, cpg, T, DD, BH
        a.spin_limit = self.spin_limit
        # slot layout inside the kernel is [W(src)][BH*DD] / [W(src)][nctas] with the *actual* BH*DD and nctas
        if self.timing is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        K._check(K.lib().lmoe_lasp_combine(ctypes.c_int(rev), ctypes.byref(a), K._st()), "lasp_combine")
        if self.timing is not None:
            e1.record()
            self.timing.append((e0, e1))


def mark_step_sync():
    """Called at a point of the step at which every rank has finished its earlier sequence-parallel exchanges (after the
    gradient reduction): the slot counters of the LASP workspaces start again."""
    for ws in _LASP.values():
        ws.since_sync = 0


def status_word(device) -> torch.Tensor:
    global STATUS
    if STATUS is None:
        STATUS = torch.zeros(4, dtype=torch.int32, device=device)
    return STATUS


def check_status(where: str = ""):
    """Raise ``CommTimeout`` if any fused kernel gave up on a bounded wait since the last check, or ``RuntimeError`` if
    a tcgen05 GEMM did (its error word is the second element of the same status tensor, so one read covers both), or if
    a decay too strong for the gated-scan kernels was seen (third element)."""
    if os.environ.get("LMOE_CANARY", "0") != "0":
        verify_canaries()
    if STATUS is None:
        return
    from ..train.watchdog import raise_on_comm_status
    vals = STATUS[:3].cpu()
    if int(vals[2]) != 0:
        STATUS.zero_()
        raise RuntimeError("a key-channel log decay below -80 over half a chunk (32 tokens) reached the chunked gated-scan "
                           f"kernels, whose bf16 operand rescaling overflows there {where}; LMOE_RWKV6_KERNEL=0 selects the "
                           "16-token torch form for RWKV6")
    if int(vals[0]) != 0:
        STATUS.zero_()
        raise_on_comm_status(vals[:1], where)
    if int(vals[1]) != 0:
        STATUS.zero_()
        raise RuntimeError(f"tcgen05 GEMM: bounded wait expired (code {int(vals[1]):#x}) {where}")


# Budget of every bounded wait of the fused kernels.  The default is far above ordinary rank skew (a rank that stalls on
# the host for a checkpoint copy or a page-in holds the others' kernels in their waits); tests that let a wait run out
# pass a short limit to the workspace they build.  ``--fused-comm-timeout-s`` / ``LMOE_COMM_TIMEOUT_S`` change it.
_TIMEOUT_S = float(os.environ.get("LMOE_COMM_TIMEOUT_S", "20"))


def set_timeout(seconds: float):
    """Seconds a fused kernel waits for a peer before it records a timeout (applies to workspaces built afterwards)."""
    global _TIMEOUT_S
    _TIMEOUT_S = float(seconds)


def default_spin_limit() -> int:
    return max(1000, int(_TIMEOUT_S * 1_000_000))            # one poll of a remote flag is about a microsecond


def default_spin_cycles() -> int:
    return max(1_000_000, int(_TIMEOUT_S * 2_000_000_000))   # SM clock cycles at ~2 GHz


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


def lasp2_vector(q, k, v, gk, scale, group):
    """Key-channel-gated linear attention (GLA, HGRN2, RWKV6 without bonus) over a sequence split across ``group``, the
    exchange (state summaries and per-channel slice decays) fused into the combine kernel."""
    from ..ops import cuda as K
    ws = lasp_workspace(group)
    D = q.shape[-1]
    scale = D ** -0.5 if scale is None else scale
    K._LASP_CTX = ws
    try:
        base = K._fused_base(q, k, v)
        if base is not None:
            return K._LsmVectorFused.apply(base, gk, scale, None)
        return K._LsmVector.apply(q, k, v, gk, scale, None)
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
        _LASP[cp.name] = LaspWorkspace(cp, mb * H * dk * dv, device, nslot=max(64, 2 * cfg.num_layers + 2))
    tpg = mesh["tp"]
    if (not tpg.is_trivial and tpg.size <= 8 and cfg is not None and tpg.name not in _TP
            and os.environ.get("LMOE_FUSED_TP", "1") != "0"):
        mb = tc.micro_batch_size if tc is not None else 1
        seq = (tc.seq_length if tc is not None else cfg.max_position_embeddings) // max(mesh.cp, 1) // tpg.size
        _TP[tpg.name] = TpWorkspace(tpg, mb * seq * cfg.hidden_size, device)
    tpep = mesh["tp_ep"]
    if (not mesh["tp"].is_trivial and not tpep.is_trivial and cfg is not None and cfg.num_experts and tpep.name not in _MOE
            and cfg.moe_topk * mesh.tp <= 16 and os.environ.get("LMOE_FUSED_MOE", "1") != "0"):
        # tensor-parallel experts: (expert, TP shard) pairs are the virtual experts of the TP x EP group
        mb = tc.micro_batch_size if tc is not None else 1
        seq = (tc.seq_length if tc is not None else cfg.max_position_embeddings) // max(mesh.cp, 1) // mesh.tp
        rows = mb * seq * cfg.moe_topk * mesh.tp
        factor = float(os.environ.get("LMOE_MOE_RECV_FACTOR", "2.0"))
        cap = int(rows * factor) + 256 * (cfg.num_experts // mesh.ep)
        _MOE[tpep.name] = MoeWorkspace(tpep, cfg.num_experts * mesh.tp, cfg.hidden_size, cap, device)
    ep = mesh["ep"]
    if (not ep.is_trivial and mesh["tp"].is_trivial and cfg is not None and cfg.num_experts and ep.name not in _MOE
            and os.environ.get("LMOE_FUSED_MOE", "1") != "0"):
        mb = tc.micro_batch_size if tc is not None else 1
        seq = (tc.seq_length if tc is not None else cfg.max_position_embeddings) // max(mesh.cp, 1)
        tokens = mb * seq * cfg.moe_topk
        factor = float(os.environ.get("LMOE_MOE_RECV_FACTOR", "2.0"))         # receive rows per rank / average
        cap = int(tokens * factor) + 256 * (cfg.num_experts // ep.size)
        _MOE[ep.name] = MoeWorkspace(ep, cfg.num_experts, cfg.hidden_size, cap, device)


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
                ("spin_limit", ctypes.c_longlong), ("slot", ctypes.c_int)]


class ZeroBufferWorkspace:
    """Symmetric parameter (bf16) and gradient (fp32) storage of one flat optimizer buffer plus the flags of its two
    barriers.  ``reduce`` and ``adam_broadcast`` are the two kernel launches of a fused ZeRO-1 step."""

    MAX_BUCKETS = 510            # flag slots for bucketed reduces (one per bucket and step)

    def __init__(self, group, numel: int, device, spin_limit: Optional[int] = None, use_multicast: bool = True):
        self.group, self.device, self.numel = group, device, numel
        self.W, self.rank = group.size, group.rank
        self.params, self.p_hdl = _symm_empty(numel, torch.bfloat16, device, group)
        self.grads, self.g_hdl = _symm_empty(numel, torch.float32, device, group)
        self.flags, self.f_hdl = _symm_empty((2 + self.MAX_BUCKETS) * self.W + 64, torch.int32, device, group)
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
        self.spin_limit = default_spin_limit() if spin_limit is None else spin_limit
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
        a.slot = 0
        K._check(K.lib().lmoe_zero_reduce(ctypes.byref(a), ctypes.c_int(K.NUM_SMS * 4), K._st()), "zero_reduce")

    # -- bucketed form: the reduction of a step is split into ranges that are launched as soon as their gradients exist
    def begin_step(self):
        """Start the bucketed reduction of one optimizer step (every rank calls it at the same point)."""
        self.epoch += 1
        self.sumsq.zero_()
        self._next_slot = 1

    def reduce_range(self, lo: int, hi: int, shard, grad_scale: float, blocks: Optional[int] = None):
        """Reduce-scatter ``[lo, hi)`` of the flat buffer: this rank sums the part of the range that lies in its shard over
        all ranks (NVLS ``multimem.ld_reduce``); a rank that owns none of it only signals that its gradients of the range
        are complete.  Every rank must issue the same sequence of ranges per step.  Runs on the current stream."""
        from ..ops import cuda as K
        assert self._next_slot <= self.MAX_BUCKETS, "too many gradient buckets in one step"
        a = self._args((max(lo, shard[0]), max(min(hi, shard[1]), max(lo, shard[0]))))
        a.grad_scale = grad_scale
        a.slot = self._next_slot
        self._next_slot += 1
        K._check(K.lib().lmoe_zero_reduce(ctypes.byref(a), ctypes.c_int(blocks or K.NUM_SMS * 2), K._st()), "zero_reduce")

    def adam_broadcast(self, shard, master, exp_avg, exp_avg_sq, lr, b1, b2, eps, wd, bc1, bc2, gscale):
        from ..ops import cuda as K
        a = self._args(shard)
        a.master, a.exp_avg, a.exp_avg_sq = master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr()
        a.lr, a.b1, a.b2, a.eps, a.wd, a.bc1, a.bc2, a.gscale = lr, b1, b2, eps, wd, bc1, bc2, gscale
        K._check(K.lib().lmoe_zero_adam_bcast(ctypes.byref(a), ctypes.c_int(K.NUM_SMS * 4), K._st()), "zero_adam_bcast")


# ---------------------------------------------------------------------------------------------
# MoE dispatch / combine over peer memory (csrc/moe_comm.cu)
# ---------------------------------------------------------------------------------------------
_MOE: Dict[str, "MoeWorkspace"] = {}


def moe_workspace(group) -> Optional["MoeWorkspace"]:
    return _MOE.get(group.name)


_MOE_LOCAL: Dict[tuple, "MoeWorkspace"] = {}


def local_moe_workspace(num_experts: int, hidden: int, rows: int, device) -> "MoeWorkspace":
    """One-rank workspace (ordinary tensors) for a MoE layer without expert parallelism: the same push / pull kernels
    replace the index_select / index_add_ permutation, which is several times slower in both directions."""
    key = (str(device), num_experts, hidden)
    ws = _MOE_LOCAL.get(key)
    if ws is None or ws.cap < rows:
        ws = MoeWorkspace(None, num_experts, hidden, rows, device)
        _MOE_LOCAL[key] = ws
    return ws


class _MoeArgs(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_void_p) for n in ("peer_cnt", "peer_flags", "peer_x", "peer_y", "status", "done_ctr")] +
                [(n, ctypes.c_int) for n in ("rank", "world", "E", "El", "cap", "h", "epoch")] +
                [("spin_limit", ctypes.c_longlong)] +
                [(n, ctypes.c_void_p) for n in ("offs", "real", "send_base", "idx", "blockhist", "blockbase")] +
                [("nchunks", ctypes.c_int)] +
                [(n, ctypes.c_void_p) for n in ("dest_rank", "dest_row", "src", "w", "out", "rows")] +
                [("n_assign", ctypes.c_int), ("k", ctypes.c_int), ("pad", ctypes.c_int)])


class MoeWorkspace:
    """Receive buffer ``x [cap, h]``, result buffer ``y [cap, h]``, count matrix and flags of one expert-parallel group.
    ``group=None`` builds a one-rank workspace out of ordinary tensors (single-GPU use and tests)."""

    def __init__(self, group, num_experts: int, hidden: int, cap_rows: int, device, spin_limit: Optional[int] = None):
        self.group, self.device = group, device
        self.W, self.rank = (group.size, group.rank) if group is not None else (1, 0)
        W = self.W
        assert num_experts % W == 0 and hidden % 8 == 0
        self.E, self.El, self.h = num_experts, num_experts // W, hidden
        self.cap = (cap_rows + 255) // 256 * 256
        if group is not None:
            self.x, hx = _symm_empty(self.cap * hidden, torch.bfloat16, device, group)
            self.y, hy = _symm_empty(self.cap * hidden, torch.bfloat16, device, group)
            self.cnt, hc = _symm_empty(W * num_experts, torch.int32, device, group)
            self.flags, hf = _symm_empty(3 * W + 64, torch.int32, device, group)
            self._hdls = (hx, hy, hc, hf)
            ptrs = [list(hd.buffer_ptrs) for hd in self._hdls]
        else:
            self.x = torch.empty(self.cap * hidden, dtype=torch.bfloat16, device=device)
            self.y = torch.empty(self.cap * hidden, dtype=torch.bfloat16, device=device)
            self.cnt = torch.empty(W * num_experts, dtype=torch.int32, device=device)
            self.flags = torch.empty(3 * W + 64, dtype=torch.int32, device=device)
            ptrs = [[t.data_ptr()] for t in (self.x, self.y, self.cnt, self.flags)]
        for t in (self.x, self.y, self.cnt, self.flags):
            t.zero_()
        self.x, self.y = self.x.view(self.cap, hidden), self.y.view(self.cap, hidden)
        self.peer_x, self.peer_y, self.peer_cnt, self.peer_flags = [
            torch.tensor(p, dtype=torch.int64, device=device) for p in ptrs]
        self.done_ctr = torch.zeros(1, dtype=torch.int32, device=device)
        self.ep_exchange = self.ep_push = self.ep_pull = 0
        self.spin_limit = default_spin_limit() if spin_limit is None else spin_limit
        torch.cuda.synchronize()
        if group is not None:
            dist.barrier(group=group.pg)

    def _args(self) -> _MoeArgs:
        a = _MoeArgs()
        a.peer_cnt, a.peer_flags = self.peer_cnt.data_ptr(), self.peer_flags.data_ptr()
        a.peer_x, a.peer_y = self.peer_x.data_ptr(), self.peer_y.data_ptr()
        a.status, a.done_ctr = status_word(self.device).data_ptr(), self.done_ctr.data_ptr()
        a.rank, a.world, a.E, a.El, a.cap, a.h = self.rank, self.W, self.E, self.El, self.cap, self.h
        a.spin_limit = self.spin_limit
        from ..ops import gemm
        a.pad = gemm.ROW_ALIGN
        return a

    def _run(self, which: int, a: _MoeArgs, name: str):
        from ..ops import cuda as K
        K._check(K.lib().lmoe_moe_comm(ctypes.c_int(which), ctypes.byref(a), ctypes.c_int(K.NUM_SMS), K._st()), name)

    def route(self, idx: torch.Tensor):
        """Top-k expert indices ``[T, k]`` (``-1`` = dropped) -> routing record: destination (rank, row) of every
        (token, slot) pair, padded offsets and real sizes of the local expert segments.  No host synchronisation."""
        T, k = idx.shape
        dev = idx.device
        flat = idx.reshape(-1).contiguous()
        if flat.dtype != torch.int64:
            flat = flat.to(torch.int64)
        nch = (T * k + 4095) // 4096
        scratch = torch.empty(2 * nch * self.E + self.El + 1 + self.El + self.E + 2 * T * k, dtype=torch.int32, device=dev)
        o = 0
        blockhist = scratch[o:o + nch * self.E]; o += nch * self.E
        blockbase = scratch[o:o + nch * self.E]; o += nch * self.E
        offs = scratch[o:o + self.El + 1]; o += self.El + 1
        real = scratch[o:o + self.El]; o += self.El
        send_base = scratch[o:o + self.E]; o += self.E
        dest_rank = scratch[o:o + T * k]; o += T * k
        dest_row = scratch[o:o + T * k]
        self.ep_exchange += 1
        a = self._args()
        a.epoch = self.ep_exchange
        a.offs, a.real, a.send_base = offs.data_ptr(), real.data_ptr(), send_base.data_ptr()
        a.idx, a.blockhist, a.blockbase, a.nchunks = flat.data_ptr(), blockhist.data_ptr(), blockbase.data_ptr(), nch
        a.dest_rank, a.dest_row = dest_rank.data_ptr(), dest_row.data_ptr()
        a.n_assign, a.k = T * k, k
        self._run(6, a, "moe_count")
        self._run(0, a, "moe_exchange")
        self._run(1, a, "moe_assign")
        return MoeRoute(T, k, dest_rank, dest_row, offs, real)

    def result_holder(self):
        """The buffer the peers pull from, for a producer that writes into it directly (``None`` on one rank, where results
        are read where they are)."""
        return None if self.group is None else _BufHolder(self.y)

    def push(self, src: torch.Tensor, route: "MoeRoute", weights: Optional[torch.Tensor], keep: bool = True) -> torch.Tensor:
        """Send every (token, slot) row of ``src [T, h]`` (times ``weights [T*k]``) to its expert's rank; returns this
        rank's receive buffer ``[cap, h]`` with zeroed padding rows: a copy with ``keep`` (the forward pass saves it for the
        weight gradient), the shared buffer itself without (the backward pass consumes it before this rank signals its
        results, and no peer pushes again before it has pulled those)."""
        assert src.is_contiguous() and src.dtype == torch.bfloat16 and src.shape == (route.T, self.h)
        self.ep_push += 1
        a = self._args()
        a.epoch = self.ep_push
        a.src = src.data_ptr()
        a.w = 0 if weights is None else weights.data_ptr()
        a.dest_rank, a.dest_row = route.dest_rank.data_ptr(), route.dest_row.data_ptr()
        a.offs, a.real = route.offs.data_ptr(), route.real.data_ptr()
        a.n_assign, a.k = route.T * route.k, route.k
        if self.group is None:
            # one rank: the receive buffer is a fresh tensor that the caller keeps, no copy out of a shared buffer
            x = torch.empty(self.cap, self.h, dtype=torch.bfloat16, device=self.device)
            self.peer_x.fill_(x.data_ptr())
            self._run(2, a, "moe_push")
            self._run(3, a, "moe_zero_pads")
            return x
        self._run(2, a, "moe_push")
        self._run(3, a, "moe_zero_pads")
        return self.x.clone() if keep else self.x

    def pull(self, y_local: torch.Tensor, route: "MoeRoute", weights: Optional[torch.Tensor], save_rows: bool):
        """Publish this rank's expert results ``[cap, h]`` and gather, weight and sum every token's ``k`` rows from their
        owners.  Returns ``(out [T, h], rows [T*k, h] or None)``."""
        self.ep_pull += 1
        if self.group is None:
            y_local = y_local.contiguous()
            self.peer_y.fill_(y_local.data_ptr())                # one rank: read the results where they are
        elif y_local.data_ptr() != self.y.data_ptr():
            self.y.copy_(y_local)                                # (the grouped GEMM normally writes into self.y itself)
        a = self._args()
        a.epoch = self.ep_pull
        out = torch.empty(route.T, self.h, dtype=torch.bfloat16, device=self.device)
        rows = torch.empty(route.T * route.k, self.h, dtype=torch.bfloat16, device=self.device) if save_rows else None
        a.w = 0 if weights is None else weights.data_ptr()
        a.out, a.rows = out.data_ptr(), 0 if rows is None else rows.data_ptr()
        a.dest_rank, a.dest_row = route.dest_rank.data_ptr(), route.dest_row.data_ptr()
        a.n_assign, a.k = route.T * route.k, route.k
        self._run(4, a, "moe_signal")
        self._run(5, a, "moe_pull")
        return out, rows


class _BufHolder:
    """A tensor behind a plain attribute, so that it can be handed to an autograd function without being tracked."""

    def __init__(self, buf):
        self.buf = buf


class MoeRoute:
    def __init__(self, T, k, dest_rank, dest_row, offs, real):
        self.T, self.k, self.dest_rank, self.dest_row, self.offs, self.real = T, k, dest_rank, dest_row, offs, real


# ---------------------------------------------------------------------------------------------
# Sequence-parallel linear layers: all-gather -> GEMM and GEMM -> reduce-scatter in one kernel (csrc/gemm_tp.cu)
# ---------------------------------------------------------------------------------------------
class _TpParams(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_int) for n in ("mode", "rank", "world", "M_loc", "T_loc", "N", "K", "ldc")] +
                [("C", ctypes.c_void_p), ("peer_inbox", ctypes.c_void_p), ("inbox_off", ctypes.c_longlong),
                 ("peer_flags", ctypes.c_void_p), ("epoch", ctypes.c_int), ("done_ctr", ctypes.c_void_p),
                 ("status", ctypes.c_void_p), ("err", ctypes.c_void_p), ("spin_cycles", ctypes.c_longlong),
                 ("peer_x", ctypes.c_void_p), ("gathered", ctypes.c_void_p), ("ready", ctypes.c_void_p), ("n_copy", ctypes.c_int)])


class _TpCommArgs(ctypes.Structure):
    _fields_ = [("peer_flags", ctypes.c_void_p), ("peer_x", ctypes.c_void_p), ("peer_inbox", ctypes.c_void_p),
                ("x_off", ctypes.c_longlong), ("inbox_off", ctypes.c_longlong), ("status", ctypes.c_void_p),
                ("rank", ctypes.c_int), ("world", ctypes.c_int), ("epoch", ctypes.c_int), ("M_loc", ctypes.c_int),
                ("T_loc", ctypes.c_int), ("cols", ctypes.c_int), ("out", ctypes.c_void_p), ("spin_limit", ctypes.c_longlong)]


class TpWorkspace:
    """Symmetric buffers of one tensor-parallel group: ``NSLOT`` published activation shards, ``NSLOT`` inboxes of
    ``W`` partial results, and the flags.  Two consecutive calls never share a slot, and a rank can be at most one call
    ahead of a peer (every call needs data of every rank), so a slot is never overwritten while a peer still reads it."""
    NSLOT = 4

    def __init__(self, group, max_shard_elems: int, device, spin_limit: Optional[int] = None):
        self.group, self.device = group, device
        self.W, self.rank = group.size, group.rank
        assert self.W <= 8
        self.max_elems = (max_shard_elems + 127) // 128 * 128
        self.xs, hx = _symm_empty(self.NSLOT * self.max_elems, torch.bfloat16, device, group)
        self.inbox, hi = _symm_empty(self.NSLOT * self.W * self.max_elems, torch.bfloat16, device, group)
        self.flags, hf = _symm_empty(2 * self.W + 64, torch.int32, device, group)
        self._hdls = (hx, hi, hf)
        self.flags.zero_()
        self.x_ptrs = list(hx.buffer_ptrs)
        self.peer_x = torch.tensor(self.x_ptrs, dtype=torch.int64, device=device)
        self.peer_inbox = torch.tensor(list(hi.buffer_ptrs), dtype=torch.int64, device=device)
        self.peer_flags = torch.tensor(list(hf.buffer_ptrs), dtype=torch.int64, device=device)
        self.done_ctr = torch.zeros(1, dtype=torch.int32, device=device)
        self.ag_calls = self.rs_calls = 0
        self.spin_limit = default_spin_limit() if spin_limit is None else spin_limit
        self.spin_cycles = default_spin_cycles() if spin_limit is None else max(1_000_000, spin_limit * 1000)
        # all-gather -> GEMM: per-slot pointer tables of the published shards, scratch for the gathered matrix, row-block flags
        self.peer_x_slot = [torch.tensor([p + 2 * s * self.max_elems for p in self.x_ptrs], dtype=torch.int64, device=device)
                            for s in range(self.NSLOT)]
        self.gathered = torch.empty(self.W * self.max_elems, dtype=torch.bfloat16, device=device)
        self.ready = torch.zeros(self.W * (self.max_elems // 1024 + 1), dtype=torch.int32, device=device)
        self.n_copy = int(os.environ.get("LMOE_TP_COPY_CTAS", "16"))
        torch.cuda.synchronize()
        dist.barrier(group=group.pg)

    def supports(self, m_loc: int, t_loc: int, cols_shard: int, n: int, k: int) -> bool:
        return (t_loc % 128 == 0 and m_loc % t_loc == 0 and n % 8 == 0 and k % 8 == 0 and cols_shard % 8 == 0
                and m_loc * cols_shard <= self.max_elems)

    def _comm(self) -> _TpCommArgs:
        a = _TpCommArgs()
        a.peer_flags, a.peer_x, a.peer_inbox = self.peer_flags.data_ptr(), self.peer_x.data_ptr(), self.peer_inbox.data_ptr()
        a.status = status_word(self.device).data_ptr()
        a.rank, a.world, a.spin_limit = self.rank, self.W, self.spin_limit
        return a

    def publish(self, x2d: torch.Tensor):
        """Copy this rank's shard ``[M_loc, cols]`` into the next slot and raise the flag on every peer."""
        from ..ops import cuda as K
        self.ag_calls += 1
        epoch, slot = self.ag_calls, self.ag_calls % self.NSLOT
        off = slot * self.max_elems
        self.xs[off: off + x2d.numel()].view_as(x2d).copy_(x2d)
        a = self._comm()
        a.epoch = epoch
        K._check(K.lib().lmoe_tp_comm(ctypes.c_int(0), ctypes.byref(a), ctypes.c_int(K.NUM_SMS), K._st()), "tp_signal")
        return epoch, off

    def _params(self, m_loc, t_loc, n, k) -> _TpParams:
        from ..ops import gemm
        p = _TpParams()
        p.rank, p.world, p.M_loc, p.T_loc, p.N, p.K = self.rank, self.W, m_loc, t_loc, n, k
        p.peer_inbox, p.peer_flags = self.peer_inbox.data_ptr(), self.peer_flags.data_ptr()
        p.done_ctr, p.status = self.done_ctr.data_ptr(), status_word(self.device).data_ptr()
        p.err = gemm._err(self.device).data_ptr()
        p.spin_cycles = self.spin_cycles
        return p

    def ag_gemm(self, pub, m_loc: int, t_loc: int, k: int, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """``gather(shards)[M_full, k] @ (w^T if not b_mn else w)`` reading the shards published as ``pub``."""
        from ..ops import cuda as K
        epoch, off = pub
        n = w.shape[1] if b_mn else w.shape[0]
        out = torch.empty(m_loc * self.W, n, dtype=torch.bfloat16, device=self.device)
        p = self._params(m_loc, t_loc, n, k)
        p.C, p.ldc, p.epoch = out.data_ptr(), n, epoch
        slot = off // self.max_elems
        p.peer_x, p.gathered, p.ready = self.peer_x_slot[slot].data_ptr(), self.gathered.data_ptr(), self.ready.data_ptr()
        p.n_copy = self.n_copy
        ptrs = (ctypes.c_void_p * 8)(self.x_ptrs[self.rank] + 2 * off, self.gathered.data_ptr(), 0, 0, 0, 0, 0, 0)
        K._check(K.lib().lmoe_gemm_tp(ctypes.c_int(0), ptrs, K._p(w), ctypes.c_int(w.shape[0]), ctypes.c_int(w.shape[1]),
                                      ctypes.c_int(int(b_mn)), ctypes.byref(p), ctypes.c_int(K.NUM_SMS), K._st()), "gemm_tp_ag")
        return out

    def gemm_rs(self, x2d: torch.Tensor, t_loc: int, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
        """``reduce_scatter(x2d[M_full, k] @ (w^T if not b_mn else w))`` -> ``[M_loc, n]``."""
        from ..ops import cuda as K
        m_full, k = x2d.shape
        m_loc = m_full // self.W
        n = w.shape[1] if b_mn else w.shape[0]
        self.rs_calls += 1
        epoch, slot = self.rs_calls, self.rs_calls % self.NSLOT
        p = self._params(m_loc, t_loc, n, k)
        p.inbox_off, p.epoch, p.ldc = slot * self.W * self.max_elems, epoch, n
        ptrs = (ctypes.c_void_p * 8)(*[x2d.data_ptr()] * 8)
        K._check(K.lib().lmoe_gemm_tp(ctypes.c_int(1), ptrs, K._p(w), ctypes.c_int(w.shape[0]), ctypes.c_int(w.shape[1]),
                                      ctypes.c_int(int(b_mn)), ctypes.byref(p), ctypes.c_int(K.NUM_SMS), K._st()), "gemm_tp_rs")
        out = torch.empty(m_loc, n, dtype=torch.bfloat16, device=self.device)
        a = self._comm()
        a.inbox_off, a.epoch, a.M_loc, a.T_loc, a.cols, a.out = p.inbox_off, epoch, m_loc, t_loc, n, out.data_ptr()
        K._check(K.lib().lmoe_tp_comm(ctypes.c_int(1), ctypes.byref(a), ctypes.c_int(K.NUM_SMS), K._st()), "tp_reduce")
        return out

    def gather(self, pub, m_loc: int, t_loc: int, cols: int) -> torch.Tensor:
        from ..ops import cuda as K
        epoch, off = pub
        out = torch.empty(m_loc * self.W, cols, dtype=torch.bfloat16, device=self.device)
        a = self._comm()
        a.x_off, a.epoch, a.M_loc, a.T_loc, a.cols, a.out = off, epoch, m_loc, t_loc, cols, out.data_ptr()
        K._check(K.lib().lmoe_tp_comm(ctypes.c_int(2), ctypes.byref(a), ctypes.c_int(K.NUM_SMS), K._st()), "tp_gather")
        return out


def _wgrad(w, dy2d, x2d):
    """``dy^T x`` on the dense tcgen05 kernel: straight into ``w.main_grad`` in fp32 when the parameter has one (returns
    None then), else a gradient tensor in the weight's dtype."""
    from ..ops import cuda as K
    if K.wgrad_into_main_grad(w, dy2d, x2d):
        return None
    return K.mm_tn(dy2d, x2d).to(w.dtype)


class _AGLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, ws):
        B, T_loc, Kd = x.shape
        x2d = x.reshape(B * T_loc, Kd)
        wb = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        y = ws.ag_gemm(ws.publish(x2d), B * T_loc, T_loc, Kd, wb, False)
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(x2d, w)
        ctx.ws, ctx.dims, ctx.has_bias = ws, (B, T_loc, Kd), bias is not None
        return y.view(B, ws.W * T_loc, -1)

    @staticmethod
    def backward(ctx, dy):
        x2d, w = ctx.saved_tensors
        ws, (B, T_loc, Kd) = ctx.ws, ctx.dims
        dy2d = dy.reshape(-1, dy.shape[-1])
        dy2d = dy2d if dy2d.is_contiguous() else dy2d.contiguous()
        wb = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        dx = ws.gemm_rs(dy2d, T_loc, wb, True)                               # (dy W) reduce-scattered
        xfull = ws.gather(ws.publish(x2d), B * T_loc, T_loc, Kd)             # re-gathered, not saved
        dw = _wgrad(w, dy2d, xfull)
        db = dy2d.sum(0) if ctx.has_bias else None
        return dx.view(B, T_loc, Kd), dw, db, None


class _LinearRS(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, ws):
        B, T_full, Kd = x.shape
        T_loc = T_full // ws.W
        x2d = x.reshape(B * T_full, Kd)
        x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
        wb = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        y = ws.gemm_rs(x2d, T_loc, wb, False)
        ctx.save_for_backward(x2d, w)
        ctx.ws, ctx.dims = ws, (B, T_loc, Kd)
        return y.view(B, T_loc, -1)

    @staticmethod
    def backward(ctx, dy):
        x2d, w = ctx.saved_tensors
        ws, (B, T_loc, Kd) = ctx.ws, ctx.dims
        N = dy.shape[-1]
        dy2d = dy.reshape(B * T_loc, N)
        wb = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        pub = ws.publish(dy2d)
        dx = ws.ag_gemm(pub, B * T_loc, T_loc, N, wb, True)                  # gather(dy) W
        dyfull = ws.gather(pub, B * T_loc, T_loc, N)
        dw = _wgrad(w, dyfull, x2d)
        return dx.view(B, ws.W * T_loc, Kd), dw, None


def _tp_ok(ws, x, weight, t_loc, cols_shard) -> bool:
    return (ws is not None and x.dim() == 3 and x.dtype == torch.bfloat16 and weight.dim() == 2
            and ws.supports(x.shape[0] * t_loc, t_loc, cols_shard, weight.shape[0], weight.shape[1]))


def allgather_linear(x, weight, bias, group, dim):
    from ..dist import collectives as C
    import torch.nn.functional as F
    ws = tp_workspace(group)
    if dim == 1 and _tp_ok(ws, x, weight, x.shape[1], x.shape[2]):
        return _AGLinear.apply(x, weight, bias, ws)
    return F.linear(C.all_gather(x, group, dim=dim), weight.to(x.dtype), None if bias is None else bias.to(x.dtype))


def linear_reducescatter(x, weight, group, dim):
    from ..dist import collectives as C
    import torch.nn.functional as F
    ws = tp_workspace(group)
    if dim == 1 and x.dim() == 3 and x.shape[1] % group.size == 0 and \
            _tp_ok(ws, x, weight, x.shape[1] // group.size, weight.shape[0]):
        return _LinearRS.apply(x, weight, ws)
    return C.reduce_scatter(F.linear(x, weight.to(x.dtype)), group, dim=dim)
