"""Device mesh and process groups.

One process per GPU.  Ranks are laid out with the tensor-parallel index fastest, then the
context/sequence-parallel index, then data-parallel, then pipeline:
``rank = ((pp * DP + dp) * CP + cp) * TP + tp``.  Expert parallelism is carved out of
the combined (dp, cp) axis, as Megatron's ``parallel_state`` does for the reference
(import sites: linear_attention.py:7, moe_layer.py:19, lasp2.py:9).  Every group the
reference asks ``parallel_state`` for has a counterpart here:

==================  ==========================================================
``tp``              tensor parallel
``cp``              context parallel = LASP-2 sequence-parallel axis
``dp``              data parallel (same tp, cp, pp)
``dp_cp``           data x context: gradient reduction group of dense parameters
``pp``              pipeline
``ep``              expert parallel (subset of dp_cp)
``edp``             expert data parallel (dp_cp / ep): gradient group of expert weights
``tp_ep``           tensor x expert (all-gather dispatcher)
``mp``              model parallel (tp x pp) for global gradient-norm reductions
``world``           everything
==================  ==========================================================

A mesh can be built without ``torch.distributed`` (world size 1): all groups then have
size 1 and every collective in :mod:`collectives` is the identity.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..config.model_config import ParallelConfig


@dataclass
class Group:
    name: str
    size: int
    rank: int
    ranks: List[int]
    pg: Optional[object] = None

    @property
    def is_trivial(self) -> bool:
        return self.size == 1


class Mesh:
    def __init__(self, par: Optional[ParallelConfig] = None, world_size: Optional[int] = None,
                 rank: Optional[int] = None, create_groups: bool = True):
        self.par = par or ParallelConfig()
        if world_size is None:
            world_size = dist.get_world_size() if dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size, self.rank = world_size, rank
        tp, pp, cp, ep = self.par.tp, self.par.pp, self.par.cp, self.par.ep
        if world_size % (tp * pp * cp) != 0:
            raise ValueError(f"world size {world_size} not divisible by tp*pp*cp = {tp * pp * cp}")
        dp = world_size // (tp * pp * cp)
        if (dp * cp) % ep != 0:
            raise ValueError(f"expert parallel size {ep} must divide dp*cp = {dp * cp}")
        self.tp, self.pp, self.cp, self.dp, self.ep = tp, pp, cp, dp, ep
        self.edp = dp * cp // ep
        # coordinates of this rank
        self.tp_rank = rank % tp
        self.cp_rank = (rank // tp) % cp
        self.dp_rank = (rank // (tp * cp)) % dp
        self.pp_rank = rank // (tp * cp * dp)
        self.dpcp_rank = self.dp_rank * cp + self.cp_rank
        self.ep_rank = self.dpcp_rank % ep
        self.edp_rank = self.dpcp_rank // ep
        self.groups: Dict[str, Group] = {}
        self._build(create_groups and dist.is_initialized() and world_size > 1)

    # ------------------------------------------------------------------
    def coord_to_rank(self, pp, dp, cp, tp) -> int:
        return ((pp * self.dp + dp) * self.cp + cp) * self.tp + tp

    def _families(self) -> Dict[str, List[List[int]]]:
        tp, pp, cp, dp, ep = self.tp, self.pp, self.cp, self.dp, self.ep
        R = self.coord_to_rank
        fam: Dict[str, List[List[int]]] = {}
        fam["tp"] = [[R(p, d, c, t) for t in range(tp)] for p in range(pp) for d in range(dp) for c in range(cp)]
        fam["cp"] = [[R(p, d, c, t) for c in range(cp)] for p in range(pp) for d in range(dp) for t in range(tp)]
        fam["dp"] = [[R(p, d, c, t) for d in range(dp)] for p in range(pp) for c in range(cp) for t in range(tp)]
        fam["dp_cp"] = [[R(p, d, c, t) for d in range(dp) for c in range(cp)] for p in range(pp) for t in range(tp)]
        fam["pp"] = [[R(p, d, c, t) for p in range(pp)] for d in range(dp) for c in range(cp) for t in range(tp)]
        fam["mp"] = [[R(p, d, c, t) for p in range(pp) for t in range(tp)] for d in range(dp) for c in range(cp)]
        fam["ep"], fam["edp"], fam["tp_ep"] = [], [], []
        for p in range(pp):
            for t in range(tp):
                line = [R(p, d, c, t) for d in range(dp) for c in range(cp)]     # dp_cp line
                for s in range(0, len(line), ep):
                    fam["ep"].append(line[s:s + ep])
                for e in range(ep):
                    fam["edp"].append(line[e::ep])
            line0 = [[R(p, d, c, t) for t in range(tp)] for d in range(dp) for c in range(cp)]
            for s in range(0, len(line0), ep):
                fam["tp_ep"].append([r for blk in line0[s:s + ep] for r in blk])
        fam["world"] = [list(range(self.world_size))]
        return fam

    def _build(self, create: bool):
        timeout = datetime.timedelta(minutes=self.par.distributed_timeout_minutes)
        for name, lists in self._families().items():
            mine = None
            for ranks in lists:
                pg = None
                if create and len(ranks) > 1:
                    pg = dist.group.WORLD if len(ranks) == self.world_size else dist.new_group(ranks, timeout=timeout)
                if self.rank in ranks:
                    mine = Group(name, len(ranks), ranks.index(self.rank), ranks, pg)
            assert mine is not None, name
            self.groups[name] = mine

    def __getitem__(self, name: str) -> Group:
        return self.groups[name]

    # pipeline helpers ---------------------------------------------------
    @property
    def is_first_stage(self): return self.pp_rank == 0
    @property
    def is_last_stage(self): return self.pp_rank == self.pp - 1
    @property
    def next_stage_rank(self): return self["pp"].ranks[(self.pp_rank + 1) % self.pp]
    @property
    def prev_stage_rank(self): return self["pp"].ranks[(self.pp_rank - 1) % self.pp]

    def describe(self) -> str:
        return (f"rank {self.rank}/{self.world_size}: tp={self.tp_rank}/{self.tp} cp={self.cp_rank}/{self.cp} "
                f"dp={self.dp_rank}/{self.dp} pp={self.pp_rank}/{self.pp} ep={self.ep_rank}/{self.ep} "
                f"edp={self.edp_rank}/{self.edp}")


_SINGLE: Optional[Mesh] = None


def single_process_mesh() -> Mesh:
    """A mesh of one rank (no process groups); layers default to it."""
    global _SINGLE
    if _SINGLE is None:
        _SINGLE = Mesh(ParallelConfig(), world_size=1, rank=0, create_groups=False)
    return _SINGLE


def init_distributed(par: ParallelConfig, backend: Optional[str] = None) -> Mesh:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT / LOCAL_RANK and
    build the mesh (counterpart of initialize.py:87-146)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    backend = backend or par.distributed_backend
    if torch.cuda.is_available() and backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, world_size=world, rank=rank,
                                timeout=datetime.timedelta(minutes=par.distributed_timeout_minutes), **kw)
    return Mesh(par, world_size=world, rank=rank)
