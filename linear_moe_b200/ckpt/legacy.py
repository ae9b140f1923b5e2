"""Megatron legacy checkpoint layout: writer and reader.

On-disk contract the reference's convertors read and write
(toolkits/model_checkpoints_convertor/qwen/hf2mcore_qwen2_dense_and_moe_gqa.py:104-262,444-473;
mistral/hf2mcore_mixtral.py:214-218)::

    <dir>/latest_checkpointed_iteration.txt            "release" or the iteration number
    <dir>/{release | iter_0000123}/mp_rank_{tp:02d}[_{pp:03d}][_{ep:03d}]/model_optim_rng.pt

with payload ``{'args', 'checkpoint_version': 3.0, 'iteration', 'model': state_dict, ...}`` plus
``optimizer`` / ``opt_param_scheduler`` / ``rng_state`` when training.  State-dict keys follow the
Megatron-Core schema; the grouped expert tensors of this framework are written under the
reference's per-expert keys ``mlp.experts.local_experts.{e}.linear_fc1/linear_fc2.weight``.

Only data-parallel rank 0 of each model-parallel coordinate writes model weights; under ZeRO-1
every data-parallel rank writes its optimizer shard next to it.  ``async_save`` hands the CPU copy
to a writer thread; the tracker file of such a save is published by :func:`finalize_async_saves` once every rank's
files are on disk.
"""
from __future__ import annotations

import os
import random
import threading
from argparse import Namespace
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..dist.mesh import Mesh

TRACKER = "latest_checkpointed_iteration.txt"
_WRITERS: List[threading.Thread] = []
_WRITER_ERRORS: List[BaseException] = []
_PENDING_TRACKERS: List[Tuple[str, str, bool]] = []      # (root, text, this rank writes it) of async saves not yet finalized


def checkpoint_name(root: str, iteration, release: bool, tp_rank: int, pp_rank: int, ep_rank: int,
                    pp: int, ep: int, filename: str = "model_optim_rng.pt") -> str:
    directory = "release" if release else f"iter_{int(iteration):07d}"
    name = f"mp_rank_{tp_rank:02d}"
    if pp > 1:
        name += f"_{pp_rank:03d}"
    if ep > 1:
        name += f"_{ep_rank:03d}"
    return os.path.join(root, directory, name, filename)


def read_tracker(root: str) -> Tuple[Optional[int], bool]:
    p = os.path.join(root, TRACKER)
    if not os.path.isfile(p):
        return None, False
    s = open(p).read().strip()
    if s == "release":
        return 0, True
    return int(s), False


def read_checkpoint_args(root: str) -> Optional[Namespace]:
    """The ``args`` namespace stored in the latest checkpoint under ``root`` (``--use-checkpoint-args``), read from the
    first model-parallel file; None when there is no checkpoint."""
    import glob
    import json
    it, release = read_tracker(root)
    if it is None:
        # the sharded format keeps the model fields in its metadata file
        tracker = os.path.join(root, "latest_sharded_iteration.txt")
        if os.path.isfile(tracker):
            meta = os.path.join(root, f"iter_{int(open(tracker).read().strip()):07d}", "metadata.json")
            stored = json.load(open(meta)).get("extra", {}).get("model_args")
            return None if stored is None else Namespace(**stored)
        return None
    directory = os.path.join(root, "release" if release else f"iter_{int(it):07d}")
    files = sorted(glob.glob(os.path.join(directory, "mp_rank_*", "model_optim_rng.pt")))
    if not files:
        return None
    ck = torch.load(files[0], map_location="cpu", weights_only=False)
    return ck.get("args")


# ---- expert key translation ------------------------------------------------
def to_reference_keys(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """``...experts.weight1 [E,h,2f]`` / ``weight2 [E,f,h]`` -> per-expert ``linear_fc1 [2f,h]`` /
    ``linear_fc2 [h,f]`` keys."""
    out = {}
    for k, v in sd.items():
        if k.endswith(".experts.weight1"):
            base = k[: -len("weight1")]
            for e in range(v.shape[0]):
                out[f"{base}local_experts.{e}.linear_fc1.weight"] = v[e].t().contiguous()
        elif k.endswith(".experts.weight2"):
            base = k[: -len("weight2")]
            for e in range(v.shape[0]):
                out[f"{base}local_experts.{e}.linear_fc2.weight"] = v[e].t().contiguous()
        else:
            out[k] = v
    return out


def from_reference_keys(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out, fc1, fc2 = {}, {}, {}
    for k, v in sd.items():
        if ".experts.local_experts." in k:
            base, rest = k.split(".experts.local_experts.")
            e, tail = rest.split(".", 1)
            (fc1 if tail.startswith("linear_fc1") else fc2).setdefault(base, {})[int(e)] = v
        elif k.endswith("._extra_state"):
            continue
        elif k.endswith(".linear_qkv.layer_norm_weight") or k.endswith(".linear_q_proj.layer_norm_weight"):
            # TransformerEngine-style fused norm + linear modules carry the pre-norm weight on the linear
            # (written by the reference's convertors when use_te): it is this framework's input_layernorm
            out[k.rsplit(".self_attention.", 1)[0] + ".input_layernorm.weight"] = v
        elif k.endswith(".mlp.linear_fc1.layer_norm_weight"):
            out[k[: -len(".mlp.linear_fc1.layer_norm_weight")] + ".pre_mlp_layernorm.weight"] = v
        else:
            out[k] = v
    for base, d in fc1.items():
        out[f"{base}.experts.weight1"] = torch.stack([d[e].t() for e in sorted(d)]).contiguous()
    for base, d in fc2.items():
        out[f"{base}.experts.weight2"] = torch.stack([d[e].t() for e in sorted(d)]).contiguous()
    return out


def _rng_state() -> dict:
    st = {"random_rng_state": random.getstate(), "np_rng_state": np.random.get_state(),
          "torch_rng_state": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda_rng_state"] = torch.cuda.get_rng_state()
    return st


def _set_rng_state(st: dict):
    random.setstate(st["random_rng_state"])
    np.random.set_state(st["np_rng_state"])
    torch.set_rng_state(st["torch_rng_state"])
    if torch.cuda.is_available() and "cuda_rng_state" in st:
        torch.cuda.set_rng_state(st["cuda_rng_state"])


def _args_namespace(cfg, par, tc, consumed_samples: int) -> Namespace:
    ns = Namespace()
    for obj in (cfg, par, tc):
        for k, v in vars(obj).items():
            setattr(ns, k, v if not isinstance(v, torch.dtype) else str(v))
    ns.consumed_train_samples = consumed_samples
    ns.padded_vocab_size = cfg.vocab_size
    return ns


def _write(obj, path: str):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def save_checkpoint(root: str, iteration, models, optimizer, scheduler, cfg, par, tc, mesh: Mesh,
                    consumed_samples: int = 0, release: bool = False):
    """Write this rank's share of the checkpoint and (rank 0, after a barrier) the tracker file."""
    finalize_async_saves()                                   # an earlier asynchronous save completes first
    os.makedirs(root, exist_ok=True)
    path = checkpoint_name(root, iteration, release, mesh.tp_rank, mesh.pp_rank, mesh.ep_rank, mesh.pp, mesh.ep)
    write_model = mesh.edp_rank == 0          # one writer per (tp, pp, ep) coordinate
    payload = None
    if write_model:
        payload = {"args": _args_namespace(cfg, par, tc, consumed_samples), "checkpoint_version": 3.0,
                   "iteration": iteration}
        for i, m in enumerate(models):
            sd = {k: v.detach().cpu() for k, v in m.state_dict().items()}
            payload["model" if len(models) == 1 else f"model{i}"] = to_reference_keys(sd)
        if optimizer is not None and not tc.no_save_optim and not optimizer.zero1:
            payload["optimizer"] = optimizer.state_dict()
        if scheduler is not None:
            payload["opt_param_scheduler"] = scheduler.state_dict()
    if not tc.no_save_rng:
        # one RNG state per expert-data-parallel rank of this model-parallel coordinate (the data-parallel ranks run
        # with different seeds; restoring rank 0's state everywhere would collapse them)
        states = [_rng_state()]
        g = mesh["edp"]
        if dist.is_initialized() and not g.is_trivial:
            states = [None] * g.size
            dist.all_gather_object(states, _rng_state(), group=g.pg)
        if payload is not None:
            payload["rng_state"] = states
    jobs = []
    if payload is not None:
        jobs.append((payload, path))
    if optimizer is not None and optimizer.zero1 and not tc.no_save_optim:
        jobs.append((optimizer.state_dict(), path.replace("model_optim_rng.pt", f"distrib_optim_{mesh.dpcp_rank:03d}.pt")))
    text = "release" if release else str(int(iteration))
    if getattr(tc, "async_save", False):
        # the tracker of this save is written by finalize_async_saves(): at the start of the next save or at the end
        # of training, after every rank has joined its writers, so it never names files that are still being written
        def work():
            try:
                for o, p in jobs:
                    _write(o, p)
            except BaseException as e:                      # surfaced by finalize_async_saves()
                _WRITER_ERRORS.append(e)
        t = threading.Thread(target=work, daemon=False)
        t.start()
        _WRITERS.append(t)
        _PENDING_TRACKERS.append((root, text, mesh.rank == 0))
        return
    for o, p in jobs:
        _write(o, p)
    if dist.is_initialized():
        dist.barrier()
    if mesh.rank == 0:
        with open(os.path.join(root, TRACKER), "w") as f:
            f.write(text)


def finalize_async_saves():
    """Collective: join this rank's writer threads, meet the other ranks, then let rank 0 publish the tracker files of
    the saves that completed.  A writer's failure is raised here (on its rank) before any tracker is written."""
    while _WRITERS:
        _WRITERS.pop().join()
    failed = 1 if _WRITER_ERRORS else 0
    if dist.is_initialized() and _PENDING_TRACKERS:
        flags = [None] * dist.get_world_size()
        dist.all_gather_object(flags, failed)
        failed_any = any(flags)
    else:
        failed_any = bool(failed)
    pending = list(_PENDING_TRACKERS)
    _PENDING_TRACKERS.clear()
    if _WRITER_ERRORS:
        e = _WRITER_ERRORS[0]
        _WRITER_ERRORS.clear()
        raise RuntimeError("asynchronous checkpoint write failed") from e
    if failed_any:
        raise RuntimeError("asynchronous checkpoint write failed on another rank; tracker not updated")
    for root, text, mine in pending:
        if mine:
            with open(os.path.join(root, TRACKER), "w") as f:
                f.write(text)


def wait_for_async_saves():
    finalize_async_saves()


def load_checkpoint(root: str, models, optimizer, scheduler, mesh: Mesh, load_rng: bool = True,
                    strict: bool = True) -> Tuple[int, int]:
    """Load into ``models`` (and optimizer/scheduler/RNG if given).  Returns (iteration, consumed samples)."""
    it, release = read_tracker(root)
    if it is None:
        raise FileNotFoundError(f"no {TRACKER} under {root}")
    path = checkpoint_name(root, it, release, mesh.tp_rank, mesh.pp_rank, mesh.ep_rank, mesh.pp, mesh.ep)
    ck = torch.load(path, map_location="cpu", weights_only=False)
    for i, m in enumerate(models):
        key = "model" if len(models) == 1 else f"model{i}"
        sd = from_reference_keys(ck[key])
        own = m.state_dict()
        sd = {k: v for k, v in sd.items() if k in own or strict}
        missing, unexpected = m.load_state_dict(sd, strict=False)
        missing = [k for k in missing if not k.endswith("_extra_state")]
        if strict and (missing or unexpected):
            raise KeyError(f"checkpoint mismatch: missing {missing[:5]}, unexpected {unexpected[:5]}")
    if optimizer is not None:
        optimizer.state_loaded = False                       # read by Trainer.load: restored masters must not be re-derived
        if optimizer.zero1:
            p = path.replace("model_optim_rng.pt", f"distrib_optim_{mesh.dpcp_rank:03d}.pt")
            if os.path.isfile(p):
                optimizer.load_state_dict(torch.load(p, map_location="cpu", weights_only=False))
                optimizer.state_loaded = True
        elif "optimizer" in ck:
            optimizer.load_state_dict(ck["optimizer"])
            optimizer.state_loaded = True
    if scheduler is not None and "opt_param_scheduler" in ck:
        scheduler.load_state_dict(ck["opt_param_scheduler"])
    if load_rng and "rng_state" in ck:
        states = ck["rng_state"]
        _set_rng_state(states[mesh.edp_rank] if mesh.edp_rank < len(states) else states[0])
    consumed = getattr(ck.get("args", Namespace()), "consumed_train_samples", 0)
    return (0 if release else int(ck.get("iteration", it))), int(consumed)
