"""Sharded ("distributed") checkpoint format with reshard-on-load.

Every model-parallel coordinate writes the tensors it owns under their GLOBAL names together with a description of
which part of the global tensor each one is; a reader with ANY (TP, PP, EP) layout fetches, for each tensor it owns,
exactly the overlapping parts of the saved shards.  This is the role of Megatron's ``sharded_state_dict`` /
dist-checkpointing, which the reference implements per module (hybrid_transformer_block.py:434-474,
transformer/mlp.py:157-230, moe/experts.py:230-273); here the placement of a tensor follows from the same sharding
rules that ``ckpt.reshard`` uses, expressed as index lists, so one generic routine serves every module.

Layout::

    <dir>/iter_0000123/shard_tp{t}_pp{p}_ep{e}.pt      {global name: local tensor}  (+ optimizer state per parameter)
    <dir>/iter_0000123/shard_tp{t}_pp{p}_ep{e}.json    {global name: {"shape": global shape, "index": {dim: ranges}}}
    <dir>/iter_0000123/metadata.json                   layout (tp, pp, ep), iteration, file list
    <dir>/latest_sharded_iteration.txt

``index[dim]`` lists, as ``[start, stop)`` ranges in local order, the global indices along ``dim`` that the local tensor
holds (absent dims are held completely).  SwiGLU fc1 halves, the parts of Mamba's ``in_proj`` and the expert tensors
(experts along dim 0 by EP, ffn along another dim by TP) are all covered by this form.
Optimizer state (fp32 master, exp_avg, exp_avg_sq) is stored per parameter in the parameter's shape under
``optimizer.<kind>.<global name>``, so it reshards with the same index lists.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config.model_config import ModelConfig
from . import reshard as RS

TRACKER = "latest_sharded_iteration.txt"
_LAYER = re.compile(r"^decoder\.layers\.(\d+)\.(.*)$")
Index = Dict[int, torch.Tensor]


def _chunk_ids(n: int, parts: int, r: int) -> torch.Tensor:
    return torch.arange(n).chunk(parts)[r]


def index_map(name: str, global_shape, cfg: ModelConfig, tp: int, ep: int, tp_rank: int, ep_rank: int) -> Index:
    """Global indices, per split dimension, of the part of tensor ``name`` that coordinate (tp_rank, ep_rank) owns."""
    kind, arg = RS._rule(name, cfg)
    out: Index = {}
    if kind in ("w1", "w2") and ep > 1:
        out[0] = _chunk_ids(global_shape[0], ep, ep_rank)
    if tp == 1 or kind == "rep":
        return out
    if kind == "dim0":
        out[0] = _chunk_ids(global_shape[0], tp, tp_rank)
    elif kind == "dim1":
        out[1] = _chunk_ids(global_shape[1], tp, tp_rank)
    elif kind == "glu0":
        half = global_shape[0] // 2
        c = _chunk_ids(half, tp, tp_rank)
        out[0] = torch.cat([c, c + half])
    elif kind == "parts0":
        ids, off = [], 0
        for size in arg:
            ids.append(_chunk_ids(size, tp, tp_rank) + off)
            off += size
        out[0] = torch.cat(ids)
    elif kind == "w1":                                      # [E, h, 2f]: each GLU half split along the last dim
        half = global_shape[2] // 2
        c = _chunk_ids(half, tp, tp_rank)
        out[2] = torch.cat([c, c + half])
    elif kind == "w2":                                      # [E, f, h]
        out[1] = _chunk_ids(global_shape[1], tp, tp_rank)
    return out


def _global_shape(name: str, local_shape, cfg: ModelConfig, tp: int, ep: int) -> List[int]:
    kind, _ = RS._rule(name, cfg)
    g = list(local_shape)
    if kind in ("w1", "w2") and ep > 1:
        g[0] *= ep
    if tp > 1 and kind != "rep":
        dim = {"dim0": 0, "glu0": 0, "parts0": 0, "dim1": 1, "w1": 2, "w2": 1}[kind]
        g[dim] *= tp
    return g


def _to_ranges(ids: torch.Tensor) -> List[List[int]]:
    v = ids.tolist()
    out, start, prev = [], v[0], v[0]
    for x in v[1:]:
        if x != prev + 1:
            out.append([start, prev + 1])
            start = x
        prev = x
    out.append([start, prev + 1])
    return out


def _from_ranges(r) -> torch.Tensor:
    return torch.cat([torch.arange(a, b) for a, b in r])


def _global_name(name: str, layer_offset: int) -> str:
    m = _LAYER.match(name)
    return f"decoder.layers.{int(m.group(1)) + layer_offset}.{m.group(2)}" if m else name


def _shard_file(root: str, iteration: int, t: int, p: int, e: int, ext: str) -> str:
    return os.path.join(root, f"iter_{int(iteration):07d}", f"shard_tp{t}_pp{p}_ep{e}.{ext}")


def describe(local_sd: Dict[str, torch.Tensor], cfg: ModelConfig, tp: int, ep: int, tp_rank: int, ep_rank: int,
             layer_offset: int = 0) -> Tuple[Dict[str, torch.Tensor], dict]:
    """Local state dict (local layer numbering) -> (tensors under global names, their placement description)."""
    tensors, meta = {}, {}
    for k, v in local_sd.items():
        if k.endswith("_extra_state") or not torch.is_tensor(v):
            continue
        base = k
        prefix = ""
        if k.startswith("optimizer."):
            _, kind, base = k.split(".", 2)
            prefix = f"optimizer.{kind}."
        g = _global_name(base, layer_offset)
        shape = _global_shape(g, v.shape, cfg, tp, ep)
        idx = index_map(g, shape, cfg, tp, ep, tp_rank, ep_rank)
        tensors[prefix + g] = v.detach().cpu()
        meta[prefix + g] = {"shape": shape, "index": {str(d): _to_ranges(i) for d, i in idx.items()}}
    return tensors, meta


def optimizer_tensors(optimizer, group_gather=None) -> Dict[str, torch.Tensor]:
    """Per-parameter optimizer state (``optimizer.{master,exp_avg,exp_avg_sq}.<name>``) from the flat buffers.  With
    ZeRO-1 the flat shards of the data-parallel ranks are gathered first (``group_gather(t, group)`` -> full buffer)."""
    out = {}
    for b in optimizer.buffers:
        full = {}
        for kind in ("master", "exp_avg", "exp_avg_sq"):
            t = getattr(b, kind)
            if t is None:
                continue
            if t.numel() != b.numel:                       # ZeRO-1 shard
                assert group_gather is not None, "ZeRO-1 optimizer state needs the data-parallel gather"
                t = group_gather(t, b.group)
            full[kind] = t
        for s in b.slots:
            for kind, t in full.items():
                out[f"optimizer.{kind}.{s.name}"] = t[s.start:s.start + s.numel].view(s.param.shape)
    return out


def save_sharded(root: str, iteration: int, models, cfg: ModelConfig, mesh, optimizer=None, layer_offsets=None,
                 extra: Optional[dict] = None):
    """Collective.  ``layer_offsets[i]`` = global index of the first layer of model chunk ``i`` on this stage (default:
    contiguous split of ``cfg.num_layers`` over the pipeline stages)."""
    from ..dist import collectives as C
    os.makedirs(os.path.join(root, f"iter_{int(iteration):07d}"), exist_ok=True)
    tensors, meta = {}, {}
    for i, m in enumerate(models):
        inner = getattr(m, "module", m)
        if layer_offsets is not None:
            off = layer_offsets[i]
        else:
            n_local = RS.num_layer_entries(inner.state_dict())
            off = mesh.pp_rank * n_local
        sd = dict(inner.state_dict())
        if optimizer is not None and i == 0:
            names = {n for n, _ in inner.named_parameters()}
            opt = optimizer_tensors(optimizer, lambda t, g: C.all_gather_raw(t.contiguous(), g, dim=0))
            sd.update({k: v for k, v in opt.items() if k.split(".", 2)[2] in names or len(models) == 1})
        t_, m_ = describe(sd, cfg, mesh.tp, mesh.ep, mesh.tp_rank, mesh.ep_rank, off)
        tensors.update(t_)
        meta.update(m_)
    if mesh.edp_rank == 0:
        f = _shard_file(root, iteration, mesh.tp_rank, mesh.pp_rank, mesh.ep_rank, "pt")
        torch.save(tensors, f + ".tmp")
        os.replace(f + ".tmp", f)
        with open(_shard_file(root, iteration, mesh.tp_rank, mesh.pp_rank, mesh.ep_rank, "json"), "w") as fh:
            json.dump(meta, fh)
    if dist.is_initialized():
        dist.barrier()
    if mesh.rank == 0:
        info = {"iteration": int(iteration), "tp": mesh.tp, "pp": mesh.pp, "ep": mesh.ep,
                "step": None if optimizer is None else optimizer.step_count, "extra": extra or {}}
        with open(os.path.join(root, f"iter_{int(iteration):07d}", "metadata.json"), "w") as fh:
            json.dump(info, fh)
        with open(os.path.join(root, TRACKER), "w") as fh:
            fh.write(str(int(iteration)))


def _scatter_block(dst: torch.Tensor, sel: Index, block: torch.Tensor):
    """``dst[outer product of sel[d] over the dims in sel] = block`` (dims not in ``sel`` are taken whole)."""
    dims = sorted(sel)
    if not dims:
        dst.copy_(block)
    elif len(dims) == 1:
        dst.index_copy_(dims[0], sel[dims[0]], block)
    else:
        d0 = dims[0]
        tmp = dst.index_select(d0, sel[d0])
        _scatter_block(tmp, {d: sel[d] for d in dims[1:]}, block)
        dst.index_copy_(d0, sel[d0], tmp)


class ShardReader:
    """Fetches any part of any saved tensor from the shard files of one iteration (files are memory-mapped)."""

    def __init__(self, root: str, iteration: Optional[int] = None):
        if iteration is None:
            iteration = int(open(os.path.join(root, TRACKER)).read().strip())
        self.dir = os.path.join(root, f"iter_{int(iteration):07d}")
        self.info = json.load(open(os.path.join(self.dir, "metadata.json")))
        self.metas: Dict[str, dict] = {}
        for f in sorted(os.listdir(self.dir)):
            if f.startswith("shard_") and f.endswith(".json"):
                self.metas[f[:-5]] = json.load(open(os.path.join(self.dir, f)))
        self._files: Dict[str, dict] = {}

    def _tensors(self, stem: str) -> dict:
        if stem not in self._files:
            self._files[stem] = torch.load(os.path.join(self.dir, stem + ".pt"), map_location="cpu", mmap=True,
                                           weights_only=True)
        return self._files[stem]

    def has(self, name: str) -> bool:
        return any(name in m for m in self.metas.values())

    def read(self, name: str, want: Index, local_shape) -> torch.Tensor:
        """The part of global tensor ``name`` selected by ``want`` (global indices per split dim, local order)."""
        out, filled = None, None
        for stem, meta in self.metas.items():
            if name not in meta:
                continue
            ent = meta[name]
            gshape = ent["shape"]
            have = {int(d): _from_ranges(r) for d, r in ent["index"].items()}
            dst_sel, src_sel, empty = {}, {}, False
            for d in set(want) | set(have):
                w = want.get(d, torch.arange(gshape[d]))
                h = have.get(d, torch.arange(gshape[d]))
                pos = torch.full((gshape[d],), -1, dtype=torch.long)
                pos[h] = torch.arange(h.numel())
                sel = pos[w]
                mask = sel >= 0
                if not bool(mask.any()):
                    empty = True
                    break
                dst_sel[d], src_sel[d] = mask.nonzero().flatten(), sel[mask]
            if empty:
                continue
            src = self._tensors(stem)[name]
            if out is None:
                out = torch.empty(tuple(local_shape), dtype=src.dtype)
                filled = torch.zeros(tuple(local_shape), dtype=torch.bool)
            part = src
            for d, sidx in src_sel.items():
                part = part.index_select(d, sidx)
            _scatter_block(out, dst_sel, part)
            _scatter_block(filled, dst_sel, torch.ones(part.shape, dtype=torch.bool))
            if bool(filled.all()):
                break
        if out is None or not bool(filled.all()):
            raise KeyError(f"sharded checkpoint does not cover all of {name}")
        return out


def load_sharded(root: str, models, cfg: ModelConfig, mesh, optimizer=None, iteration: Optional[int] = None,
                 layer_offsets=None, strict: bool = True, return_extra: bool = False):
    """Load into ``models`` (and ``optimizer``) under the CURRENT layout, whatever layout wrote the checkpoint.
    Returns the iteration."""
    rd = ShardReader(root, iteration)
    for i, m in enumerate(models):
        inner = getattr(m, "module", m)
        own = inner.state_dict()
        off = layer_offsets[i] if layer_offsets is not None else mesh.pp_rank * RS.num_layer_entries(own)
        new = {}
        for k, v in own.items():
            if k.endswith("_extra_state") or not torch.is_tensor(v):
                continue
            g = _global_name(k, off)
            if not rd.has(g):
                if strict:
                    raise KeyError(f"{g} is not in the checkpoint")
                continue
            gshape = _global_shape(g, v.shape, cfg, mesh.tp, mesh.ep)
            want = index_map(g, gshape, cfg, mesh.tp, mesh.ep, mesh.tp_rank, mesh.ep_rank)
            new[k] = rd.read(g, want, v.shape).to(v.dtype)
        inner.load_state_dict(new, strict=False)
        if optimizer is not None and i == 0:
            _load_optimizer(rd, optimizer, cfg, mesh, off)
    if return_extra:
        return int(rd.info["iteration"]), rd.info.get("extra", {})
    return int(rd.info["iteration"])


def _load_optimizer(rd: ShardReader, optimizer, cfg, mesh, layer_offset: int):
    loaded = False
    for b in optimizer.buffers:
        lo, hi = b.shard
        for kind in ("master", "exp_avg", "exp_avg_sq"):
            dst = getattr(b, kind)
            if dst is None:
                continue
            for s in b.slots:
                g = _global_name(s.name, layer_offset)
                key = f"optimizer.{kind}.{g}"
                if not rd.has(key):
                    continue
                gshape = _global_shape(g, s.param.shape, cfg, mesh.tp, mesh.ep)
                want = index_map(g, gshape, cfg, mesh.tp, mesh.ep, mesh.tp_rank, mesh.ep_rank)
                flat = rd.read(key, want, s.param.shape).reshape(-1).to(dst.dtype)
                a, z = max(s.start, lo), min(s.start + s.numel, hi)       # overlap of the slot with this rank's shard
                if a < z:
                    dst[a - lo:z - lo].copy_(flat[a - s.start:z - s.start])
                    loaded = True
    if loaded:
        if rd.info.get("step") is not None:
            optimizer.step_count = rd.info["step"]
        optimizer.state_loaded = True
