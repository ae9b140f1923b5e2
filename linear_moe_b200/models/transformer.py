"""Layer stack and causal language model.

One model class serves every family of the reference: ``GPTModel`` (softmax attention only),
``HybridGPTModel`` with ``HybridTransformerBlock`` (``L``/``N`` patterns) and ``MambaModel`` with
``MambaStack`` (``M``/``*``/``-`` patterns) — model/qwen2/model.py, model/qwen2/hybrid/
hybrid_model.py:28-248, hybrid_transformer_block.py:87-474, sequence_modeling/ssm.py:73-250,
mamba2/mamba_model.py:16-209 — for the four backbones (qwen2, llama3, mixtral, deepseek_v2), which
differ only in configuration (attention kind, router order, shared expert, biases).

A ``Block`` is one pre-norm residual layer: optional token mixer, optional FFN
(transformer_layer.py:179-273, mamba_layer.py:27-80).  Module names follow the Megatron-Core
state-dict schema so checkpoints keep the reference's keys: ``decoder.layers.{i}.
{input_layernorm,self_attention,pre_mlp_layernorm,mlp}``, ``mixer``/``norm`` for Mamba blocks,
``decoder.final_layernorm``, ``embedding.word_embeddings``, ``output_layer``.

Pipeline parallelism: a stage builds only its slice of the layer list (including hybrid
patterns, which the reference builds in full on every stage).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint as ckpt

from .. import ops
from ..config.model_config import ModelConfig
from ..dist.mesh import Mesh, single_process_mesh
from ..parallel.tensor_parallel import LMHead, VocabParallelEmbedding
from .attention import MLASelfAttention, SelfAttention
from .layout import LayerSpec, split_for_pipeline
from .lsm_layers import LinearAttention, LinearRNN
from .mamba2 import MambaMixer
from .moe import MLP, MoELayer
from .mom import MomLinearAttention


class Norm(nn.Module):
    def __init__(self, cfg: ModelConfig, device=None):
        super().__init__()
        self.eps, self.kind = cfg.norm_eps, cfg.normalization
        self.weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=cfg.params_dtype, device=device))
        self.weight.sequence_parallel_grad = True
        if self.kind == "LayerNorm":
            self.bias = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=cfg.params_dtype, device=device))
            self.bias.sequence_parallel_grad = True

    def forward(self, x):
        if self.kind == "LayerNorm":
            return ops.layer_norm(x, self.weight, self.bias, self.eps)
        return ops.rms_norm(x, self.weight, self.eps)

    def add_norm(self, x, residual):
        """``r = x + residual``; returns ``(norm(r), r)``.  ``residual=None`` starts the stream at x."""
        if residual is None:
            return self(x), x
        if self.kind == "LayerNorm":
            return ops.add_layer_norm(x, residual, self.weight, self.bias, self.eps)
        return ops.add_rms_norm(x, residual, self.weight, self.eps)


def build_mixer(cfg: ModelConfig, spec: LayerSpec, mesh: Mesh, key: str, sp: bool, device):
    n = spec.index + 1
    if spec.mixer == "attn":
        return SelfAttention(cfg, mesh, n, key, sp, device)
    if spec.mixer == "mla":
        return MLASelfAttention(cfg, mesh, n, key, sp, device)
    if spec.mixer == "mamba":
        return MambaMixer(cfg, mesh, n, key, sp, device)
    if spec.mixer == "lsm":
        if cfg.la_module in ("hgrn2", "rwkv6", "rwkv7"):
            return LinearRNN(cfg, mesh, n, key, sp, device)
        if cfg.la_module.startswith("mom_"):
            return MomLinearAttention(cfg, mesh, n, key, sp, device)
        return LinearAttention(cfg, mesh, n, key, sp, device)
    raise ValueError(spec.mixer)


class Block(nn.Module):
    """Pre-norm residual layer.  ``forward(x, residual)`` carries the residual stream separately so the
    residual add of the previous sub-layer fuses into this sub-layer's norm."""

    def __init__(self, cfg: ModelConfig, spec: LayerSpec, mesh: Mesh, key: str, sequence_parallel: bool, device=None):
        super().__init__()
        self.cfg, self.spec = cfg, spec
        mamba_style = spec.symbol in ("M", "*", "-")
        if spec.mixer is not None:
            if mamba_style and spec.mixer == "mamba":
                self.norm = Norm(cfg, device)
                self.mixer = build_mixer(cfg, spec, mesh, key + ".mixer", sequence_parallel, device)
            else:
                self.input_layernorm = Norm(cfg, device)
                self.self_attention = build_mixer(cfg, spec, mesh, key + ".self_attention", sequence_parallel, device)
        if spec.ffn is not None:
            self.pre_mlp_layernorm = Norm(cfg, device)
            if spec.ffn == "moe":
                self.mlp = MoELayer(cfg, mesh, spec.index + 1, key + ".mlp", sequence_parallel, device)
            else:
                self.mlp = MLP(cfg, mesh, key + ".mlp", sequence_parallel=sequence_parallel, device=device)

    def _mixer(self):
        return getattr(self, "mixer", None) or getattr(self, "self_attention", None)

    def _mixer_norm(self):
        return getattr(self, "norm", None) or getattr(self, "input_layernorm", None)

    def forward(self, x, residual, cache: Optional[dict] = None, position_offset: int = 0, lower_bound=None):
        """x: output of the previous sub-layer (not yet added to the stream), residual: the stream."""
        mixer = self._mixer()
        if mixer is not None:
            h, residual = self._mixer_norm().add_norm(x, residual)
            kw = {"lower_bound": lower_bound} if lower_bound is not None else {}
            x = self._drop(mixer(h, cache=cache, position_offset=position_offset, **kw))
        if self.spec.ffn is not None:
            h, residual = self.pre_mlp_layernorm.add_norm(x, residual)
            if self.cfg.moe_layer_recompute and self.spec.ffn == "moe" and self.training:
                x = ckpt.checkpoint(self.mlp, h, use_reentrant=False)
            else:
                x = self.mlp(h)
            x = self._drop(x)
        return x, residual

    def _drop(self, x):
        """``--hidden-dropout``: on every sub-layer's output before it joins the residual stream (Megatron's
        bias-dropout-add; the add itself is fused into the next norm)."""
        p = self.cfg.hidden_dropout
        return F.dropout(x, p, True) if (p > 0.0 and self.training) else x


class CausalLM(nn.Module):
    """Embedding -> blocks -> final norm -> LM head (+ loss).

    ``forward(input_ids, labels=None, ...)`` returns per-token losses ``[B,T]`` when labels are
    given, else logits, like the reference models (hybrid_model.py:160-223).  Intermediate pipeline
    stages take/return hidden states through ``hidden_in``."""

    def __init__(self, cfg: ModelConfig, mesh: Optional[Mesh] = None, *, pre_process: bool = True,
                 post_process: bool = True, pp_rank: Optional[int] = None, vpp_rank: int = 0,
                 sequence_parallel: bool = False, device=None):
        super().__init__()
        self.cfg = cfg
        self.mesh = mesh or single_process_mesh()
        mesh = self.mesh
        self.pre_process, self.post_process = pre_process, post_process
        self.sequence_parallel = sequence_parallel and mesh.tp > 1
        all_specs = cfg.layer_types()
        pp_rank = mesh.pp_rank if pp_rank is None else pp_rank
        vpp = mesh.par.virtual_pipeline_model_parallel_size
        self.specs: List[LayerSpec] = split_for_pipeline(all_specs, mesh.pp, pp_rank, vpp, vpp_rank)
        dt, sp = cfg.params_dtype, self.sequence_parallel
        if pre_process:
            self.embedding = nn.Module()
            self.embedding.word_embeddings = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, mesh=mesh,
                                                                    std=cfg.init_method_std, sequence_parallel=sp,
                                                                    dtype=dt, device=device)
        self.decoder = nn.Module()
        self.decoder.layers = nn.ModuleList(
            [Block(cfg, s, mesh, f"decoder.layers.{s.index}", sp, device) for s in self.specs])
        if post_process:
            self.decoder.final_layernorm = Norm(cfg, device)
            tied = self.embedding.word_embeddings.weight if (cfg.tie_embeddings and pre_process) else None
            # tied weights with the embedding on another pipeline stage: this stage holds a copy drawn from the same key
            # (equal values); the optimizer sums the two copies' gradients, so both receive the same update
            split_tie = cfg.tie_embeddings and not pre_process
            self.output_layer = LMHead(cfg.hidden_size, cfg.vocab_size, mesh=mesh, std=cfg.init_method_std, tied=tied,
                                       key="embedding.word_embeddings" if split_tie else "output_layer",
                                       chunk=cfg.cross_entropy_chunk, sequence_parallel=sp, dtype=dt, device=device)
            if split_tie:
                self.output_layer.weight.pp_shared_grad = "embedding"
        if pre_process and not post_process and cfg.tie_embeddings and mesh.pp > 1:
            self.embedding.word_embeddings.weight.pp_shared_grad = "embedding"
        self.offload = None
        if cfg.cpu_offloading and cfg.cpu_offloading_num_layers > 0:
            from ..parallel.offload import ActivationOffload
            self.offload = ActivationOffload(cfg.cpu_offloading_num_layers)
        if cfg.la_module == "hgrn2" and cfg.hgrn2_lower_bound:
            self.lower_bounds = nn.Parameter(torch.zeros(len(all_specs), cfg.key_dim, dtype=dt, device=device))
            if mesh.pp > 1 or vpp:
                # every layer's bound is a cumulative softmax over ALL layers' rows: each pipeline stage (and model chunk)
                # holds the whole table and contributes the gradient of its own layers
                self.lower_bounds.pp_shared_grad = "all"

    # ------------------------------------------------------------------
    def new_cache(self) -> List[dict]:
        """One dict per local block: recurrent states / KV caches for decoding."""
        return [dict() for _ in self.decoder.layers]

    def _run_blocks(self, x, residual, caches, position_offset):
        cfg = self.cfg
        layers = self.decoder.layers
        full_recompute = cfg.recompute_granularity == "full" and self.training and caches is None
        lbs = None
        if hasattr(self, "lower_bounds"):
            lb = self.lower_bounds.float().softmax(0)
            lbs = lb.cumsum(0) - lb[0]
        ready = getattr(self, "grad_ready_hook", None)
        for i, blk in enumerate(layers):
            cache = None if caches is None else caches[i]
            lb_i = None if lbs is None else lbs[blk.spec.index]
            if ready is not None and caches is None and torch.is_grad_enabled() and x.requires_grad:
                # fires when the gradient with respect to this block's input exists, i.e. after the block's whole
                # backward: its parameter gradients are final and their reduction may start
                x.register_hook(lambda g, i=i: ready(i))
            if full_recompute and self._should_recompute(i):
                x, residual = ckpt.checkpoint(blk, x, residual, None, position_offset, lb_i, use_reentrant=False)
            elif self.offload is not None and self.training and caches is None and torch.is_grad_enabled():
                with self.offload.layer(i):
                    x, residual = blk(x, residual, cache, position_offset, lb_i)
            else:
                x, residual = blk(x, residual, cache, position_offset, lb_i)
        return x, residual

    def _should_recompute(self, i: int) -> bool:
        """``uniform``: every layer (in groups of recompute_num_layers); ``block``: the first
        recompute_num_layers layers of the stage (hybrid_transformer_block.py:262-300)."""
        cfg = self.cfg
        if cfg.recompute_method == "block":
            return i < cfg.recompute_num_layers
        return True

    def forward(self, input_ids: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None, *,
                hidden_in: Optional[torch.Tensor] = None, caches: Optional[List[dict]] = None,
                position_offset: int = 0, parallel_output: bool = False, return_hidden: bool = False):
        if self.pre_process:
            x = self.embedding.word_embeddings(input_ids)
        else:
            x = hidden_in
        residual = None
        x, residual = self._run_blocks(x, residual, caches, position_offset)
        if not self.post_process:
            return x if residual is None else x + residual
        h, _ = self.decoder.final_layernorm.add_norm(x, residual)
        if return_hidden:
            return h
        return self.output_layer(h, labels, parallel_output=parallel_output)

    # ------------------------------------------------------------------
    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())
