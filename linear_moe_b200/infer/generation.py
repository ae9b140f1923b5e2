"""Text generation: sampling loop, scoring, beam search, file-driven predictor.

Reference: linear_moe/generation/api.py:25-317 (``generate_and_post_process``, ``generate``, ``beam_search``),
generation/generation.py:31-516 (token loop with repetition penalty, top-k / top-p sampling, early termination,
log-prob scoring, beam search with length penalty), generation/tokenization.py:70-120 (prompt batch building),
generation/gpt_predictor.py:27-104 (reads prompts from a file, writes completions).

Decoding is incremental for every token mixer: softmax layers keep a KV cache, linear layers keep their O(1)
recurrent state (and conv / token-shift tails), so one decode step costs the same at any context length —
the reference re-runs its chunk kernels over the growing prefix for linear layers
(linear_attention.py:260-342).  Prompts of different lengths are handled like the reference: generation
starts at the shortest prompt and prompt tokens override samples until each prompt is consumed.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import parallel_forward as PF


def modify_logits_for_top_k(logits: torch.Tensor, k: int) -> torch.Tensor:
    kth = torch.topk(logits, k, dim=-1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def modify_logits_for_top_p(logits: torch.Tensor, p: float) -> torch.Tensor:
    sorted_logits, idx = torch.sort(logits, descending=True, dim=-1)
    cum = torch.softmax(sorted_logits, dim=-1).cumsum(-1)
    remove = cum > p
    remove[..., 1:] = remove[..., :-1].clone()
    remove[..., 0] = False
    mask = torch.zeros_like(remove).scatter(-1, idx, remove)
    return logits.masked_fill(mask, float("-inf"))


def sample(logits: torch.Tensor, top_k: int = 0, top_p: float = 0.0, temperature: float = 1.0,
           vocab_size: Optional[int] = None, generator=None) -> torch.Tensor:
    """Greedy when ``top_k == 1`` (or no sampling parameter is set with temperature 0); otherwise temperature,
    then top-k or top-p filtering, then a multinomial draw."""
    assert not (top_k > 0 and top_p > 0.0), "top-k and top-p are mutually exclusive"
    if top_k == 1 or temperature == 0.0:
        out = logits.argmax(-1)
    else:
        logits = logits.float()
        if temperature != 1.0:
            logits = logits / temperature
        if top_k > 1:
            logits = modify_logits_for_top_k(logits, top_k)
        elif top_p > 0.0:
            logits = modify_logits_for_top_p(logits, top_p)
        out = torch.multinomial(torch.softmax(logits, -1), 1, generator=generator).squeeze(-1)
    if vocab_size:
        out = out.clamp(0, vocab_size - 1)
    return out


def apply_repetition_penalty(logits: torch.Tensor, tokens: torch.Tensor, penalty: float) -> torch.Tensor:
    if penalty == 1.0:
        return logits
    score = torch.gather(logits, 1, tokens)
    score = torch.where(score < 0, score * penalty, score / penalty)
    return logits.scatter(1, tokens, score)


def tokenize_prompts(tokenizer, prompts: Sequence[str], tokens_to_generate: int, add_bos: bool = False, device=None):
    """Pad prompts to ``max prompt length + tokens_to_generate`` with the eod token; returns (tokens, lengths)."""
    ids = [tokenizer.encode(p) for p in prompts]
    if add_bos and getattr(tokenizer, "bos_token_id", None) is not None:
        ids = [[tokenizer.bos_token_id] + x for x in ids]
    lengths = [len(x) for x in ids]
    total = max(lengths) + tokens_to_generate
    pad = tokenizer.eod if getattr(tokenizer, "eod", None) is not None else 0
    toks = torch.full((len(ids), total), pad, dtype=torch.long, device=device)
    for i, x in enumerate(ids):
        toks[i, : len(x)] = torch.tensor(x, dtype=torch.long)
    return toks, torch.tensor(lengths, dtype=torch.long, device=device)


@torch.no_grad()
def score_tokens(model, tokens: torch.Tensor) -> torch.Tensor:
    """Log-probability of every token given its prefix (``score_and_return_on_first_stage``); with pipeline parallelism
    the last stage computes them and every stage receives them."""
    logits = PF.stage_forward(model, tokens[:, :-1])
    out = None
    if logits is not None:
        lp = F.log_softmax(logits.float(), dim=-1)
        out = torch.gather(lp, 2, tokens[:, 1:, None]).squeeze(-1)
    B, T = tokens.shape
    return PF.broadcast_from_last_stage(model, out, (B, T - 1), torch.float32, tokens.device)


class GraphedDecodeStep:
    """One-token decode step replayed from a CUDA graph.

    A decode step of a linear-sequence model is a few hundred small launches (norms, projections of one token, state
    updates) that the host cannot issue as fast as the GPU runs them.  Models whose every cache entry has a fixed size
    (all mixers linear sequence models or Mamba2: O(1) recurrent state, no growing KV cache) make the step static, so it
    is captured once and replayed: the token is copied into a static buffer, the graph runs the whole forward, and the
    new states are copied back over the state buffers the graph reads.  Softmax-attention layers (KV cache grows by one
    row per token) are not supported and fall back to eager decoding."""

    def __init__(self, model, caches: List[dict], batch: int, device):
        self.model, self.caches = model, caches
        self.tok = torch.zeros(batch, 1, dtype=torch.long, device=device)
        self.graph: Optional["torch.cuda.CUDAGraph"] = None
        self.logits: Optional[torch.Tensor] = None
        self.failed = False                                    # the step could not be captured: eager from then on

    @staticmethod
    def supported(model, caches: List[dict], device) -> bool:
        if device.type != "cuda" or model.mesh.world_size != 1 or not caches:     # graph replay is a one-process path
            return False
        if any(s.mixer in ("attn", "mla") for s in model.specs):              # KV caches grow with every token
            return False
        return all(all(torch.is_tensor(v) for v in c.values()) for c in caches)   # nested caches (MoM) decode eagerly

    def _capture(self) -> bool:
        static = [dict(c) for c in self.caches]                # the state tensors the graph will read and update
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph):
                self.logits = self.model(self.tok, caches=self.caches, position_offset=0)
                for c, st in zip(self.caches, static):        # forward rebinds every entry to a new tensor
                    for k, v in st.items():
                        v.copy_(c[k])
                        c[k] = v
        except Exception:
            # a layer that synchronises with the host (e.g. an expert dispatch that reads token counts) cannot be
            # captured: put the states back as they were and decode eagerly from here on
            for c, st in zip(self.caches, static):
                c.clear()
                c.update(st)
            torch.cuda.synchronize()
            self.failed = True
            return False
        self.graph = graph
        return True

    def __call__(self, tok: torch.Tensor) -> torch.Tensor:
        if not self.failed and self.graph is None:
            self.tok.copy_(tok)
            self._capture()                                    # capturing records the step without running it
        if self.failed:
            return self.model(tok, caches=self.caches, position_offset=0)
        self.tok.copy_(tok)
        self.graph.replay()
        return self.logits


@torch.no_grad()
def generate_tokens(model, tokens: torch.Tensor, lengths: torch.Tensor, *, eod: Optional[int] = None, top_k: int = 0,
                    top_p: float = 0.0, temperature: float = 1.0, repetition_penalty: float = 1.0,
                    return_log_probs: bool = False, use_eod_for_early_termination: bool = True,
                    stop_on_double_eol: bool = False, stop_on_eol: bool = False, generator=None,
                    cuda_graph: bool = False) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """Fill ``tokens [B, L]`` from the shortest prompt length to L.  Returns (tokens, generated lengths, log-probs).
    ``cuda_graph``: replay the one-token steps from a CUDA graph (``GraphedDecodeStep``) when the model allows it; the
    prefill and the first two one-token steps run eagerly (they also serve as the warm-up before the capture)."""
    model.eval()
    B, L = tokens.shape
    min_len = int(lengths.min())
    caches = model.new_cache()
    done = torch.zeros(B, dtype=torch.bool, device=tokens.device)
    gen_len = torch.full((B,), L, dtype=torch.long, device=tokens.device)
    logps = torch.zeros(B, L - 1, dtype=torch.float32, device=tokens.device) if return_log_probs else None
    prev = 0
    graphed, single_steps = None, 0
    for ctx in range(min_len, L):
        if ctx - prev == 1:
            single_steps += 1
        if cuda_graph and ctx - prev == 1 and single_steps > 2:
            if graphed is None and GraphedDecodeStep.supported(model, caches, tokens.device):
                graphed = GraphedDecodeStep(model, caches, B, tokens.device)
            cuda_graph = graphed is not None
        if graphed is not None and ctx - prev == 1:
            logits = graphed(tokens[:, prev:ctx])
        else:
            # prefill once, then 1 token; under pipeline parallelism every stage runs its layers with its own caches
            logits = PF.stage_forward(model, tokens[:, prev:ctx], caches, prev)
        new = None
        if logits is not None:                                # last pipeline stage (or no pipeline): sample here
            last = logits[:, -1].float()
            last = apply_repetition_penalty(last, tokens[:, :ctx], repetition_penalty)
            new = sample(last, top_k, top_p, temperature, model.cfg.vocab_size, generator)
        # every stage gets the sampled tokens, so token buffers and termination flags stay identical on all of them
        new = PF.broadcast_from_last_stage(model, new, (B,), torch.long, tokens.device)
        started = lengths <= ctx
        tokens[:, ctx] = torch.where(started, new, tokens[:, ctx])
        if return_log_probs and logits is not None:           # after the write, so position ctx holds its final token
            lp = F.log_softmax(logits.float(), -1)
            tgt = tokens[:, prev + 1:ctx + 1]
            logps[:, prev:ctx] = torch.gather(lp, 2, tgt[..., None]).squeeze(-1)
        if eod is not None and use_eod_for_early_termination:
            hit = (tokens[:, ctx] == eod) & started
            gen_len = torch.where(hit & ~done, torch.full_like(gen_len, ctx + 1), gen_len)
            done |= hit
            if bool(done.all()):
                tokens = tokens[:, : ctx + 1]
                break
        prev = ctx
    if return_log_probs:
        logps = PF.broadcast_from_last_stage(model, logps, tuple(logps.shape), torch.float32, tokens.device)
    return tokens, gen_len, logps


@dataclass
class BeamHypotheses:
    num_beams: int
    length_penalty: float = 1.0
    beams: List[Tuple[float, torch.Tensor]] = field(default_factory=list)
    worst: float = 1e9

    def add(self, hyp: torch.Tensor, sum_logprobs: float, length: int):
        score = sum_logprobs / (length ** self.length_penalty)
        if len(self.beams) < self.num_beams or score > self.worst:
            self.beams.append((score, hyp))
            if len(self.beams) > self.num_beams:
                self.beams.sort(key=lambda x: x[0])
                self.beams.pop(0)
            self.worst = min(s for s, _ in self.beams)

    def is_done(self, best_sum_logprobs: float, cur_len: int) -> bool:
        if len(self.beams) < self.num_beams:
            return False
        return self.worst >= best_sum_logprobs / (cur_len ** self.length_penalty)


@torch.no_grad()
def beam_search(model, prompt: torch.Tensor, beam_size: int, max_new_tokens: int, eod: int, length_penalty: float = 1.0,
                num_return: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Beam search for one prompt ``[1, P]`` (``beam_search_and_return_on_first_stage``).  The whole beam is re-scored
    from its tokens each step (beams reorder, so per-beam recurrent caches are not reused)."""
    model.eval()
    device = prompt.device
    P = prompt.shape[1]
    beams = prompt.repeat(beam_size, 1)
    scores = torch.zeros(beam_size, device=device)
    scores[1:] = -1e9                                   # all beams start identical: keep one alive
    hyps = BeamHypotheses(beam_size, length_penalty)
    for step in range(max_new_tokens):
        logits = PF.full_logits(model, beams, last_only=True)[:, -1]
        lp = F.log_softmax(logits, -1)
        V = lp.shape[-1]
        cand = (scores[:, None] + lp).reshape(-1)
        top_s, top_i = torch.topk(cand, 2 * beam_size)
        b_idx, t_idx = top_i // V, top_i % V
        next_b, next_t, next_s = [], [], []
        for s, b, t in zip(top_s.tolist(), b_idx.tolist(), t_idx.tolist()):
            if t == eod:
                hyps.add(torch.cat([beams[b], torch.tensor([t], device=device)]), s, beams.shape[1] + 1 - P)
            else:
                next_b.append(b), next_t.append(t), next_s.append(s)
            if len(next_b) == beam_size:
                break
        if hyps.is_done(max(next_s) if next_s else -1e9, beams.shape[1] + 1 - P) or not next_b:
            break
        beams = torch.cat([beams[next_b], torch.tensor(next_t, device=device)[:, None]], dim=1)
        scores = torch.tensor(next_s, device=device)
    for b in range(beams.shape[0]):
        hyps.add(beams[b], float(scores[b]), beams.shape[1] - P)
    best = sorted(hyps.beams, key=lambda x: x[0], reverse=True)[:num_return]
    L = max(h.shape[0] for _, h in best)
    out = torch.full((len(best), L), eod, dtype=torch.long, device=device)
    for i, (_, h) in enumerate(best):
        out[i, : h.shape[0]] = h
    return out, torch.tensor([s for s, _ in best], device=device)


def generate_and_post_process(model, tokenizer, prompts: Sequence[str], tokens_to_generate: int = 64, *,
                              return_output_log_probs: bool = False, top_k_sampling: int = 0, top_p_sampling: float = 0.0,
                              temperature: float = 1.0, add_BOS: bool = False, use_eod_token_for_early_termination: bool = True,
                              repetition_penalty: float = 1.0, random_seed: int = -1, device=None,
                              cuda_graph: bool = False):
    """Strings in, strings out (api.py:25-111): returns (texts, token lists, log-probs or None)."""
    device = device or next(model.parameters()).device
    gen = None
    if random_seed >= 0:
        gen = torch.Generator(device=device).manual_seed(random_seed)
    tokens, lengths = tokenize_prompts(tokenizer, prompts, tokens_to_generate, add_BOS, device)
    if tokens_to_generate == 0:
        lp = score_tokens(model, tokens)
        return list(prompts), [t.tolist() for t in tokens], lp
    tokens, gen_len, lp = generate_tokens(model, tokens, lengths, eod=getattr(tokenizer, "eod", None), top_k=top_k_sampling,
                                          top_p=top_p_sampling, temperature=temperature,
                                          repetition_penalty=repetition_penalty, return_log_probs=return_output_log_probs,
                                          use_eod_for_early_termination=use_eod_token_for_early_termination, generator=gen,
                                          cuda_graph=cuda_graph)
    out_tokens = [tokens[i, : int(gen_len[i])].tolist() for i in range(tokens.shape[0])]
    texts = [tokenizer.decode(t) for t in out_tokens]
    return texts, out_tokens, lp


class GPTPredictor:
    """Prompts from ``--text-generate-input-file`` (one json or plain line per prompt) -> completions appended to
    ``--text-generate-output-file`` (gpt_predictor.py:27-104)."""

    def __init__(self, model, tokenizer, args):
        self.model, self.tok, self.args = model, tokenizer, args

    def predict(self):
        a = self.args
        with open(a.text_generate_input_file, "r", encoding="utf-8") as f:
            lines = [l.strip() for l in f if l.strip()]
        prompts = []
        for l in lines:
            try:
                row = json.loads(l)
                prompts.append(row.get("query", row.get("prompt", row.get("text", l))) if isinstance(row, dict) else l)
            except json.JSONDecodeError:
                prompts.append(l)
        outs = []
        for p in prompts:
            texts, _, _ = generate_and_post_process(self.model, self.tok, [p], tokens_to_generate=a.out_seq_length,
                                                    top_k_sampling=a.top_k, top_p_sampling=a.top_p,
                                                    temperature=a.temperature, repetition_penalty=a.repetition_penalty,
                                                    cuda_graph=getattr(a, "cuda_graph_decode", False))
            outs.append(texts[0])
        if a.text_generate_output_file and getattr(getattr(self.model, "mesh", None), "rank", 0) == 0:
            with open(a.text_generate_output_file, "a", encoding="utf-8") as f:
                for p, o in zip(prompts, outs):
                    f.write(json.dumps({"prompt": p, "output": o}, ensure_ascii=False) + "\n")
        return outs
