"""Adaptor that exposes a ``CausalLM`` to lm-evaluation-harness style callers, and the OpenCompass-style wrapper.

Reference: linear_moe/lm_evaluate.py:40-205 (``EvalHarnessAdaptor``: ``loglikelihood``, ``loglikelihood_rolling``,
``generate_until`` over a Megatron model with TP logits gather and PP send/recv) and
eval/models/qwen2_linear_moe.py:45-144 (``Qwen2LinearMoe.generate`` for OpenCompass).  The harness packages
themselves are not on this image, so this class implements the three request types of the harness API directly and
does not import ``lm_eval``; ``lm_eval`` can register it as a model through ``get_lm_eval_model``.
"""
from __future__ import annotations

from typing import Iterable, List, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import generation as G


class EvalHarnessAdaptor:
    def __init__(self, model, tokenizer, max_length: int = 2048, batch_size: int = 1, device=None):
        self.model, self.tok = model.eval(), tokenizer
        self.max_length, self.batch_size = max_length, batch_size
        self.device = device or next(model.parameters()).device
        self.eot_token_id = getattr(tokenizer, "eod", None)

    # -- helpers ---------------------------------------------------------------
    def tok_encode(self, s: str) -> List[int]:
        return self.tok.encode(s)

    @torch.no_grad()
    def _model_call(self, ids: torch.Tensor) -> torch.Tensor:
        """Logits on every rank: the stages relay the activations, the last stage's (TP-gathered) logits are broadcast."""
        from .parallel_forward import full_logits
        return full_logits(self.model, ids.to(self.device))

    def _loglikelihood_tokens(self, pairs: Sequence[Tuple[List[int], List[int]]]) -> List[Tuple[float, bool]]:
        out = []
        for ctx, cont in pairs:
            if not ctx:
                ctx = [self.eot_token_id if self.eot_token_id is not None else 0]
            full = (ctx + cont)[-(self.max_length + 1):]
            n_cont = min(len(cont), len(full) - 1)
            ids = torch.tensor([full[:-1]], dtype=torch.long)
            logits = self._model_call(ids)[0]
            lp = F.log_softmax(logits, -1)[-n_cont:]
            tgt = torch.tensor(full[-n_cont:], device=lp.device)
            ll = lp.gather(1, tgt[:, None]).sum().item()
            greedy = bool((lp.argmax(-1) == tgt).all())
            out.append((ll, greedy))
        return out

    # -- harness API -------------------------------------------------------------
    def loglikelihood(self, requests: Iterable[Tuple[str, str]]) -> List[Tuple[float, bool]]:
        return self._loglikelihood_tokens([(self.tok_encode(c), self.tok_encode(x)) for c, x in requests])

    def loglikelihood_rolling(self, requests: Iterable[Tuple[str]]) -> List[float]:
        res = []
        for (text,) in requests:
            toks = self.tok_encode(text)
            total, prev = 0.0, [self.eot_token_id if self.eot_token_id is not None else 0]
            for s in range(0, len(toks), self.max_length):
                win = toks[s:s + self.max_length]
                total += self._loglikelihood_tokens([(prev, win)])[0][0]
                prev = win[-1:]
            res.append(total)
        return res

    def generate_until(self, requests: Iterable[Tuple[str, dict]]) -> List[str]:
        outs = []
        for ctx, kw in requests:
            until = kw.get("until", []) if isinstance(kw, dict) else []
            n = kw.get("max_gen_toks", 64) if isinstance(kw, dict) else 64
            texts, toks, _ = G.generate_and_post_process(self.model, self.tok, [ctx], tokens_to_generate=n, top_k_sampling=1,
                                                         device=self.device)
            gen = self.tok.decode(toks[0][len(self.tok_encode(ctx)):])
            for u in until:
                gen = gen.split(u)[0]
            outs.append(gen)
        return outs


class LinearMoeOpenCompassModel:
    """``generate(inputs, max_out_len)`` / ``get_ppl(inputs)`` as OpenCompass model wrappers expect."""

    def __init__(self, model, tokenizer, max_seq_len: int = 2048):
        self.ad = EvalHarnessAdaptor(model, tokenizer, max_seq_len)

    def generate(self, inputs: List[str], max_out_len: int = 64) -> List[str]:
        return self.ad.generate_until([(s, {"max_gen_toks": max_out_len}) for s in inputs])

    def get_ppl(self, inputs: List[str]) -> List[float]:
        out = []
        for s in inputs:
            n = max(len(self.ad.tok_encode(s)), 1)
            out.append(-self.ad.loglikelihood_rolling([(s,)])[0] / n)
        return out


def get_lm_eval_model(model, tokenizer, **kw):
    """Wrap for lm-evaluation-harness when that package is installed; otherwise return the bare adaptor."""
    ad = EvalHarnessAdaptor(model, tokenizer, **kw)
    try:
        from lm_eval.api.model import LM                      # optional dependency
    except Exception:
        return ad

    class _LM(LM):
        def loglikelihood(self, requests):
            return ad.loglikelihood([r.args for r in requests])

        def loglikelihood_rolling(self, requests):
            return ad.loglikelihood_rolling([r.args for r in requests])

        def generate_until(self, requests):
            return ad.generate_until([r.args for r in requests])
    return _LM()
