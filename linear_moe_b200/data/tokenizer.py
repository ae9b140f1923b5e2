"""Tokenizer table: ``--patch-tokenizer-type`` -> wrapper with a uniform interface.

Reference: linear_moe/tokenizer/__init__.py:17-31 (``_vocab_size_with_padding``), :38-471
(``build_tokenizer`` and the per-family wrappers around HuggingFace ``AutoTokenizer``).  All HF-backed
types share one wrapper here; they differ only in special-token handling.  ``NullTokenizer`` needs no
files and serves synthetic-data runs.
"""
from __future__ import annotations

from typing import List, Optional

from ..config.arguments import pad_vocab

_HF_TYPES = {
    "LLamaTokenizer": {}, "LLama2Tokenizer": {}, "LLama3Tokenizer": {"pad": "<|finetune_right_pad_id|>"},
    "Qwen2Tokenizer": {"pad": "<|extra_0|>", "eos": "<|endoftext|>"}, "QwenTokenizer": {"pad": "<|extra_0|>"},
    "QwenVLTokenizer": {"pad": "<|extra_0|>"}, "MistralTokenizer": {"pad": "<unk>"},
    "DeepSeekV2Tokenizer": {"pad": "<｜end▁of▁sentence｜>"}, "YiTokenizer": {}, "FalconTokenizer": {},
    "BloomTokenizerFromHF": {}, "BloomTokenizerFromCustom": {}, "ChatGLMTokenizerFromHF": {},
    "GLM10BZHTokenizerFromHF": {}, "StarcoderTokenizerFromHF": {}, "VicunaTokenizerFromHF": {}, "OPTTokenizer": {},
}


class NullTokenizer:
    """Whitespace-separated integers; vocabulary size given on the command line."""

    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size
        self.eos_token_id = vocab_size - 1
        self.pad_token_id = vocab_size - 1
        self.eod = self.eos_token_id

    def encode(self, text: str) -> List[int]:
        return [int(t) % self.vocab_size for t in text.split()]

    tokenize = encode

    def decode(self, ids) -> str:
        return " ".join(str(int(i)) for i in ids)

    detokenize = decode


class HFTokenizer:
    def __init__(self, path: str, kind: str, max_length: Optional[int] = None, extra_vocab_size: int = 0):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(path, padding_side="right", use_fast=False, trust_remote_code=True,
                                                 model_max_length=max_length)
        spec = _HF_TYPES.get(kind, {})
        if self.tok.pad_token is None:
            if "pad" in spec:
                self.tok.add_special_tokens({"pad_token": spec["pad"]})
            else:
                self.tok.pad_token = self.tok.eos_token
        if "eos" in spec and self.tok.eos_token is None:
            self.tok.eos_token = spec["eos"]
        self.extra_vocab_size = extra_vocab_size

    @property
    def vocab_size(self):
        return len(self.tok) + self.extra_vocab_size

    @property
    def eos_token_id(self):
        return self.tok.eos_token_id

    @property
    def pad_token_id(self):
        return self.tok.pad_token_id

    @property
    def eod(self):
        return self.tok.eos_token_id

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False)

    tokenize = encode

    def decode(self, ids) -> str:
        return self.tok.decode(ids, skip_special_tokens=True)

    detokenize = decode

    def __call__(self, *a, **kw):
        return self.tok(*a, **kw)


def build_tokenizer(kind: str, path: Optional[str] = None, vocab_size: Optional[int] = None,
                    extra_vocab_size: int = 0, max_length: Optional[int] = None,
                    make_divisible_by: int = 128, tp: int = 1):
    """Returns ``(tokenizer, padded_vocab_size)``."""
    if kind == "NullTokenizer" or path is None:
        tok = NullTokenizer(vocab_size or 32000)
        return tok, pad_vocab(tok.vocab_size + extra_vocab_size, make_divisible_by, tp)
    if kind in ("JiebaBPETokenizer", "IcetkGLM130BTokenizer"):
        raise NotImplementedError(f"{kind} needs its vendored vocabulary files, which are not shipped")
    tok = HFTokenizer(path, kind, max_length, extra_vocab_size)
    return tok, pad_vocab(tok.vocab_size, make_divisible_by, tp)
