"""``--dataset`` switch -> (train, valid) datasets (linear_moe/data/__init__.py:29-228)."""
from __future__ import annotations

import numpy as np

from .datasets import BlendedDataset, GPTDataset, IndexedDataset, RawJsonDataset, SyntheticTokenDataset
from .tokenizer import build_tokenizer


def _split_documents(n_docs: int, split: str):
    w = [float(x) for x in split.split(",")]
    w = w + [0.0] * (3 - len(w))
    tot = sum(w)
    bounds = np.cumsum([0] + [int(round(x / tot * n_docs)) for x in w])
    bounds[-1] = n_docs
    return [np.arange(bounds[i], bounds[i + 1], dtype=np.int64) for i in range(3)]


def build_pretrain_dataset_from_idxmap(paths, seq_length, num_samples, seed, split, cache_dir=None):
    """``paths`` is either one prefix or ``w1 prefix1 w2 prefix2 ...`` (Megatron blend syntax)."""
    if len(paths) == 1:
        weights, prefixes = [1.0], list(paths)
    else:
        weights, prefixes = [float(x) for x in paths[0::2]], list(paths[1::2])
    trains, valids = [], []
    for p in prefixes:
        ds = IndexedDataset(p)
        tr, va, _ = _split_documents(len(ds), split)
        trains.append(GPTDataset(ds, seq_length, num_samples, seed, tr, cache_dir=cache_dir))
        if len(va):
            valids.append(GPTDataset(ds, seq_length, max(num_samples // 100, 1), seed, va, cache_dir=cache_dir))
    if len(trains) == 1:
        return trains[0], (valids[0] if valids else None)
    train = BlendedDataset(trains, weights, num_samples)
    valid = BlendedDataset(valids, weights[: len(valids)], max(num_samples // 100, 1)) if valids else None
    return train, valid


def build_datasets(args, cfg, tc):
    n = tc.train_iters * tc.global_batch_size
    if tc.dataset == "Synthetic":
        return SyntheticTokenDataset(cfg.vocab_size, tc.seq_length, seed=tc.seed), \
            SyntheticTokenDataset(cfg.vocab_size, tc.seq_length, seed=tc.seed + (1 << 24))
    if tc.dataset == "LLama-Pretrain-Idxmap":
        return build_pretrain_dataset_from_idxmap(tc.data_path, tc.seq_length, n, tc.seed, tc.split,
                                                  cache_dir=getattr(args, "data_cache_path", None))
    tok, _ = build_tokenizer(args.patch_tokenizer_type, args.tokenizer_model, cfg.vocab_size, args.extra_vocab_size)
    L = tc.max_padding_length or tc.seq_length
    sft = tc.dataset == "LLama-SFT"
    train = RawJsonDataset(tc.train_data or tc.data_path, tok, L, sft=sft)
    valid = RawJsonDataset(tc.valid_data, tok, L, sft=sft) if tc.valid_data else None
    return train, valid
