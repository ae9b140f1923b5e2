"""jsonl(.zst / .gz) -> tokenised Megatron mmap ``.bin/.idx`` (toolkits/pretrain_data_preprocessing/
preprocess_data_megatron.py:32-418: ``Encoder``, ``Partition``).

  python -m linear_moe_b200.data.preprocess --input a.jsonl b.jsonl --json-keys text --output-prefix out/corpus \
      --patch-tokenizer-type Qwen2Tokenizer --load /path/to/tokenizer --append-eod --workers 8
"""
from __future__ import annotations

import argparse
import gzip
import io
import json
import multiprocessing as mp
import os
from typing import Iterator, List

import numpy as np

from .datasets import IndexedDataset
from .tokenizer import build_tokenizer

_TOK = None
_ARGS = None


def _open(path: str) -> Iterator[str]:
    if path.endswith(".gz"):
        return gzip.open(path, "rt", encoding="utf-8")
    if path.endswith(".zst"):
        import zstandard                                   # optional; only needed for .zst inputs
        return io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(open(path, "rb")), encoding="utf-8")
    return open(path, "r", encoding="utf-8")


def _init(args):
    global _TOK, _ARGS
    _ARGS = args
    _TOK, _ = build_tokenizer(args.patch_tokenizer_type, args.load, args.vocab_size)


def _encode(line: str) -> List[List[int]]:
    line = line.strip()
    if not line:
        return []
    row = json.loads(line)
    docs = []
    for key in _ARGS.json_keys:
        text = row.get(key, "")
        if not text:
            continue
        ids = _TOK.encode(text)
        if _ARGS.append_eod:
            ids.append(_TOK.eod)
        docs.append(ids)
    return docs


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input", nargs="+", required=True)
    p.add_argument("--json-keys", nargs="+", default=["text"])
    p.add_argument("--output-prefix", required=True)
    p.add_argument("--patch-tokenizer-type", default="NullTokenizer")
    p.add_argument("--load", default=None, help="tokenizer path")
    p.add_argument("--vocab-size", type=int, default=32000)
    p.add_argument("--append-eod", action="store_true")
    p.add_argument("--workers", type=int, default=1)
    p.add_argument("--partitions", type=int, default=1, help="write this many shards (<prefix>_<i>)")
    args = p.parse_args(argv)
    os.makedirs(os.path.dirname(os.path.abspath(args.output_prefix)), exist_ok=True)
    docs: List[np.ndarray] = []

    def lines():
        for path in args.input:
            with _open(path) as f:
                yield from f
    if args.workers > 1:
        with mp.Pool(args.workers, initializer=_init, initargs=(args,)) as pool:
            for ds in pool.imap(_encode, lines(), chunksize=64):
                docs.extend(np.asarray(d, dtype=np.int32) for d in ds)
    else:
        _init(args)
        for l in lines():
            docs.extend(np.asarray(d, dtype=np.int32) for d in _encode(l))
    n = max(args.partitions, 1)
    for i in range(n):
        part = docs[i::n]
        prefix = args.output_prefix if n == 1 else f"{args.output_prefix}_{i}"
        IndexedDataset.write(prefix + "_text_document", part)
    print(f"wrote {len(docs)} documents, {sum(len(d) for d in docs)} tokens")


if __name__ == "__main__":
    main()
