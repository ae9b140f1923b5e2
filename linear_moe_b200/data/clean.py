"""Raw-corpus preparation in front of the tokenising preprocessor (``data/preprocess.py``).

Counterpart of the small scripts of the reference's ``toolkits/pretrain_data_preprocessing``:

* ``clean``   JSON arrays of records (``content`` / ``output`` / ``text`` fields, the WuDao layout) -> one JSON object per
  line with the cleaned text, as ``{"text": ...}`` for pretraining or ``{"instruction": "", "input": "", <key>: ...}`` for
  the SFT reader (``clean_raw_text.py:12-46``, ``preprocess_wudao2.py:11-44``);
* ``to-list`` JSON lines -> one indented JSON array, in place or to a new file (``convert_json_to_list.py``);
* ``pack``    tokenise JSON lines, concatenate all documents and cut the stream into samples of exactly
  ``sequence_length`` tokens (the remainder is dropped), written as a Megatron ``.bin`` / ``.idx`` pair whose documents
  are the samples (``qwen_hf_preprocess_datasets.py:8-57`` writes a ``datasets`` folder instead).

Cleaning: URLs are removed, every character outside letters, digits, CJK unified ideographs and a fixed set of Latin and
CJK punctuation is dropped, then runs of spaces collapse to one.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
from concurrent.futures import ProcessPoolExecutor
from typing import Iterable, Iterator, List, Optional, Sequence

import numpy as np

_URL = re.compile(r"https?://[\x21-\x7e]+")
_SPACES = re.compile(r" {2,}")
_KEEP_PUNCT = ".,-%*/&()+! " + "，。《》•、＆—（）：？！“”·"
_DROP = re.compile("[^0-9A-Za-z一-龥" + re.escape(_KEEP_PUNCT) + "]+")
TEXT_FIELDS = ("output", "content", "text")


def clean_text(raw: str) -> str:
    return _SPACES.sub(" ", _DROP.sub("", _URL.sub("", raw))).strip()


def _records(path: str) -> Iterator[dict]:
    """Records of a JSON array file or a JSON-lines file; an unreadable file yields nothing."""
    with open(path, "r", encoding="utf-8") as f:
        head = f.read(1)
        f.seek(0)
        try:
            if head == "[":
                yield from json.load(f)
            else:
                for line in f:
                    if line.strip():
                        yield json.loads(line)
        except ValueError:
            return


def clean_file(src: str, dst: str, target_key: Optional[str] = None, min_chars: int = 0) -> int:
    """Clean every record's text field; ``target_key`` None writes ``{"text": ...}``, otherwise an SFT record whose
    answer field is ``target_key``.  Returns the number of records written."""
    n = 0
    with open(dst, "w", encoding="utf-8") as out:
        for rec in _records(src):
            field = next((k for k in TEXT_FIELDS if k in rec), None)
            if field is None:
                continue
            text = clean_text(str(rec[field]))
            if len(text) < min_chars:
                continue
            row = {"text": text} if target_key is None else {"instruction": "", "input": "", target_key: text}
            out.write(json.dumps(row, ensure_ascii=False) + "\n")
            n += 1
    return n


def clean_dir(input_dir: str, output_dir: str, target_key: Optional[str] = None, processes: Optional[int] = None,
              min_chars: int = 0) -> int:
    os.makedirs(output_dir, exist_ok=True)
    files = sorted(glob.glob(os.path.join(input_dir, "*.json")) + glob.glob(os.path.join(input_dir, "*.jsonl")))
    jobs = [(f, os.path.join(output_dir, os.path.basename(f)), target_key, min_chars) for f in files]
    if not jobs:
        return 0
    if (processes or 1) <= 1 or len(jobs) == 1:
        return sum(clean_file(*j) for j in jobs)
    import multiprocessing
    with ProcessPoolExecutor(max_workers=processes, mp_context=multiprocessing.get_context("spawn")) as ex:
        return sum(ex.map(_clean_job, jobs))


def _clean_job(job) -> int:
    return clean_file(*job)


def jsonl_to_list(path: str, dst: Optional[str] = None) -> int:
    rows = list(_records(path))
    with open(dst or path, "w", encoding="utf-8") as f:
        json.dump(rows, f, ensure_ascii=False, indent=4)
    return len(rows)


def pack_tokens(docs: Iterable[Sequence[int]], sequence_length: int) -> List[np.ndarray]:
    """Concatenate token lists and cut the stream into rows of ``sequence_length`` tokens; the tail is dropped."""
    rows: List[np.ndarray] = []
    buf: List[int] = []
    for d in docs:
        buf.extend(int(t) for t in d)
        while len(buf) >= sequence_length:
            rows.append(np.asarray(buf[:sequence_length], dtype=np.int64))
            del buf[:sequence_length]
    return rows


def pack_file(src: str, prefix: str, tokenizer, sequence_length: int, key: str = "text", append_eod: bool = False) -> int:
    from .datasets import IndexedDataset

    def docs():
        for rec in _records(src):
            ids = list(tokenizer.tokenize(str(rec.get(key, ""))))
            if append_eod:
                ids.append(tokenizer.eod)
            yield ids
    rows = pack_tokens(docs(), sequence_length)
    vocab = getattr(tokenizer, "vocab_size", 1 << 31)
    IndexedDataset.write(prefix, rows, dtype=np.uint16 if vocab < 65500 else np.int32)
    return len(rows)


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = p.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("clean")
    c.add_argument("--input-dir", "-i", required=True)
    c.add_argument("--output-dir", "-o", required=True)
    c.add_argument("--target-key", "-k", default=None, help="write SFT records with this answer field instead of {'text'}")
    c.add_argument("--num-processes", "-p", type=int, default=None)
    c.add_argument("--min-chars", type=int, default=0)
    t = sub.add_parser("to-list")
    t.add_argument("files", nargs="+")
    k = sub.add_parser("pack")
    k.add_argument("--input", required=True)
    k.add_argument("--output-prefix", required=True)
    k.add_argument("--sequence-length", type=int, default=2048)
    k.add_argument("--json-key", default="text")
    k.add_argument("--patch-tokenizer-type", default="NullTokenizer")
    k.add_argument("--load", default=None, help="tokenizer path")
    k.add_argument("--vocab-size", type=int, default=32000)
    k.add_argument("--append-eod", action="store_true")
    a = p.parse_args(argv)
    if a.cmd == "clean":
        print(f"{clean_dir(a.input_dir, a.output_dir, a.target_key, a.num_processes, a.min_chars)} records")
    elif a.cmd == "to-list":
        for f in a.files:
            print(f"{f}: {jsonl_to_list(f)} records")
    else:
        from .tokenizer import build_tokenizer
        tok, _ = build_tokenizer(a.patch_tokenizer_type, a.load, a.vocab_size, 0)
        print(f"{pack_file(a.input, a.output_prefix, tok, a.sequence_length, a.json_key, a.append_eod)} samples")


if __name__ == "__main__":
    main()
