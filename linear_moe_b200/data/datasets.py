"""Datasets and batch construction.

* ``SyntheticTokenDataset`` — uniform random token ids from a seed (the benchmark configurations
  use this; the reference's ``MockGPTDataset`` switch is pretrain_qwen.py:278-281).
* ``IndexedDataset`` / ``GPTDataset`` — Megatron mmap ``.bin/.idx`` token store with document /
  sample / shuffle indices (the reference's ``LLamaIdxMapDataset``, data/llama.py:225-320, built on
  ``megatron.core.datasets``).  The sample index is built by the C++ helper
  ``csrc/host/index_builder.cpp`` when the host library is present, else by the numpy fallback.
* ``RawJsonDataset`` — json/jsonl pretrain or SFT samples padded to ``max_padding_length`` with the
  prompt masked out of the labels (``LLamaRawDataset``, data/llama.py:60-222).
* ``get_batch`` — labels = tokens shifted by one, eos/pad masked to -100, position ids, context-
  parallel slicing into *contiguous* chunks (LASP-2 needs rank order = sequence order; the
  reference's zig-zag CP slicing breaks that), and the TP-rank-0 build + broadcast of
  data/utils.py:29-127.
"""
from __future__ import annotations

import json
import os
import queue
import struct
import threading
from typing import Dict, Iterator, List, Optional, Sequence

import numpy as np
import torch

from ..dist import collectives as C
from ..dist.mesh import Mesh

IGNORE_INDEX = -100


class SyntheticTokenDataset(torch.utils.data.Dataset):
    """Sample i is ``seq_length + 1`` uniform ids in ``[0, vocab)`` drawn from ``seed + i``."""

    def __init__(self, vocab_size: int, seq_length: int, num_samples: int = 1 << 30, seed: int = 0):
        self.vocab, self.seq, self.n, self.seed = vocab_size, seq_length, num_samples, seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed + int(i))
        return {"text": torch.randint(0, self.vocab, (self.seq + 1,), generator=g, dtype=torch.int64)}


# ---- Megatron indexed dataset ---------------------------------------------
_HDR = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}


class IndexedDataset:
    """Reader/writer of the Megatron ``MMapIndexedDataset`` format (``<prefix>.bin`` + ``<prefix>.idx``)."""

    def __init__(self, prefix: str):
        with open(prefix + ".idx", "rb") as f:
            assert f.read(9) == _HDR, "not a Megatron mmap index"
            (version,) = struct.unpack("<Q", f.read(8))
            (code,) = struct.unpack("<B", f.read(1))
            (n_seq,) = struct.unpack("<Q", f.read(8))
            (n_doc,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        self.dtype = _DTYPES[code]
        idx = np.memmap(prefix + ".idx", mode="r", order="C")
        self.sizes = np.frombuffer(idx, dtype=np.int32, count=n_seq, offset=offset)
        self.pointers = np.frombuffer(idx, dtype=np.int64, count=n_seq, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(idx, dtype=np.int64, count=n_doc,
                                     offset=offset + self.sizes.nbytes + self.pointers.nbytes)
        self.data = np.memmap(prefix + ".bin", mode="r", order="C")
        self.dtype_code = code
        self.prefix = prefix

    def __len__(self):
        return len(self.sizes)

    def get(self, i: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        n = self.sizes[i] - offset if length is None else length
        return np.frombuffer(self.data, dtype=self.dtype, count=n,
                             offset=self.pointers[i] + offset * np.dtype(self.dtype).itemsize)

    @staticmethod
    def write(prefix: str, docs: Sequence[np.ndarray], dtype=np.int32):
        code = {v: k for k, v in _DTYPES.items()}[dtype]
        sizes, pointers, p = [], [], 0
        with open(prefix + ".bin", "wb") as f:
            for d in docs:
                a = np.asarray(d, dtype=dtype)
                f.write(a.tobytes(order="C"))
                sizes.append(len(a))
                pointers.append(p)
                p += a.nbytes
        with open(prefix + ".idx", "wb") as f:
            f.write(_HDR)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", code))
            f.write(struct.pack("<Q", len(sizes)))
            f.write(struct.pack("<Q", len(sizes) + 1))
            f.write(np.asarray(sizes, dtype=np.int32).tobytes())
            f.write(np.asarray(pointers, dtype=np.int64).tobytes())
            f.write(np.arange(len(sizes) + 1, dtype=np.int64).tobytes())


def build_sample_idx(sizes: np.ndarray, doc_idx: np.ndarray, seq_length: int, num_epochs: int,
                     tokens_per_epoch: int) -> np.ndarray:
    """``sample_idx[i] = (position in doc_idx, token offset in that document)`` of the start of sample
    ``i``; samples are ``seq_length + 1`` tokens that overlap by one (Megatron ``helpers.build_sample_idx``)."""
    from ..utils import hostlib
    lib = hostlib.load()
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    if lib is not None:
        return hostlib.build_sample_idx(lib, sizes, doc_idx, seq_length, num_samples)
    out = np.zeros((num_samples + 1, 2), dtype=np.int64)
    di, off = 0, 0
    for s in range(1, num_samples + 1):
        remaining = seq_length + 1
        while remaining != 0:
            dlen = sizes[doc_idx[di]] - off
            remaining -= dlen
            if remaining <= 0:
                off += remaining + dlen - 1
                remaining = 0
            else:
                di += 1
                off = 0
        out[s] = (di, off)
    return out


class GPTDataset(torch.utils.data.Dataset):
    """Fixed-length samples drawn across document boundaries of an ``IndexedDataset``."""

    def __init__(self, indexed: IndexedDataset, seq_length: int, num_samples: int, seed: int = 1234,
                 documents: Optional[np.ndarray] = None, cache_dir: Optional[str] = None):
        """``cache_dir`` (``--data-cache-path``): the three index arrays are stored there under a name derived from
        everything they depend on and memory-mapped by later runs (and by the other ranks) instead of being rebuilt."""
        self.ds, self.seq = indexed, seq_length
        docs = np.arange(len(indexed), dtype=np.int64) if documents is None else documents
        cached = self._cache_files(cache_dir, indexed, seq_length, num_samples, seed, docs)
        if cached is not None and all(os.path.isfile(f) for f in cached):
            self.doc_idx, self.sample_idx, self.shuffle_idx = (np.load(f, mmap_mode="r") for f in cached)
            self.doc_idx, self.sample_idx = np.ascontiguousarray(self.doc_idx), np.ascontiguousarray(self.sample_idx)
        else:
            tokens_per_epoch = int(np.sum(indexed.sizes[docs]))
            epochs = max(1, -(-(num_samples * seq_length + 1) // max(tokens_per_epoch, 1)))
            rng = np.random.RandomState(seed)
            self.doc_idx = np.concatenate([rng.permutation(docs) for _ in range(epochs)]).astype(np.int64)
            self.sample_idx = build_sample_idx(np.asarray(indexed.sizes), self.doc_idx, seq_length, epochs, tokens_per_epoch)
            self.shuffle_idx = rng.permutation(len(self.sample_idx) - 1)
            if cached is not None and int(os.environ.get("RANK", "0")) == 0:
                os.makedirs(cache_dir, exist_ok=True)
                for f, a in zip(cached, (self.doc_idx, self.sample_idx, self.shuffle_idx)):
                    tmp = f + f".tmp{os.getpid()}.npy"
                    np.save(tmp, a)
                    os.replace(tmp, f)                    # a reader never sees a half-written file
        # aligned in-memory copies of the two per-document tables for the native gather (they sit at unaligned offsets
        # of the memory-mapped .idx file)
        self._sizes = np.require(indexed.sizes, dtype=np.int32, requirements=["C", "A"])
        self._pointers = np.require(indexed.pointers, dtype=np.int64, requirements=["C", "A"])

    @staticmethod
    def _cache_files(cache_dir, indexed, seq_length, num_samples, seed, docs):
        if not cache_dir:
            return None
        import hashlib
        h = hashlib.sha256()
        h.update(repr((os.path.abspath(getattr(indexed, "prefix", "")), len(indexed), int(np.sum(indexed.sizes[docs])),
                       seq_length, num_samples, seed, len(docs), int(docs[0]) if len(docs) else -1,
                       int(docs[-1]) if len(docs) else -1)).encode())
        key = h.hexdigest()[:24]
        return [os.path.join(cache_dir, f"{key}_{part}.npy") for part in ("doc_idx", "sample_idx", "shuffle_idx")]

    def __len__(self):
        return len(self.shuffle_idx)

    def __getitem__(self, i):
        i = self.shuffle_idx[i % len(self.shuffle_idx)]
        (d0, o0), (d1, o1) = self.sample_idx[i], self.sample_idx[i + 1]
        if d0 == d1:
            toks = self.ds.get(self.doc_idx[d0], o0, o1 - o0 + 1)
        else:
            parts = [self.ds.get(self.doc_idx[d0], o0)]
            parts += [self.ds.get(self.doc_idx[d]) for d in range(d0 + 1, d1)]
            parts.append(self.ds.get(self.doc_idx[d1], 0, o1 + 1))
            toks = np.concatenate(parts)
        return {"text": torch.from_numpy(toks.astype(np.int64))}

    def __getitems__(self, indices):
        """Batched fetch (``torch.utils.data`` calls this with a whole batch of indices): one native call assembles all
        samples from the memory-mapped file on several host threads; without the host library, one by one."""
        from ..utils import hostlib
        lib = hostlib.load()
        if lib is None or np.dtype(self.ds.dtype).kind not in "iu":
            return [self[i] for i in indices]
        n = len(self.shuffle_idx)
        rows = self.shuffle_idx[np.asarray(indices, dtype=np.int64) % n]
        toks = hostlib.gather_gpt_samples(lib, self.ds.data, self.ds.dtype_code, self._sizes, self._pointers,
                                          self.doc_idx, self.sample_idx, rows, self.seq)
        batch = torch.from_numpy(toks)
        return [{"text": batch[i]} for i in range(len(rows))]


class BlendedDataset(torch.utils.data.Dataset):
    """Weighted mixture of datasets: sample i comes from the dataset whose running share is furthest
    below its weight (Megatron ``build_blending_indices``)."""

    def __init__(self, datasets: List[torch.utils.data.Dataset], weights: List[float], size: int):
        w = np.asarray(weights, dtype=np.float64)
        w = w / w.sum()
        self.datasets = datasets
        if not 1 <= len(datasets) <= 256:
            raise ValueError(f"a blend takes 1 to 256 datasets, got {len(datasets)}")
        from ..utils import hostlib
        lib = hostlib.load()
        if lib is not None:
            self.ds_index, self.ds_sample = hostlib.build_blending_indices(lib, w, size)
            return
        self.ds_index = np.zeros(size, dtype=np.uint8)
        self.ds_sample = np.zeros(size, dtype=np.int64)
        counts = np.zeros(len(datasets), dtype=np.int64)
        for i in range(size):
            err = w * max(i, 1) - counts
            d = int(np.argmax(err))
            self.ds_index[i], self.ds_sample[i] = d, counts[d]
            counts[d] += 1

    def __len__(self):
        return len(self.ds_index)

    def __getitem__(self, i):
        return self.datasets[self.ds_index[i]][int(self.ds_sample[i])]

    def __getitems__(self, indices):
        """Batched fetch: the indices are grouped by component dataset and every component that has a batched fetch of
        its own (the native gather of ``GPTDataset``) is asked once."""
        idx = np.asarray(indices, dtype=np.int64) % len(self.ds_index)
        out = [None] * len(idx)
        which = self.ds_index[idx]
        for d in np.unique(which):
            pos = np.nonzero(which == d)[0]
            ds = self.datasets[int(d)]
            local = [int(self.ds_sample[idx[p]]) % len(ds) for p in pos]
            batched = getattr(ds, "__getitems__", None)
            rows = batched(local) if batched is not None else [ds[j] for j in local]
            for p, r in zip(pos, rows):
                out[int(p)] = r
        return out


class RawJsonDataset(torch.utils.data.Dataset):
    """json / jsonl samples with ``instruction``/``input``/``output`` (SFT) or ``text``/``content`` (pretrain).
    Every sample is padded or truncated to ``max_padding_length + 1``; for SFT the prompt tokens get label
    -100 (data/llama.py:60-222)."""

    def __init__(self, paths: Sequence[str], tokenizer, max_padding_length: int, sft: bool = False):
        self.tok, self.L, self.sft = tokenizer, max_padding_length, sft
        self.samples: List[dict] = []
        for path in paths:
            with open(path, "r", encoding="utf-8") as f:
                if path.endswith(".jsonl"):
                    rows = [json.loads(l) for l in f if l.strip()]
                else:
                    rows = json.load(f)
            self.samples.extend(rows)

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        row = self.samples[i]
        pad = self.tok.pad_token_id if self.tok.pad_token_id is not None else self.tok.eos_token_id
        if self.sft:
            prompt = row.get("instruction", "") + row.get("input", "")
            p_ids = self.tok.encode(prompt)
            a_ids = self.tok.encode(row.get("output", "")) + [self.tok.eos_token_id]
            ids = (p_ids + a_ids)[: self.L + 1]
            labels = ([IGNORE_INDEX] * len(p_ids) + a_ids)[: self.L + 1]
        else:
            ids = (self.tok.encode(row.get("text", row.get("content", ""))) + [self.tok.eos_token_id])[: self.L + 1]
            labels = list(ids)
        n = self.L + 1 - len(ids)
        ids = ids + [pad] * n
        labels = labels + [IGNORE_INDEX] * n
        return {"text": torch.tensor(ids, dtype=torch.int64), "labels_full": torch.tensor(labels, dtype=torch.int64)}


# ---- batches ---------------------------------------------------------------
def make_batch(sample: Dict[str, torch.Tensor], eod_token: Optional[int] = None, eod_mask_loss: bool = False,
               pad_token: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """``text [B, S+1]`` -> tokens, labels (shifted by one), loss_mask, position_ids."""
    text = sample["text"]
    tokens, labels = text[:, :-1].contiguous(), text[:, 1:].contiguous()
    if "labels_full" in sample:
        labels = sample["labels_full"][:, 1:].contiguous()
    labels = labels.clone()
    if eod_mask_loss and eod_token is not None:
        labels[tokens == eod_token] = IGNORE_INDEX
    if pad_token is not None:
        labels[labels == pad_token] = IGNORE_INDEX
    loss_mask = (labels != IGNORE_INDEX).float()
    pos = torch.arange(tokens.shape[1], dtype=torch.int64, device=tokens.device)[None].expand_as(tokens)
    return {"tokens": tokens, "labels": labels, "loss_mask": loss_mask, "position_ids": pos}


def slice_for_context_parallel(batch: Dict[str, torch.Tensor], mesh: Mesh) -> Dict[str, torch.Tensor]:
    """Keep this rank's contiguous chunk of the sequence dimension."""
    cp = mesh["cp"]
    if cp.is_trivial:
        return batch
    out = {}
    for k, v in batch.items():
        n = v.shape[1] // cp.size
        out[k] = v[:, cp.rank * n:(cp.rank + 1) * n].contiguous()
    return out


def broadcast_batch_over_tp(batch: Optional[Dict[str, torch.Tensor]], mesh: Mesh, shape, device) -> Dict[str, torch.Tensor]:
    """TP rank 0 built the batch; the other TP ranks receive it (data/utils.py:29-127)."""
    g = mesh["tp"]
    if g.is_trivial:
        return batch
    keys = [("tokens", torch.int64), ("labels", torch.int64), ("loss_mask", torch.float32), ("position_ids", torch.int64)]
    out = {}
    for k, dt in keys:
        t = batch[k].to(device) if g.rank == 0 else torch.empty(shape, dtype=dt, device=device)
        out[k] = C.broadcast_(t, g, 0)
    return out


class BatchIterator:
    """Infinite iterator over micro-batches for this rank's data-parallel replica.

    Consecutive global sample indices are dealt round-robin over DP ranks, so a run with DP=W sees the
    same global batch as a single process that reads W micro-batches."""

    def __init__(self, dataset, micro_batch_size: int, mesh: Mesh, device, *, consumed_samples: int = 0,
                 eod_token=None, eod_mask_loss=False, pad_token=None, pin: bool = True, prefetch: int = 0):
        """``prefetch`` (``--num-workers``) > 0: a host thread reads, assembles and pins up to ``2 * prefetch``
        micro-batches ahead of the training loop; the order of the batches is the same as without it."""
        self.ds, self.mbs, self.mesh, self.device = dataset, micro_batch_size, mesh, device
        self._consumed = consumed_samples
        self.kw = dict(eod_token=eod_token, eod_mask_loss=eod_mask_loss, pad_token=pad_token)
        self.pin = pin and torch.cuda.is_available()
        self.prefetch = max(int(prefetch or 0), 0)
        self._queue, self._thread, self._stop, self._ahead = None, None, None, consumed_samples

    # position in the global sample stream; assigning it (a resume) discards what was read ahead
    @property
    def consumed(self) -> int:
        return self._consumed

    @consumed.setter
    def consumed(self, value: int):
        self._shutdown()
        self._consumed = self._ahead = int(value)

    def __iter__(self):
        return self

    def _host_batch(self, start: int):
        mesh = self.mesh
        base = start + mesh.dp_rank * self.mbs
        idx = [(base + i) % len(self.ds) for i in range(self.mbs)]
        batched = getattr(self.ds, "__getitems__", None)        # one native call for the whole micro-batch where there is one
        rows = batched(idx) if batched is not None else [self.ds[j] for j in idx]
        sample = {k: torch.stack([r[k] for r in rows]) for k in rows[0]}
        batch = make_batch(sample, **self.kw)
        batch = slice_for_context_parallel(batch, mesh)
        if self.pin:
            batch = {k: v.contiguous().pin_memory() for k, v in batch.items()}
        return batch

    def _worker(self, q, stop):
        step = self.mbs * self.mesh.dp
        if self.pin and getattr(self.device, "type", None) == "cuda":
            torch.cuda.set_device(self.device)             # pinning allocates through this thread's current device
        try:
            while not stop.is_set():
                item = (self._ahead, self._host_batch(self._ahead))
                self._ahead += step
                while not stop.is_set():
                    try:
                        q.put(item, timeout=0.1)
                        break
                    except queue.Full:
                        continue
        except BaseException as e:                         # hand the error to the training thread
            q.put((None, e))

    def _shutdown(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=10.0)
        self._queue, self._thread, self._stop = None, None, None

    def __next__(self):
        step = self.mbs * self.mesh.dp
        if self.prefetch == 0:
            batch = self._host_batch(self._consumed)
        else:
            if self._thread is None:
                self._queue, self._stop, self._ahead = queue.Queue(maxsize=2 * self.prefetch), threading.Event(), self._consumed
                self._thread = threading.Thread(target=self._worker, args=(self._queue, self._stop), daemon=True)
                self._thread.start()
            start, batch = self._queue.get()
            if start is None:
                self._shutdown()
                raise batch
            assert start == self._consumed, (start, self._consumed)
        self._consumed += step
        return {k: v.to(self.device, non_blocking=True) for k, v in batch.items()}

    def __del__(self):
        try:
            self._shutdown()
        except Exception:
            pass
