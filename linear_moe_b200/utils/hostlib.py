"""ctypes binding of the host-side C++ helpers (``lib/liblmoe_host.so``)."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

_LIB = None
_TRIED = False


GATHER_ERRORS = {2: "an index outside its table", 3: "a token range outside the .bin file",
                 4: "a sample that does not hold seq_length + 1 tokens", 5: "a token type that is not an integer type"}


def lib_path() -> str:
    """``LMOE_HOST_LIB`` names another build of the library (the sanitizer build in the tests)."""
    return os.environ.get("LMOE_HOST_LIB") or os.path.join(
        os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "liblmoe_host.so")


def load() -> Optional[ctypes.CDLL]:
    global _LIB, _TRIED
    if not _TRIED:
        _TRIED = True
        p = lib_path()
        if os.path.exists(p):
            _LIB = ctypes.CDLL(p)
            for fn in ("lmoe_build_sample_idx", "lmoe_build_blending_indices", "lmoe_gather_gpt_samples"):
                getattr(_LIB, fn).restype = ctypes.c_int
    return _LIB


def _ptr(a: np.ndarray):
    return ctypes.c_void_p(a.ctypes.data)


def build_sample_idx(lib, sizes: np.ndarray, doc_idx: np.ndarray, seq_length: int, num_samples: int) -> np.ndarray:
    sizes = np.require(sizes, dtype=np.int32, requirements=["C", "A"])       # the .idx tables sit at unaligned file offsets
    doc_idx = np.require(doc_idx, dtype=np.int64, requirements=["C", "A"])
    out = np.zeros((num_samples + 1, 2), dtype=np.int64)
    rc = lib.lmoe_build_sample_idx(sizes.ctypes.data_as(ctypes.c_void_p), doc_idx.ctypes.data_as(ctypes.c_void_p),
                                   ctypes.c_int64(len(doc_idx)), ctypes.c_int64(seq_length),
                                   ctypes.c_int64(num_samples), out.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise ValueError("documents exhausted while building the sample index")
    return out


def build_blending_indices(lib, weights: np.ndarray, size: int):
    """``(ds_index uint8 [size], ds_sample int64 [size])``: sample i comes from the dataset whose running count lags its
    weight the most."""
    w = np.ascontiguousarray(weights, dtype=np.float64)
    ds_index = np.zeros(size, dtype=np.uint8)
    ds_sample = np.zeros(size, dtype=np.int64)
    rc = lib.lmoe_build_blending_indices(_ptr(ds_index), _ptr(ds_sample), _ptr(w), ctypes.c_int32(len(w)),
                                         ctypes.c_int64(size))
    if rc != 0:
        raise ValueError(f"a blend takes 1 to 256 datasets, got {len(w)}")
    return ds_index, ds_sample


def gather_gpt_samples(lib, data: np.ndarray, dtype_code: int, sizes: np.ndarray, pointers: np.ndarray,
                       doc_idx: np.ndarray, sample_idx: np.ndarray, indices: np.ndarray, seq_length: int,
                       nthreads: int = 4) -> np.ndarray:
    """``[len(indices), seq_length + 1]`` int64 tokens of the samples ``indices`` (positions in ``sample_idx``), read from
    the memory-mapped ``.bin`` bytes ``data``.  The index tables must be C-contiguous arrays of their file dtypes."""
    assert data.dtype == np.uint8 and sample_idx.ndim == 2 and sample_idx.shape[1] == 2
    for a, dt in ((sizes, np.int32), (pointers, np.int64), (doc_idx, np.int64), (sample_idx, np.int64)):
        assert a.dtype == dt and a.flags.c_contiguous and a.flags.aligned, "index tables: aligned C arrays of their file dtypes"
    idx = np.ascontiguousarray(indices, dtype=np.int64)
    out = np.empty((len(idx), seq_length + 1), dtype=np.int64)
    rc = lib.lmoe_gather_gpt_samples(
        _ptr(data), ctypes.c_int64(data.nbytes), ctypes.c_int32(dtype_code), _ptr(sizes), _ptr(pointers),
        ctypes.c_int64(len(sizes)), _ptr(doc_idx), ctypes.c_int64(len(doc_idx)), _ptr(sample_idx),
        ctypes.c_int64(len(sample_idx) - 1), _ptr(idx), ctypes.c_int64(len(idx)), ctypes.c_int64(seq_length),
        _ptr(out), ctypes.c_int32(nthreads))
    if rc != 0:
        raise ValueError("sample gather failed: " + GATHER_ERRORS.get(rc, f"code {rc}"))
    return out
