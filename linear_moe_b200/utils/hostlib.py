"""ctypes binding of the host-side C++ helpers (``lib/liblmoe_host.so``)."""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

_LIB = None
_TRIED = False


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "liblmoe_host.so")


def load() -> Optional[ctypes.CDLL]:
    global _LIB, _TRIED
    if not _TRIED:
        _TRIED = True
        p = lib_path()
        if os.path.exists(p):
            _LIB = ctypes.CDLL(p)
            _LIB.lmoe_build_sample_idx.restype = ctypes.c_int
    return _LIB


def build_sample_idx(lib, sizes: np.ndarray, doc_idx: np.ndarray, seq_length: int, num_samples: int) -> np.ndarray:
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int64)
    out = np.zeros((num_samples + 1, 2), dtype=np.int64)
    rc = lib.lmoe_build_sample_idx(sizes.ctypes.data_as(ctypes.c_void_p), doc_idx.ctypes.data_as(ctypes.c_void_p),
                                   ctypes.c_int64(len(doc_idx)), ctypes.c_int64(seq_length),
                                   ctypes.c_int64(num_samples), out.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise ValueError("documents exhausted while building the sample index")
    return out
