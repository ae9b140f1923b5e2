"""Binding of the tcgen05 / TMA / TMEM GEMM family (``csrc/gemm_tcgen05.cu``): dense bf16 GEMM with fused
SwiGLU epilogue, and grouped (per-expert) GEMM."""
from __future__ import annotations

import torch

_ENABLED = False


def available() -> bool:
    return _ENABLED


def supports_swiglu(x, w) -> bool:
    return False


def supports_grouped(x, w1, w2) -> bool:
    return False
