"""Registry for the NVLink peer-memory communicator (filled in by
:mod:`.symm_comm` once symmetric buffers have been exchanged).  Collective
call sites ask :func:`active_comm` and fall back to NCCL / Gloo when it
returns None."""
from __future__ import annotations

from typing import Optional

_ACTIVE = {}


def set_active_comm(comm, group=None) -> None:
    _ACTIVE[id(group) if group is not None else None] = comm


def active_comm(group=None):
    """The live communicator of ``group``, or None (none registered, or it was marked dead
    after a peer timeout)."""
    comm = _ACTIVE.get(id(group) if group is not None else None)
    if comm is not None and getattr(comm, "dead", False):
        return None
    return comm


def clear() -> None:
    _ACTIVE.clear()
