"""NVLink peer-memory communicator (symmetric buffers + in-kernel collectives).

``try_enable(numel)`` sets up the communicator for the default process group
and registers it with :mod:`.symm`; it returns False (leaving NCCL in charge)
when peer access or the kernel library is unavailable.
"""
from __future__ import annotations


def try_enable(numel: int, group=None) -> bool:
    try:
        from .peer import PeerComm
    except Exception:
        return False
    try:
        comm = PeerComm.create(numel, group=group)
    except Exception:
        return False
    if comm is None:
        return False
    from . import symm
    symm.set_active_comm(comm, group)
    return True
