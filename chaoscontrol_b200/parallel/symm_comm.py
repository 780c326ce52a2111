"""NVLink peer-memory communicator (symmetric buffers + in-kernel collectives).

``try_enable(numel)`` sets up the communicator for a process group and registers
it with :mod:`.symm`.  The outcome is the same on every rank: ``PeerComm.create``
votes, so either all ranks get the communicator or none does.  ``enable`` is the
strict form for callers that must not run on the library fallback (the
benchmark): it raises with the reason instead of returning False.
"""
from __future__ import annotations

_last_reason = ""


def try_enable(numel: int, group=None) -> bool:
    """True when the peer-memory communicator is up on every rank; False (with the
    reason available from :func:`last_reason`) when collectives stay on NCCL / gloo."""
    global _last_reason
    _last_reason = ""
    try:
        from . import peer
    except Exception as exc:                      # library missing, no CUDA build: same on every rank
        _last_reason = f"import failed: {type(exc).__name__}: {exc}"
        return False
    comm = peer.PeerComm.create(numel, group=group)
    if comm is None:
        _last_reason = peer.last_failure or "peer communicator unavailable"
        return False
    from . import symm
    symm.set_active_comm(comm, group)
    return True


def last_reason() -> str:
    return _last_reason


def enable(numel: int, group=None):
    """Like :func:`try_enable` but raises ``RuntimeError`` with the reason on failure; returns the
    communicator."""
    if not try_enable(numel, group):
        raise RuntimeError(f"peer-memory communicator unavailable: {_last_reason}")
    from . import symm
    return symm.active_comm(group)


def disable(group=None) -> None:
    """Collective teardown of the registered communicator (every rank, before the process group is
    destroyed)."""
    from . import symm
    comm = symm.active_comm(group)
    if comm is not None:
        symm.set_active_comm(None, group)
        comm.close()
