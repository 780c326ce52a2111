"""Drop-oldest single-producer / single-consumer ring of fixed-shape numpy slots
in POSIX shared memory (API of src/chaoscontrol/episodic/ipc.py:149-391:
``ShmRing.create / attach / try_write / try_read / dropped_count / close /
close_and_unlink``).

One segment holds a 256-byte header followed by the slot table::

    int64[0..2]   head, tail, dropped     (monotonic counters; slot = counter % capacity)
    int64[3..5]   capacity, ndim, itemsize
    int64[6..13]  slot shape (up to 8 dims)
    bytes[128..]  numpy dtype string (e.g. ``<f4``), NUL padded

``attach`` checks the caller's shape / dtype / capacity against the header before
any view of the slots is built: shared memory is rounded up to whole pages, so a
wrong claim would otherwise fit and read garbage.  The writer never blocks: on a
full ring it advances ``tail`` (dropping the oldest slot) and counts the drop.
The wire-record rings of the controller proper are the C++ lock-free rings of
``native/ring.h``; this class is the general-purpose numpy one.
"""
from __future__ import annotations

from multiprocessing.shared_memory import SharedMemory
from typing import Optional, Sequence

import numpy as np

MAX_NDIM = 8
_HEADER_BYTES = 256
_HEAD, _TAIL, _DROPPED, _CAP, _NDIM, _ITEM, _SHAPE0 = 0, 1, 2, 3, 4, 5, 6
_DTYPE_OFF, _DTYPE_LEN = 128, 64

__all__ = ["ShmRing", "MAX_NDIM"]


class ShmRing:
    def __init__(self, shm: SharedMemory, slot_shape: tuple[int, ...], dtype: np.dtype, capacity: int,
                 owner: bool) -> None:
        self._shm, self._owner = shm, owner
        self._shape, self._dtype, self._cap = slot_shape, dtype, capacity
        self._hdr = np.ndarray((16,), dtype=np.int64, buffer=shm.buf)
        self._slots = np.ndarray((capacity, *slot_shape), dtype=dtype, buffer=shm.buf, offset=_HEADER_BYTES)
        self._closed = self._unlinked = False

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _norm(slot_shape: Sequence[int], dtype, capacity: int) -> tuple[tuple[int, ...], np.dtype, int]:
        if capacity <= 0:
            raise ValueError(f"capacity must be positive; got {capacity}")
        shape = tuple(int(d) for d in slot_shape)
        if len(shape) > MAX_NDIM:
            raise ValueError(f"slot_shape has {len(shape)} dims; MAX_NDIM={MAX_NDIM}")
        return shape, np.dtype(dtype), int(capacity)

    @classmethod
    def create(cls, *, name: str, slot_shape: Sequence[int], dtype, capacity: int) -> "ShmRing":
        """Producer side: allocates a new zeroed segment ``name`` (``FileExistsError`` if present)."""
        shape, dt, cap = cls._norm(slot_shape, dtype, capacity)
        nbytes = _HEADER_BYTES + cap * int(np.prod(shape, dtype=np.int64)) * dt.itemsize
        shm = SharedMemory(name=name, create=True, size=max(nbytes, _HEADER_BYTES + 1))
        np.ndarray((nbytes,), dtype=np.uint8, buffer=shm.buf)[:] = 0
        hdr = np.ndarray((16,), dtype=np.int64, buffer=shm.buf)
        hdr[_CAP], hdr[_NDIM], hdr[_ITEM] = cap, len(shape), dt.itemsize
        hdr[_SHAPE0:_SHAPE0 + len(shape)] = shape
        tag = dt.str.encode()[:_DTYPE_LEN]
        shm.buf[_DTYPE_OFF:_DTYPE_OFF + len(tag)] = tag
        return cls(shm, shape, dt, cap, owner=True)

    @classmethod
    def attach(cls, *, name: str, slot_shape: Sequence[int], dtype, capacity: int) -> "ShmRing":
        """Consumer side: opens ``name`` and validates the claimed layout against the header."""
        shape, dt, cap = cls._norm(slot_shape, dtype, capacity)
        shm = SharedMemory(name=name, create=False)
        try:
            hdr = np.ndarray((16,), dtype=np.int64, buffer=shm.buf)
            stored_shape = tuple(int(x) for x in hdr[_SHAPE0:_SHAPE0 + int(hdr[_NDIM])])
            stored_dt = bytes(shm.buf[_DTYPE_OFF:_DTYPE_OFF + _DTYPE_LEN]).split(b"\0", 1)[0].decode()
            if int(hdr[_CAP]) != cap:
                raise ValueError(f"capacity mismatch: ring was created with {int(hdr[_CAP])}, caller claims {cap}")
            if stored_shape != shape:
                raise ValueError(f"slot_shape mismatch: ring was created with {stored_shape}, caller claims {shape}")
            if stored_dt != dt.str:
                raise ValueError(f"dtype mismatch: ring was created with {stored_dt}, caller claims {dt.str}")
        except Exception:
            del hdr
            shm.close()
            raise
        del hdr
        return cls(shm, shape, dt, cap, owner=False)

    # ------------------------------------------------------------------ data path
    def try_write(self, item: np.ndarray) -> None:
        if not isinstance(item, np.ndarray):
            raise ValueError(f"try_write requires numpy.ndarray; got {type(item).__name__}")
        if item.shape != self._shape:
            raise ValueError(f"shape mismatch: ring expects {self._shape}, got {tuple(item.shape)}")
        if item.dtype != self._dtype:
            raise ValueError(f"dtype mismatch: ring expects {self._dtype}, got {item.dtype}")
        h = self._hdr
        head, tail = int(h[_HEAD]), int(h[_TAIL])
        if head - tail >= self._cap:
            h[_TAIL] = tail + 1
            h[_DROPPED] += 1
        self._slots[head % self._cap] = item
        h[_HEAD] = head + 1                        # publish after the payload

    def try_read(self) -> Optional[np.ndarray]:
        """Oldest unread slot as a caller-owned copy, or ``None`` when empty."""
        h = self._hdr
        head, tail = int(h[_HEAD]), int(h[_TAIL])
        if head == tail:
            return None
        out = self._slots[tail % self._cap].copy()
        h[_TAIL] = tail + 1
        return out

    def __len__(self) -> int:
        return int(self._hdr[_HEAD]) - int(self._hdr[_TAIL])

    def dropped_count(self) -> int:
        return int(self._hdr[_DROPPED])

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        if self._closed:
            return
        self._hdr = self._slots = None          # views must go before the mapping
        self._shm.close()
        self._closed = True

    def close_and_unlink(self) -> None:
        self.close()
        if self._unlinked:
            return
        if self._owner:
            try:
                self._shm.unlink()
            except FileNotFoundError:
                pass
        self._unlinked = True
