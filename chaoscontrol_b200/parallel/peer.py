"""``PeerComm``: symmetric buffers over CUDA IPC plus the in-kernel all-reduce of
``csrc/comm.cu``.

One process per GPU on one node.  Each rank allocates a bf16 data buffer, an
fp32 reduced-slice staging buffer and a signal pad, exports them with CUDA IPC,
and maps every peer's copies (handles travel through the process group's object
all-gather).  ``all_reduce_`` then launches the pack / reduce kernels on the
current stream; no NCCL call is involved.

Timeouts: every device-side wait is bounded by ``timeout_ms``; a rank that
never signals makes the others record ``CCB_ERR_PEER_TIMEOUT`` in the status
word (read with :func:`chaoscontrol_b200.ops._lib.read_status`) and return with
their gradients unreduced, instead of hanging.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import i64, vp

_lib.register_sig("ccb_comm_malloc", [i64], vp)
_lib.register_sig("ccb_comm_free", [vp])
_lib.register_sig("ccb_ipc_get", [vp, vp])
_lib.register_sig("ccb_ipc_open", [vp], vp)
_lib.register_sig("ccb_ipc_close", [vp])
_lib.register_sig("ccb_allreduce", [vp, i64, C.c_float, vp, vp, vp, i64, i64, i64, vp, i64, i64, vp])
_lib.register_sig("ccb_comm_wait_probe", [vp, i64, i64, vp, vp])
_lib.register_sig("ccb_sharded_sync", [i64, vp, vp, i64, C.c_float, vp, i64, vp, vp, vp, i64, i64, i64, vp, i64, vp])

MAX_RANKS = 8
ONE_SHOT_MAX_BYTES = 64 << 20      # bf16 payload; above this the two-shot kernels run


class PeerComm:
    def __init__(self) -> None:
        self.rank = 0
        self.ws = 1
        self.numel = 0
        self.epoch = 0
        self.timeout_ms = 2000
        self._own: list[int] = []
        self._opened: list[int] = []
        self._bufs = self._bufs2 = self._pads = None
        self._counters = None

    # ------------------------------------------------------------------
    @classmethod
    def create(cls, numel: int, group=None, timeout_ms: int = 2000) -> Optional["PeerComm"]:
        if not (dist.is_available() and dist.is_initialized()):
            return None
        ws = dist.get_world_size(group)
        if ws < 2 or ws > MAX_RANKS or not _lib.available():
            return None
        L = _lib.lib()
        self = cls()
        self.rank, self.ws, self.timeout_ms = dist.get_rank(group), ws, timeout_ms
        unit = 8 * ws
        self.numel = (numel + unit - 1) // unit * unit
        sizes = {"buf": self.numel * 2, "buf2": (self.numel // ws) * 4, "pad": 4 * MAX_RANKS * 4}
        mine, handles = {}, {}
        for k, nbytes in sizes.items():
            p = L.ccb_comm_malloc(max(nbytes, 256))
            if not p:
                raise RuntimeError(f"peer comm: allocation of {nbytes} bytes failed: "
                                   f"{L.ccb_last_error().decode()}")
            mine[k] = p
            self._own.append(p)
            h = (C.c_char * 64)()
            _lib.check(L.ccb_ipc_get(p, h), "ipc_get")
            handles[k] = bytes(h)
        gathered: list = [None] * ws
        dist.all_gather_object(gathered, handles, group=group)
        tables = {k: (C.c_void_p * MAX_RANKS)() for k in sizes}
        for r in range(ws):
            for k in sizes:
                if r == self.rank:
                    tables[k][r] = mine[k]
                else:
                    p = L.ccb_ipc_open(C.create_string_buffer(gathered[r][k], 64))
                    if not p:
                        raise RuntimeError(f"peer comm: cannot map rank {r}'s {k}: "
                                           f"{L.ccb_last_error().decode()}")
                    self._opened.append(p)
                    tables[k][r] = p
        self._bufs, self._bufs2, self._pads = tables["buf"], tables["buf2"], tables["pad"]
        self._counters = torch.zeros(8, dtype=torch.int32, device="cuda")
        dist.barrier(group=group)
        return self

    # ------------------------------------------------------------------
    def all_reduce_(self, flat: torch.Tensor, average: bool = True, mode: Optional[int] = None) -> None:
        """In-place sum (or mean) of a flat fp32 CUDA tensor across ranks."""
        if flat.dtype != torch.float32 or not flat.is_contiguous():
            raise TypeError("PeerComm.all_reduce_ needs a contiguous fp32 tensor")
        n = flat.numel()
        if n > self.numel:
            raise ValueError(f"tensor of {n} elements exceeds the symmetric buffer ({self.numel})")
        unit = 8 * self.ws
        n_pad = (n + unit - 1) // unit * unit
        if n_pad != n:
            # the arena pads its length to a multiple of 128 elements; anything else goes via a copy
            tmp = torch.zeros(n_pad, dtype=torch.float32, device=flat.device)
            tmp[:n].copy_(flat)
            self.all_reduce_(tmp, average=average, mode=mode)
            flat.copy_(tmp[:n])
            return
        if mode is None:
            mode = 0 if n * 2 <= ONE_SHOT_MAX_BYTES else 1
        self.epoch += 1
        scale = 1.0 / self.ws if average else 1.0
        _lib.check(_lib.lib().ccb_allreduce(flat.data_ptr(), n, scale, self._bufs, self._bufs2,
                                            self._pads, self.rank, self.ws, self.epoch,
                                            self._counters.data_ptr(), mode, self.timeout_ms,
                                            _lib.stream_ptr()), "allreduce")

    # ------------------------------------------------------------------
    def make_ranges(self, ranges: list[tuple[int, int, int]]) -> torch.Tensor:
        """Device table for :meth:`sharded_reduce_` / :meth:`sharded_gather_` from
        ``(element offset, element count, owner)`` triples (owner -1: replicated).
        Offsets and counts must be multiples of 8 elements."""
        rows = []
        for off, cnt, owner in ranges:
            if off % 8 or cnt % 8:
                raise ValueError(f"range ({off}, {cnt}) is not aligned to 8 elements")
            rows.append([off // 8, cnt // 8, int(owner) & 0xFFFFFFFF])      # third word: {int32 owner, int32 pad}
        t = torch.tensor(rows, dtype=torch.int64).reshape(-1, 3)
        return t.to("cuda")

    def sharded_reduce_(self, flat_grad: torch.Tensor, ranges: torch.Tensor, average: bool = True) -> None:
        """Sums the owned and the replicated ranges of ``flat_grad`` over ranks, in
        place; ranges owned by other ranks are left untouched (stale)."""
        n = flat_grad.numel()
        if flat_grad.dtype != torch.float32 or n % 8 or n > self.numel:
            raise ValueError("sharded_reduce_ needs an fp32 flat tensor, length % 8 == 0, within the buffer")
        self.epoch += 1
        self._sharded(0, flat_grad, None, n, 1.0 / self.ws if average else 1.0, ranges)

    def sharded_gather_(self, flat_param: torch.Tensor, ranges: torch.Tensor) -> None:
        """Publishes this rank's owned ranges of the bf16 ``flat_param`` and pulls every
        other owner's ranges from its buffer.  Must follow ``sharded_reduce_`` of the same step."""
        if flat_param.dtype != torch.bfloat16:
            raise TypeError("sharded_gather_ moves bf16 parameters")
        self._sharded(1, None, flat_param, flat_param.numel() // 8 * 8, 1.0, ranges)

    def _sharded(self, phase, grad, param, n, scale, ranges) -> None:
        _lib.check(_lib.lib().ccb_sharded_sync(
            phase, _lib.ptr(grad), _lib.ptr(param), n, scale, ranges.data_ptr(), ranges.shape[0], self._bufs,
            self._bufs2, self._pads, self.rank, self.ws, self.epoch, self._counters.data_ptr(), self.timeout_ms,
            _lib.stream_ptr()), "sharded_sync")

    def close(self) -> None:
        L = _lib.lib()
        torch.cuda.synchronize()
        for p in self._opened:
            L.ccb_ipc_close(p)
        for p in self._own:
            L.ccb_comm_free(p)
        self._opened, self._own = [], []
