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

    def close(self) -> None:
        L = _lib.lib()
        torch.cuda.synchronize()
        for p in self._opened:
            L.ccb_ipc_close(p)
        for p in self._own:
            L.ccb_comm_free(p)
        self._opened, self._own = [], []
