"""``PeerComm``: symmetric buffers over CUDA IPC plus the in-kernel all-reduce of
``csrc/comm.cu``.

One process per GPU on one node.  Each rank allocates a bf16 data buffer, an
fp32 reduced-slice staging buffer and a signal pad, exports them with CUDA IPC,
and maps every peer's copies (handles travel through the process group's object
all-gather).  ``all_reduce_`` then launches the pack / reduce kernels on the
current stream; no NCCL call is involved.

The epoch that tags every collective's flags lives in device memory (slot 15 of the
counter array) and is advanced by the kernels themselves, so a collective's launch
arguments never change: a training step that contains collectives can be captured in
a CUDA graph.

Timeouts: every device-side wait is bounded by ``timeout_ms``; a rank that
never signals makes the others record ``CCB_ERR_PEER_TIMEOUT`` in the status
word and return with their gradients unreduced, instead of hanging.  The host
learns of it from :meth:`PeerComm.check` (the training loops fold it into their
stop-flag consensus, so every rank raises on the same step); a communicator that
saw a timeout is marked dead and refuses further collectives.

Creation is all-or-nothing across the group: every rank reports whether its own
set-up worked, the minimum is taken over the group, and unless every rank
succeeded the buffers are released again everywhere and ``create`` returns
``None`` with the reason kept in :data:`last_failure`.
"""
from __future__ import annotations

import os

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
_lib.register_sig("ccb_allreduce", [vp, i64, C.c_float, vp, vp, vp, i64, i64, vp, i64, i64, vp])
_lib.register_sig("ccb_comm_wait_probe", [vp, i64, i64, vp, vp])
_lib.register_sig("ccb_sharded_sync", [i64, vp, vp, i64, C.c_float, vp, i64, vp, vp, vp, i64, i64, vp, i64, vp])
_lib.register_sig("ccb_allreduce_ranges", [vp, vp, i64, i64, C.c_float, vp, vp, vp, i64, i64, vp, i64, i64, vp])
_lib.register_sig("ccb_comm_bcast", [vp, i64, i64, vp, vp, vp, i64, i64, vp, i64, vp])
_lib.register_sig("ccb_comm_flag_max", [i64, vp, i64, i64, i64, vp, i64, vp])
_lib.register_sig("ccb_comm_clear", [vp, i64])

MAX_RANKS = 8
PAD_ROWS = 8
ONE_SHOT_MAX_BYTES = 64 << 20      # bf16 payload; above this the two-shot kernels run
last_failure: str = ""             # why the most recent PeerComm.create() gave up (empty: it did not)


class PeerCommError(RuntimeError):
    """A peer-memory collective did not complete (a peer's flag never arrived)."""



class PeerComm:
    def __init__(self) -> None:
        self.rank = 0
        self.ws = 1
        self.numel = 0
        self.timeout_ms = 2000
        self._own: list[int] = []
        self._opened: list[int] = []
        self._bufs = self._bufs2 = self._pads = None
        self._counters = None
        self._flag_out = None
        self._flag_seq = 0
        self.group = None
        self.dead = False

    # ------------------------------------------------------------------
    @classmethod
    def create(cls, numel: int, group=None, timeout_ms: int = 2000) -> Optional["PeerComm"]:
        global last_failure
        last_failure = ""
        if not (dist.is_available() and dist.is_initialized()):
            last_failure = "torch.distributed is not initialised"
            return None
        ws = dist.get_world_size(group)
        if ws < 2 or ws > MAX_RANKS:
            last_failure = f"world size {ws} outside 2..{MAX_RANKS}"
            return None
        self = cls()
        self.rank, self.ws, self.timeout_ms, self.group = dist.get_rank(group), ws, timeout_ms, group
        # every rank runs every collective below, whatever happened to it locally: a rank that failed
        # contributes empty handles and a zero to the vote
        err = ""
        handles: dict = {}
        mine: dict = {}
        sizes: dict = {}
        L = None
        try:
            if not _lib.available():
                raise RuntimeError("kernel library or CUDA device unavailable")
            L = _lib.lib()
            unit = 8 * ws
            self.numel = (numel + unit - 1) // unit * unit
            sizes = {"buf": self.numel * 2, "buf2": (self.numel // ws) * 4, "pad": PAD_ROWS * MAX_RANKS * 4}
            for k, nbytes in sizes.items():
                p = L.ccb_comm_malloc(max(nbytes, 256))
                if not p:
                    raise RuntimeError(f"allocation of {nbytes} bytes failed: {L.ccb_last_error().decode()}")
                mine[k] = p
                self._own.append(p)
                h = (C.c_char * 64)()
                _lib.check(L.ccb_ipc_get(p, h), "ipc_get")
                handles[k] = bytes(h)
        except Exception as exc:
            err = f"rank {self.rank}: {type(exc).__name__}: {exc}"
            handles = {}
        gathered: list = [None] * ws
        dist.all_gather_object(gathered, handles, group=group)
        if not err and all(g for g in gathered):
            try:
                tables = {k: (C.c_void_p * MAX_RANKS)() for k in sizes}
                for r in range(ws):
                    for k in sizes:
                        if r == self.rank:
                            tables[k][r] = mine[k]
                        else:
                            p = L.ccb_ipc_open(C.create_string_buffer(gathered[r][k], 64))
                            if not p:
                                raise RuntimeError(f"cannot map rank {r}'s {k}: {L.ccb_last_error().decode()}")
                            self._opened.append(p)
                            tables[k][r] = p
                self._bufs, self._bufs2, self._pads = tables["buf"], tables["buf2"], tables["pad"]
                self._counters = torch.zeros(16, dtype=torch.int32, device="cuda")
                self._flag_out = torch.zeros(1, dtype=torch.int32, device="cuda")
            except Exception as exc:
                err = f"rank {self.rank}: {type(exc).__name__}: {exc}"
        elif not err:
            err = f"rank {self.rank}: a peer could not export its buffers"
        # the vote: the communicator exists only if it exists on every rank
        errs: list = [None] * ws
        dist.all_gather_object(errs, err, group=group)
        bad = [e for e in errs if e]
        if bad:
            last_failure = "; ".join(bad)
            self._release(barriers=True)
            return None
        dist.barrier(group=group)
        return self

    # ------------------------------------------------------------------
    def all_reduce_(self, flat: torch.Tensor, average: bool = True, mode: Optional[int] = None) -> None:
        """In-place sum (or mean) of a flat fp32 CUDA tensor across ranks."""
        self._alive()
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
            forced = os.environ.get("CCB_ALLREDUCE_MODE")          # 0 one-shot, 1 two-shot (A/B measurements)
            mode = int(forced) if forced in ("0", "1") else (0 if n * 2 <= ONE_SHOT_MAX_BYTES else 1)
        scale = 1.0 / self.ws if average else 1.0
        _lib.check(_lib.lib().ccb_allreduce(flat.data_ptr(), n, scale, self._bufs, self._bufs2,
                                            self._pads, self.rank, self.ws,
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
            self._bufs2, self._pads, self.rank, self.ws, self._counters.data_ptr(), self.timeout_ms,
            _lib.stream_ptr()), "sharded_sync")

    # ------------------------------------------------------------------
    def all_reduce_ranges_(self, flat_grad: torch.Tensor, ranges: torch.Tensor, r0: int, r1: int, *,
                           average: bool = True, blocks: int = 0, stream: Optional[int] = None) -> None:
        """One bucket of an overlapped exchange: in-place sum (or mean) of rows ``[r0, r1)`` of a
        :meth:`make_ranges` table (the owner column is ignored), as its own epoch, on ``stream``
        (raw handle; default: the current stream) with ``blocks`` small blocks per kernel."""
        self._alive()
        if flat_grad.dtype != torch.float32 or flat_grad.numel() > self.numel:
            raise ValueError("all_reduce_ranges_ needs an fp32 flat tensor within the symmetric buffer")
        _lib.check(_lib.lib().ccb_allreduce_ranges(
            flat_grad.data_ptr(), ranges.data_ptr(), int(r0), int(r1), 1.0 / self.ws if average else 1.0,
            self._bufs, self._bufs2, self._pads, self.rank, self.ws, self._counters.data_ptr(),
            int(blocks), self.timeout_ms, _lib.stream_ptr() if stream is None else stream), "allreduce_ranges")

    def broadcast_(self, flat: torch.Tensor, src: int = 0) -> None:
        """Every rank's ``flat`` (contiguous, byte length a multiple of 16 and within the buffer)
        becomes a copy of rank ``src``'s, through the root's symmetric buffer."""
        self._alive()
        nbytes = flat.numel() * flat.element_size()
        if not flat.is_contiguous() or nbytes % 16 or nbytes > self.numel * 2:
            raise ValueError("broadcast_ needs a contiguous tensor of 16-byte words within the symmetric buffer")
        _lib.check(_lib.lib().ccb_comm_bcast(flat.data_ptr(), nbytes, int(src), self._bufs, self._bufs2,
                                             self._pads, self.rank, self.ws,
                                             self._counters.data_ptr(), self.timeout_ms, _lib.stream_ptr()),
                   "bcast")

    def flag_max(self, value: int) -> int:
        """Maximum over ranks of a small integer (0..255) exchanged through the signal pads: one
        one-warp kernel and one 4-byte read-back.  Raises :class:`PeerCommError` when a peer did not
        answer within the timeout."""
        self._flag_seq += 1
        _lib.check(_lib.lib().ccb_comm_flag_max(int(value) & 0xFF, self._pads, self.rank, self.ws,
                                                self._flag_seq, self._flag_out.data_ptr(), self.timeout_ms,
                                                _lib.stream_ptr()), "flag_max")
        got = int(self._flag_out.item())
        if got < 0:
            self.dead = True
            _lib.read_status(reset=True)
            raise PeerCommError(f"rank {self.rank}: a peer did not answer the flag exchange within "
                                f"{self.timeout_ms} ms")
        return got

    # ------------------------------------------------------------------
    def _alive(self) -> None:
        if self.dead:
            raise PeerCommError("this communicator saw a peer timeout and is closed for collectives")

    def timed_out(self) -> bool:
        """Synchronises and reads the device status word: True when a collective of this process
        gave up on a peer since the last call (the word is cleared).  Does not change the
        communicator's state; :func:`chaoscontrol_b200.parallel.distributed.should_stop_now` shares
        the answer with the other ranks and then every rank marks it dead and raises together."""
        st = _lib.read_status(reset=False)
        if st == 3:                                     # CCB_ERR_PEER_TIMEOUT
            _lib.read_status(reset=True)
            return True
        return False

    def resync(self) -> None:
        """Collective recovery after a timeout (every rank of the group calls it, between steps, with
        no collective of this communicator in flight): drain the GPU, meet on the host, clear this
        rank's own signal pad and arrival counters, restart the epoch and flag sequence from zero,
        meet again.  Afterwards the communicator is usable as if freshly created; buffers stay mapped."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        own_pad = self._pads[self.rank]
        _lib.check(_lib.lib().ccb_comm_clear(own_pad, PAD_ROWS * MAX_RANKS * 4), "comm_clear")
        self._counters.zero_()                    # arrival counters and the device-resident epoch
        self._flag_seq = 0
        _lib.read_status(reset=True)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self.dead = False

    def _release(self, barriers: bool) -> None:
        """Unmap the peers' buffers, then free this rank's own.  With ``barriers`` every rank first
        drains its GPU, and nobody frees memory that a peer still has mapped."""
        L = _lib.lib() if _lib.available() else None
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if barriers:
            dist.barrier(group=self.group)
        for p in self._opened:
            L.ccb_ipc_close(p)
        self._opened = []
        if barriers:
            dist.barrier(group=self.group)
        for p in self._own:
            L.ccb_comm_free(p)
        self._own = []
        self._bufs = self._bufs2 = self._pads = None

    def close(self, barriers: bool = True) -> None:
        """Collective teardown (call on every rank, before ``destroy_process_group``): synchronise,
        barrier, close the imported handles, barrier, free the exported buffers."""
        if not self._own and not self._opened:
            return
        use_barriers = barriers and dist.is_available() and dist.is_initialized()
        self._release(barriers=use_barriers)
        self.dead = True
