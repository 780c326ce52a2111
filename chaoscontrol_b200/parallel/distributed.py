"""Data-parallel primitives: parameter broadcast, gradient all-reduce, fused
grad clip, stop-flag consensus, rank resolution.

Public names and contracts follow src/chaoscontrol/distributed.py:34-274 of
the reference.  The differences are where the bytes live: when the model owns
a :class:`~chaoscontrol_b200.utils.arena.ParamArena` the gradients already sit
in one flat fp32 buffer, so the all-reduce is a single collective on that
buffer with no flatten / unflatten copies, and the clip is three small kernel
launches on it.  On a B200 node the collective itself is the NVLink
peer-memory kernel of :mod:`.symm` when that layer is up, NCCL otherwise.
"""
from __future__ import annotations

import os
from typing import Iterable, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..utils.arena import get_arena


def broadcast_params(model: torch.nn.Module) -> None:
    """Make every rank start from rank 0's parameters: one flat broadcast when the parameters share
    an arena -- through rank 0's symmetric buffer when the peer-memory communicator is up, a library
    broadcast otherwise -- and per-tensor broadcasts without an arena."""
    arena = get_arena(model)
    if arena is not None:
        from . import symm
        comm = symm.active_comm(None)
        flat = arena.flat_param
        nbytes = flat.numel() * flat.element_size()
        if comm is not None and flat.is_cuda and nbytes % 16 == 0 and nbytes <= comm.numel * 2:
            comm.broadcast_(flat, src=0)
            return
        dist.broadcast(flat, src=0)
        return
    for p in model.parameters():
        dist.broadcast(p.data, src=0)


def allreduce_grads(model: torch.nn.Module, world_size: int, *,
                    group: "dist.ProcessGroup | None" = None,
                    op: "dist.ReduceOp" = dist.ReduceOp.AVG,
                    materialize_zeros: bool = False) -> None:
    """Reduce all parameter gradients across ranks with ONE collective.

    ``op=AVG`` averages; ``op=SUM`` with caller-side pre-scaling lets ranks with
    different roles join one reduction.  ``materialize_zeros`` fills missing
    grads with zeros so every rank contributes an identically shaped buffer.
    Gradient tensors keep their identity (``data_ptr``) across the call.
    """
    arena = get_arena(model)
    if arena is not None and arena.grads_fresh:
        if getattr(arena, "grads_reduced", False):
            arena.grads_reduced = False              # the engine's overlapped exchange already ran
            return
        _allreduce_flat(arena.flat_grad, world_size, group, op)
        return
    if materialize_zeros:
        for p in model.parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)
    grads = [p.grad for p in model.parameters() if p.grad is not None]
    if not grads:
        return
    flat = torch._utils._flatten_dense_tensors(grads)
    _allreduce_flat(flat, world_size, group, op)
    for g, s in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
        g.copy_(s)


def _allreduce_flat(flat: torch.Tensor, world_size: int, group, op) -> None:
    from . import symm
    comm = symm.active_comm(group)
    if comm is not None and flat.is_cuda and op in (dist.ReduceOp.AVG, dist.ReduceOp.SUM):
        comm.all_reduce_(flat, average=(op == dist.ReduceOp.AVG))
        return
    if op == dist.ReduceOp.AVG and not flat.is_cuda:
        # gloo has no AVG: sum then scale
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        flat.div_(dist.get_world_size(group))
        return
    dist.all_reduce(flat, op=op, group=group)


class AsyncGradAllReducer:
    """Per-parameter asynchronous all-reduce launched from post-accumulate-grad
    hooks so communication overlaps the rest of backward; ``wait()`` before the
    clip / optimizer step (cf. distributed.py:100-172 of the reference)."""

    def __init__(self, model: torch.nn.Module, world_size: int, *, group=None) -> None:
        self.world_size = int(world_size)
        self.group = group
        self._handles: list = []
        self._works: list = []
        self._closed = False
        if self.world_size > 1:
            for p in model.parameters():
                if p.requires_grad:
                    self._handles.append(p.register_post_accumulate_grad_hook(self._hook))

    def _hook(self, p: torch.Tensor) -> None:
        if self._closed or p.grad is None:
            return
        if p.grad.is_cuda:
            work = dist.all_reduce(p.grad, op=dist.ReduceOp.AVG, group=self.group, async_op=True)
            self._works.append((work, None))
        else:
            work = dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._works.append((work, p.grad))

    def wait(self) -> None:
        for work, cpu_grad in self._works:
            work.wait()
            if cpu_grad is not None:
                cpu_grad.div_(self.world_size)
        self._works.clear()

    def close(self) -> None:
        self.wait()
        for h in self._handles:
            h.remove()
        self._handles.clear()
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def clip_grad_norm_fused(parameters: Iterable[torch.nn.Parameter], max_norm: float,
                         norm_type: float = 2.0) -> torch.Tensor:
    """Global L2 clip with an unconditional multiply (no host sync); returns the
    pre-clip norm.  Same tolerance contract as ``torch.nn.utils.clip_grad_norm_``."""
    if float(norm_type) != 2.0:
        raise NotImplementedError("clip_grad_norm_fused only implements L2 (norm_type=2.0); "
                                  "fall back to torch.nn.utils.clip_grad_norm_ for other norms.")
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return torch.zeros(())
    flat = torch._utils._flatten_dense_tensors(grads)
    total_norm = flat.norm(p=2)
    coef = torch.clamp(max_norm / (total_norm + 1e-6), max=1.0)
    flat.mul_(coef)
    for g, s in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
        g.copy_(s)
    return total_norm


def clip_arena_grad_norm(arena, max_norm: float) -> torch.Tensor:
    """Clip the arena's flat fp32 gradient in place; returns the norm (device scalar)."""
    g = arena.flat_grad
    if g.is_cuda:
        stat = torch.empty(3, dtype=torch.float32, device=g.device)
        _lib.check(_lib.lib().ccb_clip_grad_norm(g.data_ptr(), g.numel(), float(max_norm),
                                                 stat.data_ptr(), _lib.stream_ptr()), "clip")
        return stat[2]
    total = g.norm(p=2)
    g.mul_(torch.clamp(max_norm / (total + 1e-6), max=1.0))
    return total


def should_stop_now(local_should_stop: bool, device: torch.device, ddp_active: bool, *,
                    group: "dist.ProcessGroup | None" = None) -> bool:
    """Any rank wants to stop => every rank stops on the same step.  All ranks run the same
    exchange unconditionally when DDP is active.

    With the peer-memory communicator the flag travels through the signal pads (one one-warp kernel,
    no library collective), and it carries a second bit: "one of my peer-memory collectives timed
    out since the last check".  If any rank reports that, EVERY rank marks the communicator dead and
    raises ``PeerCommError`` here, on the same step, instead of stepping on unreduced gradients.
    """
    if not ddp_active:
        return local_should_stop
    from . import symm
    comm = symm.active_comm(group)
    if comm is not None and device.type == "cuda":
        from .peer import PeerCommError
        value = (1 if local_should_stop else 0) | (2 if comm.timed_out() else 0)
        got = comm.flag_max(value)
        if got >= 2:
            comm.dead = True
            raise PeerCommError("a rank reported that a peer-memory collective timed out: gradients of the "
                                "last steps may be unreduced; stopping on every rank")
        return got == 1
    flag = torch.tensor([1.0 if local_should_stop else 0.0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    return flag.item() > 0.5


def resolve_ddp_context(rank: Optional[int], world_size: Optional[int]) -> tuple[int, int]:
    """(rank, world_size) from explicit args, the initialised process group, the
    torchrun environment, or (0, 1)."""
    if rank is not None and world_size is not None:
        return int(rank), int(world_size)
    if rank is not None or world_size is not None:
        raise ValueError("rank and world_size must both be provided, or both be None. "
                         f"Got rank={rank}, world_size={world_size}.")
    if dist.is_available() and dist.is_initialized():
        return int(dist.get_rank()), int(dist.get_world_size())
    er, ew = os.environ.get("RANK"), os.environ.get("WORLD_SIZE")
    if er is not None and ew is not None:
        return int(er), int(ew)
    return 0, 1
