"""Distributed Muon: every rank reduces, orthogonalises and updates only the
matrices it owns, then the updated parameters are gathered.

Per step (``ws`` ranks, flat gradient ``g``, flat bf16 parameters ``p``):

1. *reduce*: gradients are staged once as bf16; each rank sums, from all
   peers' staging buffers, the ranges it owns plus the small replicated ranges
   (everything AdamW updates).  Bytes in per GPU are those of a reduce-scatter.
2. *clip*: the global norm needs one scalar all-reduce of the owned partial
   sums of squares.
3. *update*: momentum, Newton-Schulz (tcgen05 GEMMs) and the apply run on the
   owned sub-batch of each shape group, i.e. ``1/ws`` of the optimizer's FLOPs;
   AdamW runs replicated.  (Momentum buffers keep their full-size layout for
   checkpoint compatibility; only the owned slices are read or written.)
4. *gather*: owned parameter ranges are published through the same staging
   buffer and pulled by every peer.

Steps 1 and 4 are the in-kernel peer-memory collectives of ``csrc/comm.cu``
(``PeerComm.sharded_reduce_`` / ``sharded_gather_``).  Without peer memory
(CPU / gloo, or one rank) the same ownership plan runs on ``torch.distributed``
collectives, which is what the CPU tests exercise.

The reference ships this scheme only in its vendored contest baseline
(baselines/parameter_golf/sota/train_gpt.py:123-268: reduce-scatter per bank,
NS on the shard, all-gather overlapped with the next bank).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..optim.muon import Muon
from ..utils.arena import ParamArena

__all__ = ["OwnershipPlan", "plan_ownership", "DistributedMuon"]


@dataclass
class OwnershipPlan:
    world_size: int
    shards: list[list[tuple[int, int]]]            # [rank][group] -> (first matrix, end matrix) owned
    ranges: list[tuple[int, int, int]]             # (element offset, element count, owner | -1)
    norm_ranges: list[tuple[int, int, int]]        # disjoint cover of all gradients, for the global norm

    def owned(self, rank: int) -> list[tuple[int, int]]:
        return self.shards[rank]


def plan_ownership(arena: ParamArena, world_size: int) -> OwnershipPlan:
    """Contiguous sub-batches of every shape group, handed out so that the
    Newton-Schulz cost (~ rows * cols * min(rows, cols) per matrix) is balanced:
    groups are visited most expensive first and each group's chunks start at the
    rank with the least load so far."""
    load = [0.0] * world_size
    shards: list[list[tuple[int, int]]] = [[(0, 0)] * len(arena.muon_groups) for _ in range(world_size)]
    ranges: list[tuple[int, int, int]] = []
    norm_ranges: list[tuple[int, int, int]] = []
    order = sorted(range(len(arena.muon_groups)),
                   key=lambda i: -(arena.muon_groups[i].shape[0] * arena.muon_groups[i].shape[1] *
                                   min(arena.muon_groups[i].shape)))
    for gi in order:
        g = arena.muon_groups[gi]
        r, c = g.shape
        per = r * c
        cost = float(per * min(r, c))
        chunks = min(g.count, world_size)
        base, extra = divmod(g.count, chunks)
        start_rank = min(range(world_size), key=lambda k: load[k])
        first = 0
        for j in range(chunks):
            n = base + (1 if j < extra else 0)
            rank = (start_rank + j) % world_size
            shards[rank][gi] = (first, first + n)
            ranges.append((g.offset + first * per, n * per, rank))
            # matrices that ride along in the batch but belong to AdamW are counted with the replicated set
            norm_ranges += [(g.offset + m * per, per, rank) for m in range(first, first + n) if m not in g.skip]
            load[rank] += n * cost
            first += n
    for a0, a1 in arena.adamw_ranges:
        lo, hi = a0 // 8 * 8, (a1 + 7) // 8 * 8
        ranges.append((lo, hi - lo, -1))
        norm_ranges.append((a0, a1 - a0, -1))
    return OwnershipPlan(world_size, shards, ranges, norm_ranges)


class DistributedMuon:
    """Wraps an arena-bound :class:`Muon`; ``step()`` replaces the pair
    "all-reduce gradients, optimizer step" of plain data parallelism."""

    def __init__(self, optimizer: Muon, arena: ParamArena, *, group=None, comm=None,
                 grad_clip_norm: float = 0.0) -> None:
        self.opt, self.arena, self.group, self.comm = optimizer, arena, group, comm
        self.ws = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.ws > 1 else 0
        self.grad_clip_norm = float(grad_clip_norm)
        self.plan = plan_ownership(arena, self.ws)
        optimizer.bind_arena(arena)
        optimizer.set_arena_shard({gi: se for gi, se in enumerate(self.plan.owned(self.rank))}
                                  if self.ws > 1 else None)
        self._use_peer = (comm is not None and arena.flat_param.is_cuda and
                          arena.flat_param.dtype == torch.bfloat16 and arena.flat_grad.numel() % 8 == 0)
        self._ranges_dev = comm.make_ranges(self.plan.ranges) if self._use_peer else None
        # disjoint, so a gradient element is scaled exactly once
        self._mine = [(o, n) for o, n, owner in self.plan.norm_ranges if owner in (self.rank, -1)]

    # ------------------------------------------------------------------ pieces
    def _reduce(self) -> None:
        g = self.arena.flat_grad
        if self.ws == 1:
            return
        if self._use_peer:
            self.comm.sharded_reduce_(g, self._ranges_dev, average=True)
            return
        # collective fallback: same result on the owned + replicated ranges
        dist.all_reduce(g, group=self.group)
        g.div_(self.ws)

    def _clip(self) -> Optional[torch.Tensor]:
        if self.grad_clip_norm <= 0:
            return None
        g = self.arena.flat_grad
        sq = torch.zeros(1, dtype=torch.float32, device=g.device)
        for off, n, owner in self.plan.norm_ranges:
            if owner == self.rank or (owner == -1 and self.rank == 0):
                sq += g[off:off + n].pow(2).sum()
        if self.ws > 1:
            dist.all_reduce(sq, group=self.group)
        norm = sq.sqrt()
        scale = (self.grad_clip_norm / (norm + 1e-6)).clamp(max=1.0)
        for off, n in self._mine:
            g[off:off + n].mul_(scale)
        return norm

    def _gather(self) -> None:
        if self.ws == 1:
            return
        p = self.arena.flat_param
        if self._use_peer:
            self.comm.sharded_gather_(p, self._ranges_dev)
            return
        for off, n, owner in self.plan.ranges:
            if owner >= 0:
                dist.broadcast(p[off:off + n], src=dist.get_global_rank(self.group, owner) if self.group else owner,
                               group=self.group)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self) -> Optional[torch.Tensor]:
        """Returns the pre-clip global gradient norm when clipping is on."""
        arena = self.arena
        if not arena.grads_fresh:
            arena.pull_grads()
        self._reduce()
        norm = self._clip()
        arena.grads_fresh = True
        if not arena.flat_param.is_cuda:
            arena.materialize_grads()          # the host optimizer path reads p.grad
        self.opt.step()
        self._gather()
        return norm

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.opt.zero_grad(set_to_none=set_to_none)

    @property
    def param_groups(self):
        return self.opt.param_groups
