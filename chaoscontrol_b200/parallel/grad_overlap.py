"""Gradient exchange overlapped with backward for the kernel training engine.

The reference ships the idea as per-parameter asynchronous NCCL all-reduces
launched from autograd hooks (src/chaoscontrol/distributed.py:100-172, wired at
experiments/23_fast_path/runner_fast_path.py:10038-10044).  Here the engine has
no autograd graph but knows exactly when each gradient is final, so the arena
is cut into buckets in the order backward produces them::

    bucket 0        lm_head.weight                      ready after the LM-head kernels
    bucket 1 .. L   layer L-1 .. 0: packed projections, out_proj, fc, proj
    bucket L+1      embed.weight + the AdamW tail (norm gains, log_a)    ready last

Each bucket is one pack + one-shot peer-load reduce (``csrc/comm.cu``) with its
own epoch, launched on a side stream behind an event the engine records when
the bucket's last gradient kernel has been queued.  Early buckets use a few
small blocks that share the SMs with the GEMMs still running; the last one
takes the whole GPU because nothing else is left to run.  The optimizer's
stream waits for the side stream once, before the clip.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..utils.arena import ParamArena


class OverlappedGradReducer:
    def __init__(self, arena: ParamArena, comm, layer_names: list[dict], *, early_blocks: int = 32) -> None:
        self.arena, self.comm = arena, comm
        self.early_blocks = int(early_blocks)
        L = len(layer_names)

        def rng(name: str, count_mult: int = 1) -> tuple[int, int, int]:
            off, shp = arena.slots[name]
            n = 1
            for s in shp:
                n *= s
            return (off, n * count_mult, -1)

        rows: list[tuple[int, int, int]] = []
        self.bounds: list[tuple[int, int]] = []

        def close_bucket(start: int) -> None:
            self.bounds.append((start, len(rows)))

        s0 = len(rows)
        rows.append(rng("lm_head.weight"))
        close_bucket(s0)
        for i in reversed(range(L)):
            n = layer_names[i]
            s0 = len(rows)
            rows.append(rng(n["sel"], 4))                    # select | in | gate | delta, adjacent
            rows += [rng(n["out"]), rng(n["fc"]), rng(n["proj"])]
            close_bucket(s0)
        s0 = len(rows)
        rows.append(rng("embed.weight"))
        a0, a1 = arena.adamw_range
        a1 = min((a1 + 7) // 8 * 8, arena.flat_grad.numel())
        rows.append((a0, a1 - a0, -1))
        close_bucket(s0)
        covered = sum(c for _, c, _ in rows)
        used = sum(p.numel() for p in arena.params.values())
        if covered < used:
            raise ValueError(f"gradient buckets cover {covered} of {used} parameters: the arena holds tensors "
                             "the engine's bucket plan does not know")
        self.table = comm.make_ranges(rows)
        self.side = torch.cuda.Stream()
        self._ready = [torch.cuda.Event() for _ in self.bounds]
        self._done = torch.cuda.Event()
        self.n_buckets = len(self.bounds)

    # bucket indices as the engine names them
    @property
    def head_bucket(self) -> int:
        return 0

    def layer_bucket(self, layer: int, num_layers: int) -> int:
        return 1 + (num_layers - 1 - layer)

    @property
    def last_bucket(self) -> int:
        return self.n_buckets - 1

    def bucket_ready(self, k: int) -> None:
        """Call on the engine's stream once every kernel writing bucket ``k`` has been queued."""
        ev = self._ready[k]
        ev.record()
        self.side.wait_event(ev)
        r0, r1 = self.bounds[k]
        blocks = 0 if k == self.last_bucket else self.early_blocks
        self.comm.all_reduce_ranges_(self.arena.flat_grad, self.table, r0, r1, average=True, blocks=blocks,
                                     stream=self.side.cuda_stream)

    def finish(self) -> None:
        """The current stream continues only after every bucket has been reduced."""
        self._done.record(self.side)
        torch.cuda.current_stream().wait_event(self._done)
        self.arena.grads_reduced = True         # type: ignore[attr-defined]


#: measured per-direction peer bandwidth of this pool's B200s (bytes / s), for the overlap rule below
PEER_BYTES_PER_S = 770e9
#: overlap only when the exchange left exposed at the end of the step would exceed this many seconds
OVERLAP_MIN_EXPOSED_S = 0.4e-3


def overlap_wanted(payload_bytes: int, world_size: int) -> bool:
    """``CCB_GRAD_OVERLAP=1`` / ``0`` forces the bucketed, overlapped exchange on / off.  Unset: overlap
    only when one exchange after backward would take longer than ``OVERLAP_MIN_EXPOSED_S`` (bf16 payload
    read from ``world_size - 1`` peers at the measured peer bandwidth).  Measured on 4 x B200 with the
    10.8 M-parameter submission model (21.5 MB payload, ~0.1 ms of peer reads): one exchange after
    backward 33.15-33.19 ms per step, six overlapped buckets 33.54-33.62 ms, one GPU alone 32.61 ms;
    the side-stream kernels cost the concurrent backward more than the ~0.1 ms they hide."""
    import os
    env = os.environ.get("CCB_GRAD_OVERLAP")
    if env is not None:
        return env != "0"
    return payload_bytes * max(world_size - 1, 0) / PEER_BYTES_PER_S > OVERLAP_MIN_EXPOSED_S


def reducer_for(engine, world_size: int, group=None, *, force: bool = False) -> Optional[OverlappedGradReducer]:
    """The engine's cached reducer when the overlapped exchange is wanted (:func:`overlap_wanted`, or
    ``force``: the caller asked for the overlapped mode by name) and the peer-memory communicator of
    ``group`` is alive and spans ``world_size`` ranks, else None (the caller reduces once after the step)."""
    from . import symm
    if not engine.arena.flat_grad.is_cuda:
        return None
    if not force and not overlap_wanted(engine.arena.flat_grad.numel() * 2, world_size):
        return None
    comm = symm.active_comm(group)
    if comm is None or comm.ws != world_size:
        return None
    red = getattr(engine, "_reducer", None)
    if red is None or red.comm is not comm:
        red = OverlappedGradReducer(engine.arena, comm, engine._names)
        engine._reducer = red
    return red
