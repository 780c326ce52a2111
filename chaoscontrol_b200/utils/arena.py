"""Flat parameter / gradient storage for the kernel training path.

``ParamArena.install(model)`` re-homes every parameter of a bare-SSM
``CareStudentLM`` as a view into one contiguous buffer, ordered so that

* the four ``[D, D]`` content projections of a layer (select, in, gate, delta)
  are adjacent -> the trunk reads them as one packed ``[4D, D]`` weight with no
  concatenation;
* Muon's matrix parameters are grouped by shape -> every shape group is
  literally a ``[G, rows, cols]`` tensor for the batched Newton-Schulz GEMMs;
* everything updated by AdamW (norm gains, ``log_a``, ``delta_proj``) forms one
  contiguous tail -> one multi-tensor kernel launch;

and allocates a matching flat fp32 gradient buffer that the hand-scheduled
backward writes into.  Gradient all-reduce, clipping and the optimizer then
work on flat ranges: no flatten / unflatten copies (the reference's
``allreduce_grads`` flattens and copies back every step,
src/chaoscontrol/distributed.py:86-97).

State-dict keys are untouched: parameters keep their names, only their
storage moves.  ``model.to(dtype)`` after installation breaks the views; call
``install`` last.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Optional

import torch
import torch.nn as nn


@dataclass
class ArenaGroup:
    """One Muon shape group: ``count`` matrices of ``shape`` stored back to back."""
    shape: tuple[int, int]
    names: list[str]
    offset: int            # element offset of the first matrix in the flat buffers
    count: int = 0
    skip: set = field(default_factory=set)   # batch indices whose update is not applied

    @property
    def numel(self) -> int:
        return self.count * self.shape[0] * self.shape[1]


@dataclass
class ParamArena:
    flat_param: torch.Tensor                       # model dtype
    flat_grad: torch.Tensor                        # fp32
    slots: dict[str, tuple[int, tuple[int, ...]]]  # name -> (offset, shape)
    muon_groups: list[ArenaGroup]
    adamw_range: tuple[int, int]                   # [start, end) element range
    adamw_names: list[str]
    params: dict[str, nn.Parameter] = field(default_factory=dict)
    grads_fresh: bool = False
    _grad_lowp: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------
    @staticmethod
    def _is_muon(name: str, p: torch.Tensor) -> bool:
        if name.endswith(".delta_proj.weight") or ".delta_proj." in name:
            return False
        return p.ndim == 2

    @classmethod
    def install(cls, model: nn.Module) -> "ParamArena":
        named = [(n, p) for n, p in model.named_parameters()]
        if not named:
            raise ValueError("model has no parameters")
        dtype = named[0][1].dtype
        device = named[0][1].device
        if any(p.dtype != dtype or p.device != device for _, p in named):
            raise ValueError("ParamArena needs all parameters on one device with one dtype")
        by_name = dict(named)

        # 1. per-layer packed projections first (they are [D, D] Muon / AdamW members
        #    too, so remember where they land and build the groups from offsets).
        order: list[str] = []
        packed_sets: list[list[str]] = []
        for n, _ in named:
            if n.endswith(".core.select_proj.weight"):
                base = n[: -len("select_proj.weight")]
                quad = [base + s for s in ("select_proj.weight", "in_proj.weight", "gate_proj.weight",
                                           "delta_proj.weight")]
                if all(q in by_name and by_name[q].shape == by_name[n].shape for q in quad):
                    packed_sets.append(quad)
        packed_members = {q for quad in packed_sets for q in quad}

        # Muon groups by shape.  Packed members of shape [D, D] stay in their packed
        # position; the [D, D] group is then described by an index list instead of
        # one contiguous range, so keep them out of the contiguous groups and give
        # them their own "strided" group below.
        shapes: dict[tuple[int, int], list[str]] = {}
        adamw: list[str] = []
        for n, p in named:
            if n in packed_members:
                continue
            if cls._is_muon(n, p):
                shapes.setdefault(tuple(p.shape), []).append(n)
            else:
                adamw.append(n)

        offset = 0
        slots: dict[str, tuple[int, tuple[int, ...]]] = {}

        def place(n: str) -> None:
            nonlocal offset
            p = by_name[n]
            slots[n] = (offset, tuple(p.shape))
            offset += p.numel()
            offset = (offset + 127) // 128 * 128      # keep every tensor 256-byte aligned

        muon_groups: list[ArenaGroup] = []
        adamw_ranges: list[tuple[int, int]] = []
        # Packed quads are laid out [select, in, gate, delta] x L back to back.  The
        # whole run is ONE batch of 4L matrices for Newton-Schulz; delta_proj (an
        # AdamW parameter) rides along and its result is discarded (`skip`), which
        # costs a few percent of a sub-millisecond op and keeps the batch dense.
        if packed_sets:
            D0, D1 = by_name[packed_sets[0][0]].shape
            assert (D0 * D1) % 128 == 0, "packed projections need numel % 128 == 0"
            g = ArenaGroup(shape=(D0, D1), names=[], offset=offset)
            for quad in packed_sets:
                for j, q in enumerate(quad):
                    if j == 3:
                        adamw_ranges.append((offset, offset + by_name[q].numel()))
                    place(q)
                    g.names.append(q)
            g.count = len(g.names)
            g.skip = {i for i in range(g.count) if i % 4 == 3}
            muon_groups.append(g)
        for shp, names in sorted(shapes.items(), key=lambda kv: (kv[0][0] * kv[0][1], kv[0])):
            # a shape group is read as a dense [count, r, c] batch (stride r * c) by Muon and by the
            # ownership plan, while `place` pads every tensor to 128 elements: the two agree only when
            # r * c is a multiple of 128; the Newton-Schulz GEMMs want 8-element aligned rows and columns
            if (shp[0] * shp[1]) % 128 or shp[0] % 8 or shp[1] % 8:
                raise ValueError(f"ParamArena: matrix shape {shp} ({names[0]}) needs rows and columns in "
                                 "multiples of 8 and rows * columns in multiples of 128")
            g = ArenaGroup(shape=shp, names=list(names), offset=offset, count=len(names))
            for n in names:
                place(n)
            muon_groups.append(g)
        a0 = offset
        for n in adamw:
            place(n)
        a1 = offset
        adamw_ranges.append((a0, a1))

        flat_param = torch.zeros(offset, dtype=dtype, device=device)
        flat_grad = torch.zeros(offset, dtype=torch.float32, device=device)
        arena = cls(flat_param=flat_param, flat_grad=flat_grad, slots=slots, muon_groups=muon_groups,
                    adamw_range=(a0, a1), adamw_names=adamw)
        arena.packed_sets = packed_sets          # type: ignore[attr-defined]
        arena.adamw_ranges = adamw_ranges        # type: ignore[attr-defined]
        with torch.no_grad():
            for n, p in named:
                off, shp = slots[n]
                view = flat_param[off: off + p.numel()].view(shp)
                view.copy_(p.data)
                p.data = view
                arena.params[n] = p
        model._ccb_arena = arena                 # type: ignore[attr-defined]
        return arena

    # ------------------------------------------------------------------
    def param_view(self, name: str) -> torch.Tensor:
        off, shp = self.slots[name]
        n = 1
        for s in shp:
            n *= s
        return self.flat_param[off: off + n].view(shp)

    def grad_view(self, name: str) -> torch.Tensor:
        off, shp = self.slots[name]
        n = 1
        for s in shp:
            n *= s
        return self.flat_grad[off: off + n].view(shp)

    def zero_grad(self) -> None:
        self.flat_grad.zero_()
        self.grads_fresh = False

    def materialize_grads(self) -> None:
        """Expose the flat fp32 gradients as ``p.grad`` in the parameter dtype."""
        if self.flat_param.dtype == torch.float32:
            src = self.flat_grad
        else:
            if self._grad_lowp is None:
                self._grad_lowp = torch.empty_like(self.flat_param)
            self._grad_lowp.copy_(self.flat_grad)
            src = self._grad_lowp
        for n, p in self.params.items():
            off, shp = self.slots[n]
            p.grad = src[off: off + p.numel()].view(shp)

    def pull_grads(self) -> None:
        """Inverse of :meth:`materialize_grads`: gather ``p.grad`` into the flat buffer."""
        for n, p in self.params.items():
            g = self.grad_view(n)
            if p.grad is None:
                g.zero_()
            else:
                g.copy_(p.grad)
        self.grads_fresh = True

    def still_valid(self) -> bool:
        """True while every parameter is still a view of the flat buffer."""
        base = self.flat_param.data_ptr()
        es = self.flat_param.element_size()
        for n, p in self.params.items():
            if p.data_ptr() != base + self.slots[n][0] * es or p.dtype != self.flat_param.dtype:
                return False
        return True


def get_arena(model: nn.Module) -> Optional[ParamArena]:
    arena = getattr(model, "_ccb_arena", None)
    if arena is not None and not arena.still_valid():
        return None
    return arena
