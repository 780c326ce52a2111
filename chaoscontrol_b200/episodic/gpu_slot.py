"""Device-resident slot tensor that carries episodic write payloads and query
candidates between ranks in one collective per step
(layout of src/chaoscontrol/episodic/gpu_slot.py:50-261).

One fp32 row per payload, ``slot_dim = 8 + 2*S + 2*D`` cells::

    0 valid_mask | 1 pressure | 2 pre_write_ce | 3 protection_score
    4..5 key_fp (int64 bits) | 6..7 value_anchor_id (int64 bits)
    8..8+2S value_tok_ids (S int64) | key_rep (D fp32) | residual (D fp32)

int64 fields are reinterpretations of even-aligned fp32 pairs, which is why
the row width must stay even and the tensor fp32 and contiguous.

``pack_payload`` / ``unpack_payload`` handle one row.  ``pack_payload_rows`` /
``unpack_payload_rows`` move ALL rows of a step with a handful of vectorised
device ops (no per-row host round trips), which is the path a training step
should use.
"""
from __future__ import annotations

from typing import Any

import torch

__all__ = ["SLOT_DIM_BASE", "slot_dim", "make_slot_tensor", "pack_payload", "unpack_payload",
           "pack_payload_rows", "unpack_payload_rows"]

SLOT_DIM_BASE = 8


def slot_dim(*, span_length: int, key_rep_dim: int) -> int:
    if span_length <= 0:
        raise ValueError(f"span_length must be positive; got {span_length}")
    if key_rep_dim <= 0:
        raise ValueError(f"key_rep_dim must be positive; got {key_rep_dim}")
    width = SLOT_DIM_BASE + 2 * int(span_length) + 2 * int(key_rep_dim)
    assert width % 2 == 0, "slot rows must start on 8-byte boundaries for the int64 fields"
    return width


def make_slot_tensor(*, k_max: int, span_length: int, key_rep_dim: int, device,
                     dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Zeroed ``[k_max, slot_dim]``: every row starts invalid (``valid_mask`` 0)."""
    if k_max <= 0:
        raise ValueError(f"k_max must be positive; got {k_max}")
    if dtype != torch.float32:
        raise ValueError("make_slot_tensor requires dtype=torch.float32 so the int64-via-view reinterpret "
                         f"aligns; got dtype={dtype}")
    return torch.zeros(int(k_max), slot_dim(span_length=span_length, key_rep_dim=key_rep_dim), device=device,
                       dtype=dtype)


def _check_row(slot: torch.Tensor, S: int, D: int) -> None:
    width = slot_dim(span_length=S, key_rep_dim=D)
    if slot.dim() != 1 or slot.shape[0] != width:
        raise ValueError(f"slot must have shape ({width},); got {tuple(slot.shape)}")
    if slot.dtype != torch.float32:
        raise ValueError(f"slot must be fp32; got dtype={slot.dtype}")
    if not slot.is_contiguous():
        raise ValueError("slot must be contiguous for the int64 reinterpret")


def pack_payload(slot: torch.Tensor, *, valid_mask: float, pressure: float, key_fp: int, value_anchor_id: int,
                 value_tok_ids: torch.Tensor, key_rep: torch.Tensor, residual: torch.Tensor, span_length: int,
                 key_rep_dim: int, pre_write_ce: float = float("nan"), protection_score: float = 0.0) -> None:
    """Writes one payload into a ``[slot_dim]`` row view, in place."""
    S, D = int(span_length), int(key_rep_dim)
    _check_row(slot, S, D)
    for name, t, n in (("value_tok_ids", value_tok_ids, S), ("key_rep", key_rep, D), ("residual", residual, D)):
        if t.shape != (n,):
            raise ValueError(f"{name} must have shape ({n},); got {tuple(t.shape)}")
    slot[0], slot[1], slot[2], slot[3] = float(valid_mask), float(pressure), float(pre_write_ce), float(protection_score)
    slot[4:6].view(torch.int64)[0] = int(key_fp)
    slot[6:8].view(torch.int64)[0] = int(value_anchor_id)
    slot[8:8 + 2 * S].view(torch.int64).copy_(value_tok_ids.detach().to(torch.int64))
    slot[8 + 2 * S:8 + 2 * S + D].copy_(key_rep.detach().to(torch.float32))
    slot[8 + 2 * S + D:8 + 2 * S + 2 * D].copy_(residual.detach().to(torch.float32))


def unpack_payload(slot: torch.Tensor, *, span_length: int, key_rep_dim: int) -> dict[str, Any]:
    """One row as Python scalars and cloned tensors."""
    S, D = int(span_length), int(key_rep_dim)
    _check_row(slot, S, D)
    head = slot[:4].tolist()
    ints = slot[4:8].view(torch.int64).tolist()
    return {"valid_mask": head[0], "pressure": head[1], "pre_write_ce": head[2], "protection_score": head[3],
            "key_fp": int(ints[0]), "value_anchor_id": int(ints[1]),
            "value_tok_ids": slot[8:8 + 2 * S].view(torch.int64).clone(),
            "key_rep": slot[8 + 2 * S:8 + 2 * S + D].clone(),
            "residual": slot[8 + 2 * S + D:8 + 2 * S + 2 * D].clone()}


def pack_payload_rows(slots: torch.Tensor, *, pressure: torch.Tensor, key_fp: torch.Tensor,
                      value_anchor_id: torch.Tensor, value_tok_ids: torch.Tensor, key_rep: torch.Tensor,
                      residual: torch.Tensor, pre_write_ce: torch.Tensor | None = None,
                      protection_score: torch.Tensor | None = None) -> int:
    """Fills the first ``N`` rows of ``slots [K, slot_dim]`` from batched fields
    (``value_tok_ids [N, S]``, ``key_rep`` / ``residual [N, D]``, the rest ``[N]``) and
    zeroes the remaining rows.  Returns ``N``.  Everything stays on the device."""
    N, S = value_tok_ids.shape
    D = key_rep.shape[1]
    if slots.shape[1] != slot_dim(span_length=S, key_rep_dim=D) or slots.dtype != torch.float32:
        raise ValueError(f"slots must be fp32 [K, {slot_dim(span_length=S, key_rep_dim=D)}]; got "
                         f"{tuple(slots.shape)} {slots.dtype}")
    if N > slots.shape[0]:
        raise ValueError(f"{N} payloads do not fit {slots.shape[0]} slot rows")
    slots.zero_()
    rows = slots[:N]
    dev = slots.device
    rows[:, 0] = 1.0
    rows[:, 1] = pressure.to(dev, torch.float32)
    rows[:, 2] = float("nan") if pre_write_ce is None else pre_write_ce.to(dev, torch.float32)
    rows[:, 3] = 0.0 if protection_score is None else protection_score.to(dev, torch.float32)
    as_i64 = slots.view(torch.int64)                           # [K, slot_dim / 2]
    as_i64[:N, 2] = key_fp.to(dev, torch.int64)
    as_i64[:N, 3] = value_anchor_id.to(dev, torch.int64)
    as_i64[:N, 4:4 + S] = value_tok_ids.to(dev, torch.int64)
    rows[:, 8 + 2 * S:8 + 2 * S + D] = key_rep.to(dev, torch.float32)
    rows[:, 8 + 2 * S + D:] = residual.to(dev, torch.float32)
    return N


def unpack_payload_rows(slots: torch.Tensor, *, span_length: int, key_rep_dim: int) -> dict[str, torch.Tensor]:
    """All valid rows (``valid_mask > 0.5``) as batched tensors; one mask, no per-row sync."""
    S, D = int(span_length), int(key_rep_dim)
    if slots.dim() != 2 or slots.shape[1] != slot_dim(span_length=S, key_rep_dim=D):
        raise ValueError(f"slots must be [K, {slot_dim(span_length=S, key_rep_dim=D)}]; got {tuple(slots.shape)}")
    rows = slots[slots[:, 0] > 0.5].contiguous()
    as_i64 = rows.view(torch.int64)
    return {"pressure": rows[:, 1], "pre_write_ce": rows[:, 2], "protection_score": rows[:, 3],
            "key_fp": as_i64[:, 2], "value_anchor_id": as_i64[:, 3], "value_tok_ids": as_i64[:, 4:4 + S],
            "key_rep": rows[:, 8 + 2 * S:8 + 2 * S + D], "residual": rows[:, 8 + 2 * S + D:]}
