"""Ordered slot-mutation records between memory-serving ranks.

The maintenance rank decides what happens to a slot; the packet-serving rank
holds the low-latency mirror that feeds residual packets.  A ``SlotCommit`` is
the small record that carries one decision across (public surface of the
reference's src/chaoscontrol/slot_commit.py:18-250).  A commit names the
generation it was computed against; a mirror at another generation drops it
(stale) and keeps serving what it has.

Dispatch here is a table from action to handler rather than an if-chain, so a
new action is one entry.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum
from typing import Any, Callable

import torch

from .slot_table import SlotTable

__all__ = ["SlotCommit", "SlotCommitAction", "SlotCommitDType", "apply_slot_commit_to_model",
           "apply_append_slot_commit_to_model", "slot_commit_dtype_code", "slot_commit_dtype_from_code"]


class SlotCommitAction(IntEnum):
    APPEND = 0
    PRESERVE = 1
    DECAY = 2
    EVICT = 3
    REFRESH = 4
    QUARANTINE = 5
    DISTILL = 6
    RELEASE = 7

    def __str__(self) -> str:
        return self.name


SLOT_COMMIT_APPEND = SlotCommitAction.APPEND
SLOT_COMMIT_PRESERVE = SlotCommitAction.PRESERVE
SLOT_COMMIT_DECAY = SlotCommitAction.DECAY
SLOT_COMMIT_EVICT = SlotCommitAction.EVICT
SLOT_COMMIT_REFRESH = SlotCommitAction.REFRESH
SLOT_COMMIT_QUARANTINE = SlotCommitAction.QUARANTINE
SLOT_COMMIT_DISTILL = SlotCommitAction.DISTILL
SLOT_COMMIT_RELEASE = SlotCommitAction.RELEASE
SLOT_COMMIT_CODE_TO_ACTION = {int(a): a for a in SlotCommitAction}


class SlotCommitDType(IntEnum):
    FLOAT32 = 0
    FLOAT16 = 1
    BFLOAT16 = 2


SLOT_COMMIT_DTYPE_TO_CODE = {torch.float32: SlotCommitDType.FLOAT32, torch.float16: SlotCommitDType.FLOAT16,
                             torch.bfloat16: SlotCommitDType.BFLOAT16}
SLOT_COMMIT_CODE_TO_DTYPE = {v: k for k, v in SLOT_COMMIT_DTYPE_TO_CODE.items()}


def _coerce_action(action) -> SlotCommitAction:
    if isinstance(action, SlotCommitAction):
        return action
    if isinstance(action, str):
        if action not in SlotCommitAction.__members__:
            raise ValueError(f"unknown SlotCommit action: {action}")
        return SlotCommitAction[action]
    try:
        return SlotCommitAction(int(action))
    except ValueError as exc:
        raise ValueError(f"unknown SlotCommit action code: {action}") from exc


@dataclass(frozen=True)
class SlotCommit:
    """One ordered slot mutation.  ``APPEND`` has no base generation; every
    other action must say which generation it was computed against."""

    slot_id: int
    action: Any
    step: int
    base_generation: int | None
    new_generation: int
    bucket_id: int = -1
    event_id: int = 0
    survival_factor: float = 1.0
    tensor: torch.Tensor | None = None
    reason: str = ""

    def __post_init__(self) -> None:
        action = _coerce_action(self.action)
        base = self.base_generation
        if action is SLOT_COMMIT_APPEND:
            if base is not None and int(base) >= 0:
                raise ValueError("APPEND SlotCommit must use base_generation=None")
            base = None
        elif base is None:
            raise ValueError(f"{action.name} SlotCommit requires base_generation")
        else:
            base = int(base)
        for name, val in (("slot_id", int(self.slot_id)), ("action", action), ("step", int(self.step)),
                          ("base_generation", base), ("new_generation", int(self.new_generation)),
                          ("bucket_id", int(self.bucket_id)), ("event_id", int(self.event_id)),
                          ("survival_factor", float(self.survival_factor)), ("reason", str(self.reason))):
            object.__setattr__(self, name, val)


def _resolve(table: SlotTable, c: SlotCommit) -> tuple[int | None, str]:
    """By slot id; failing that, by (event id, bucket) for slots the two ranks
    numbered independently."""
    if table.record(c.slot_id) is not None:
        return c.slot_id, "slot_id"
    if c.event_id == 0:
        return None, "missing_slot"
    for sid in table.active_slot_ids():
        rec = table.record(sid)
        if rec is None or int(rec.event_id) != c.event_id:
            continue
        if c.bucket_id >= 0 and int(rec.bucket_id) != c.bucket_id:
            continue
        return sid, "event_id"
    return None, "missing_slot"


def _stamp(table: SlotTable, sid: int, generation: int) -> None:
    rec = table.record(int(sid))
    if rec is not None:
        rec.write_generation = int(generation)


def _do_refresh(model, table, sid, c):
    if c.tensor is None:
        return False, "missing_tensor"
    table.replace_tensor(sid, c.tensor, bump_generation=False)
    return True, "refreshed"


def _do_decay(model, table, sid, c):
    table.scale_survival(sid, c.survival_factor)
    return True, "decayed"


def _do_quarantine(model, table, sid, c):
    table.quarantine(sid)
    return True, "quarantined"


def _do_release(model, table, sid, c):
    table.release(sid)
    return True, "released"


def _do_evict(model, table, sid, c):
    table.retire(sid, reason="evicted")
    return True, "evicted"


def _do_distill(model, table, sid, c):
    """Retire the slot but keep its gist: a latent trace on the store and an
    EMA step of the bucket's prototype."""
    if c.tensor is not None:
        outer = model.outer_model
        traces = getattr(outer, "_latent_traces", None)
        if traces is not None:
            traces.append({"bucket_id": int(c.bucket_id), "centroid_contrib": c.tensor.detach().clone()})
            cap = int(outer.max_slots or 0)
            if cap > 0:
                del traces[: max(0, len(traces) - cap)]
        protos = getattr(model, "bucket_prototypes_module", None)
        buf = getattr(protos, "prototypes", None)
        if protos is not None and buf is not None and 0 <= int(c.bucket_id) < int(getattr(protos, "k_max", 0)):
            protos.update(int(c.bucket_id),
                          c.tensor.detach().reshape(-1, c.tensor.shape[-1]).to(device=buf.device, dtype=buf.dtype))
    table.retire(sid, reason="distilled")
    return True, "distilled"


_HANDLERS: dict[SlotCommitAction, Callable] = {
    SLOT_COMMIT_REFRESH: _do_refresh, SLOT_COMMIT_DECAY: _do_decay, SLOT_COMMIT_QUARANTINE: _do_quarantine,
    SLOT_COMMIT_RELEASE: _do_release, SLOT_COMMIT_EVICT: _do_evict, SLOT_COMMIT_DISTILL: _do_distill,
}


def apply_slot_commit_to_model(model: Any, commit: SlotCommit) -> tuple[bool, str]:
    """Applies a maintenance commit to a packet-serving mirror: ``(accepted, reason)``."""
    if commit.action is SLOT_COMMIT_APPEND:
        raise ValueError("APPEND commits must use apply_append_slot_commit_to_model")
    if commit.base_generation is None:
        raise ValueError(f"{commit.action.name} commit requires base_generation")
    table = model.outer_model.table
    sid, why = _resolve(table, commit)
    if sid is None:
        return False, why
    rec = table.record(sid)
    if rec is None:
        return False, "missing_record"
    if int(rec.write_generation) != commit.base_generation:
        return False, "stale_generation"
    if commit.action is SLOT_COMMIT_PRESERVE:
        return True, "preserved"
    handler = _HANDLERS.get(commit.action)
    if handler is None:
        return False, "unknown_action"
    ok, what = handler(model, table, sid, commit)
    if ok:
        _stamp(table, sid, commit.new_generation)
    return ok, what


def apply_append_slot_commit_to_model(model: Any, commit: SlotCommit) -> tuple[bool, str]:
    """Applies a packet-rank append to a maintenance-rank replica (idempotent)."""
    if commit.action is not SLOT_COMMIT_APPEND:
        raise ValueError("apply_append_slot_commit_to_model only accepts APPEND commits")
    if commit.tensor is None:
        return False, "missing_tensor"
    outer = model.outer_model
    table = outer.table
    have = table.record(commit.slot_id)
    if have is not None:
        same = int(have.write_generation) == commit.new_generation
        return (True, "already_present") if same else (False, "slot_id_collision")
    cap = int(outer.max_slots or 0)
    if cap > 0 and len(table) >= cap:
        return False, "replica_capacity_full"
    table.append_with_id(commit.slot_id, commit.tensor, bucket_id=commit.bucket_id, event_id=commit.event_id,
                         step=commit.step, survival=1.0, generation=commit.new_generation)
    return True, "appended"


def slot_commit_dtype_code(dtype: torch.dtype) -> int:
    if dtype not in SLOT_COMMIT_DTYPE_TO_CODE:
        raise ValueError(f"unsupported SlotCommit tensor dtype: {dtype}")
    return int(SLOT_COMMIT_DTYPE_TO_CODE[dtype])


def slot_commit_dtype_from_code(code: int) -> torch.dtype:
    try:
        return SLOT_COMMIT_CODE_TO_DTYPE[SlotCommitDType(int(code))]
    except (ValueError, KeyError) as exc:
        raise ValueError(f"unsupported SlotCommit tensor dtype code: {code}") from exc
