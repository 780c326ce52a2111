"""Slot table: identity and lifecycle bookkeeping for episodic memory slots.

Same public surface as the reference table (src/chaoscontrol/slot_table.py:56-364:
``append`` / ``append_with_id`` / ``retire`` / ``retire_many`` / ``quarantine`` /
``release`` / ``replace_tensor`` / ``scale_survival`` / ``visible_indices`` /
``slot_matrix`` / ``state_dict``), different storage: slot vectors live in ONE
dense, geometrically grown ``[capacity, dim]`` tensor on the owner's device,
rows in insertion order.  A read over all visible slots is then a view of that
matrix (no per-read concatenation of hundreds of tiny tensors), a retirement is
one ``index_select`` compaction, and a batched append is one ``copy_``.

Slot ids are stable for the life of a slot; physical rows shift on retirement.
Metadata that the host control plane edits (survival, bucket, event id,
priority) stays in Python lists beside the dense matrix.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Iterable, Sequence

import torch

__all__ = ["SlotTable", "SlotRecord", "SlotId"]

SlotId = int

SLOT_WARMING = "WARMING"
SLOT_ACTIVE = "ACTIVE"
SLOT_DECAYING = "DECAYING"
SLOT_QUARANTINED = "QUARANTINED"
SLOT_DISTILLING = "DISTILLING"
SLOT_RETIRED = "RETIRED"


@dataclass
class SlotRecord:
    """Per-slot lifecycle telemetry (field set of reference slot_table.py:27-53)."""

    slot_id: SlotId
    state: str = SLOT_WARMING
    created_step: int = 0
    last_scored_step: int = 0
    last_used_step: int = 0
    write_generation: int = 0
    bucket_id: int = -1
    event_id: int = 0
    utility_ema: float = 0.0
    marginal_gain_ema: float = 0.0
    sharpness_ema: float = 0.0
    activation_drift_ema: float = 0.0
    representation_drift_ema: float = 0.0
    semantic_drift_ema: float = 0.0
    contradiction_ema: float = 0.0
    retrieval_mass_ema: float = 0.0
    peak_utility: float = 0.0
    peak_sharpness: float = 0.0
    score_count: int = 0
    negative_streak: int = 0
    positive_streak: int = 0
    refresh_count: int = 0
    quarantine_count: int = 0
    last_action: str = "PRESERVE"
    retire_reason: str = ""


class _SlotRows(Sequence):
    """List-like view of the dense matrix as ``[1, dim]`` rows.

    Exists so code written against a list of slot tensors (``table._slots[i]``,
    ``len``, iteration, truthiness) keeps working on the dense store.
    """

    def __init__(self, table: "SlotTable") -> None:
        self._t = table

    def __len__(self) -> int:
        return self._t._n

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(self._t._n))]
        n = self._t._n
        if i < 0:
            i += n
        if not 0 <= i < n:
            raise IndexError(i)
        return self._t._store[i:i + 1]

    def __setitem__(self, i: int, value: torch.Tensor) -> None:
        n = self._t._n
        if i < 0:
            i += n
        if not 0 <= i < n:
            raise IndexError(i)
        self._t._store[i].copy_(value.detach().reshape(-1))

    def __eq__(self, other) -> bool:
        return list(self) == other


class SlotTable:
    """Dense slot storage with persistent ids and lifecycle tracking."""

    def __init__(self) -> None:
        self._next_id: int = 0
        self._records: dict[SlotId, SlotRecord] = {}
        self._id_to_physical: dict[SlotId, int] = {}
        self._physical_to_id: dict[int, SlotId] = {}
        self._store: torch.Tensor | None = None     # [capacity, dim]
        self._n: int = 0
        self._survival: list[float] = []
        self._slot_buckets: list[int] = []
        self._slot_event_ids: list[int] = []
        self._priority: list[float] = []

    # ------------------------------------------------------------------ storage
    @property
    def _slots(self) -> _SlotRows:
        return _SlotRows(self)

    @_slots.setter
    def _slots(self, value: Iterable[torch.Tensor]) -> None:
        rows = [v.detach().reshape(1, -1) for v in value]
        self._n = 0
        self._store = None
        if rows:
            mat = torch.cat(rows, dim=0)
            self._reserve(mat.shape[0], mat)
            self._store[: mat.shape[0]].copy_(mat)
            self._n = mat.shape[0]

    def _reserve(self, n_total: int, like: torch.Tensor) -> None:
        if self._store is not None and self._store.shape[0] >= n_total:
            return
        cap = 64 if self._store is None else self._store.shape[0]
        while cap < n_total:
            cap *= 2
        # the store outlives any inference-mode scope a writer runs in: allocate it as a normal tensor so
        # later in-place slot edits are legal from every context
        with torch.inference_mode(False):
            new = torch.zeros(cap, like.shape[-1], dtype=like.dtype, device=like.device)
            if self._store is not None and self._n:
                new[: self._n].copy_(self._store[: self._n])
        self._store = new

    def __len__(self) -> int:
        return self._n

    @property
    def n_active(self) -> int:
        return self._n

    def _allocate_id(self) -> SlotId:
        sid = self._next_id
        self._next_id += 1
        return sid

    # ------------------------------------------------------------------ inserts
    def _install(self, sid: SlotId, row: torch.Tensor, *, bucket_id: int, event_id: int, step: int,
                 survival: float, generation: int) -> SlotId:
        sid = int(sid)
        if sid in self._id_to_physical:
            raise ValueError(f"slot_id {sid} already exists")
        row = row.detach().reshape(1, -1)
        self._reserve(self._n + 1, row)
        phys = self._n
        self._store[phys].copy_(row[0])
        self._n += 1
        self._survival.append(float(survival))
        self._slot_buckets.append(int(bucket_id))
        self._slot_event_ids.append(int(event_id))
        self._priority.append(1.0)
        self._id_to_physical[sid] = phys
        self._physical_to_id[phys] = sid
        self._next_id = max(int(self._next_id), sid + 1)
        self._records[sid] = SlotRecord(slot_id=sid, created_step=int(step), write_generation=int(generation),
                                        bucket_id=int(bucket_id), event_id=int(event_id))
        return sid

    def append(self, tensor: torch.Tensor, *, bucket_id: int = -1, event_id: int = 0, step: int = 0,
               survival: float = 0.0) -> SlotId:
        return self._install(self._allocate_id(), tensor, bucket_id=bucket_id, event_id=event_id, step=step,
                             survival=survival, generation=0)

    def append_with_id(self, slot_id: SlotId, tensor: torch.Tensor, *, bucket_id: int = -1, event_id: int = 0,
                       step: int = 0, survival: float = 0.0, generation: int = 0) -> SlotId:
        """Appends a replicated slot whose identity was assigned elsewhere."""
        return self._install(slot_id, tensor, bucket_id=bucket_id, event_id=event_id, step=step,
                             survival=survival, generation=generation)

    def append_rows(self, rows: torch.Tensor, bucket_ids: Sequence[int], event_ids: Sequence[int], *,
                    survival: float = 0.0, step: int = 0) -> list[SlotId]:
        """Batched append: one device copy for ``rows`` ``[N, dim]``."""
        n = int(rows.shape[0])
        if n == 0:
            return []
        rows = rows.detach()
        self._reserve(self._n + n, rows)
        self._store[self._n:self._n + n].copy_(rows)
        out = []
        for i in range(n):
            sid = self._allocate_id()
            phys = self._n + i
            self._survival.append(float(survival))
            self._slot_buckets.append(int(bucket_ids[i]))
            self._slot_event_ids.append(int(event_ids[i]))
            self._priority.append(1.0)
            self._id_to_physical[sid] = phys
            self._physical_to_id[phys] = sid
            self._records[sid] = SlotRecord(slot_id=sid, created_step=int(step), bucket_id=int(bucket_ids[i]),
                                            event_id=int(event_ids[i]))
            out.append(sid)
        self._n += n
        return out

    # ------------------------------------------------------------------ removal
    def retire(self, slot_id: SlotId, *, reason: str = "evicted") -> bool:
        return bool(self.retire_many([slot_id], reason=reason))

    def retire_many(self, slot_ids: list[SlotId], *, reason: str = "evicted") -> list[SlotId]:
        valid = [sid for sid in dict.fromkeys(slot_ids) if sid in self._id_to_physical]
        if not valid:
            return []
        drop = {self._id_to_physical[sid] for sid in valid}
        keep = [i for i in range(self._n) if i not in drop]
        if keep:
            idx = torch.tensor(keep, dtype=torch.long, device=self._store.device)
            self._store[: len(keep)] = self._store.index_select(0, idx)
        self._n = len(keep)
        for name in ("_survival", "_slot_buckets", "_slot_event_ids", "_priority"):
            old = getattr(self, name)
            setattr(self, name, [old[i] for i in keep])
        for sid in valid:
            del self._id_to_physical[sid]
            rec = self._records.get(sid)
            if rec is not None:
                rec.write_generation += 1
                rec.state = SLOT_RETIRED
                rec.retire_reason = reason
        self._rebuild_physical_maps()
        return valid

    def _rebuild_physical_maps(self) -> None:
        order = sorted(self._id_to_physical, key=self._id_to_physical.get)
        self._id_to_physical = {sid: phys for phys, sid in enumerate(order)}
        self._physical_to_id = {phys: sid for phys, sid in enumerate(order)}

    # ------------------------------------------------------------------ lifecycle
    def _bump(self, slot_id: SlotId) -> SlotRecord | None:
        rec = self._records.get(slot_id)
        if rec is not None:
            rec.write_generation += 1
        return rec

    def quarantine(self, slot_id: SlotId) -> bool:
        phys = self._id_to_physical.get(slot_id)
        if phys is None:
            return False
        self._priority[phys] = 0.0
        rec = self._bump(slot_id)
        if rec is not None:
            rec.state = SLOT_QUARANTINED
            rec.quarantine_count += 1
        return True

    def release(self, slot_id: SlotId) -> bool:
        phys = self._id_to_physical.get(slot_id)
        if phys is None:
            return False
        self._priority[phys] = 1.0
        rec = self._bump(slot_id)
        if rec is not None:
            rec.state = SLOT_ACTIVE
        return True

    def replace_tensor(self, slot_id: SlotId, tensor: torch.Tensor, *, bump_generation: bool = True) -> bool:
        phys = self._id_to_physical.get(slot_id)
        if phys is None:
            return False
        self._store[phys].copy_(tensor.detach().reshape(-1))
        if bump_generation:
            self._bump(slot_id)
        return True

    def scale_survival(self, slot_id: SlotId, factor: float) -> bool:
        phys = self._id_to_physical.get(slot_id)
        if phys is None:
            return False
        self._survival[phys] *= float(factor)
        self._bump(slot_id)
        return True

    # ------------------------------------------------------------------ queries
    def get_tensor(self, slot_id: SlotId) -> torch.Tensor | None:
        phys = self._id_to_physical.get(slot_id)
        return None if phys is None else self._store[phys:phys + 1]

    def record(self, slot_id: SlotId) -> SlotRecord | None:
        return self._records.get(slot_id)

    def active_records(self) -> list[SlotRecord]:
        return [self._records[sid] for sid in self._id_to_physical if sid in self._records]

    def active_slot_ids(self) -> list[SlotId]:
        return list(self._id_to_physical.keys())

    def physical_to_slot_id(self, phys: int) -> SlotId | None:
        return self._physical_to_id.get(phys)

    def slot_id_to_physical(self, slot_id: SlotId) -> int | None:
        return self._id_to_physical.get(slot_id)

    def visible_indices(self, *, read_cutoff: int | None = None, bucket_id: int | None = None) -> list[int]:
        """Physical rows a reader may see: optional bucket filter, and event ids
        no newer than ``read_cutoff`` (multi-version visibility)."""
        cutoff = None if read_cutoff is None else int(read_cutoff)
        if cutoff is None and bucket_id is None:
            return list(range(self._n))
        return [i for i in range(self._n)
                if (bucket_id is None or self._slot_buckets[i] == bucket_id)
                and (cutoff is None or self._slot_event_ids[i] <= cutoff)]

    def slot_matrix(self, indices: list[int] | None = None) -> torch.Tensor:
        if self._n == 0 or (indices is not None and not indices):
            return torch.zeros(0, 0)
        if indices is None or (len(indices) == self._n and indices[0] == 0 and indices[-1] == self._n - 1):
            return self._store[: self._n]
        if indices[-1] - indices[0] + 1 == len(indices):      # contiguous run: still a view
            return self._store[indices[0]:indices[-1] + 1]
        idx = torch.tensor(indices, dtype=torch.long, device=self._store.device)
        return self._store.index_select(0, idx)

    def priority_vector(self, indices: list[int] | None = None) -> torch.Tensor:
        if indices is None:
            indices = list(range(self._n))
        if not indices:
            return torch.zeros(0)
        return torch.tensor([self._priority[i] for i in indices], dtype=torch.float32)

    # ------------------------------------------------------------------ persistence
    def state_dict(self) -> dict:
        recs = {sid: {f.name: getattr(rec, f.name) for f in fields(rec)}
                for sid, rec in self._records.items() if rec.state != SLOT_RETIRED}
        return {
            "next_id": self._next_id,
            "slots": [self._store[i:i + 1].cpu().clone() for i in range(self._n)],
            "survival": list(self._survival),
            "slot_buckets": list(self._slot_buckets),
            "slot_event_ids": list(self._slot_event_ids),
            "priority": list(self._priority),
            "id_to_physical": dict(self._id_to_physical),
            "records": recs,
        }

    def load_state_dict(self, d: dict, *, device: torch.device | None = None) -> None:
        self._next_id = d["next_id"]
        self._slots = [s.to(device) if device is not None else s for s in d["slots"]]
        self._survival = list(d["survival"])
        self._slot_buckets = list(d["slot_buckets"])
        self._slot_event_ids = list(d["slot_event_ids"])
        self._priority = list(d.get("priority", [1.0] * self._n))
        self._id_to_physical = {int(k): int(v) for k, v in d["id_to_physical"].items()}
        self._rebuild_physical_maps()
        self._records = {int(sid): SlotRecord(**rec) for sid, rec in d.get("records", {}).items()}

    def purge_retired(self) -> int:
        gone = [sid for sid, rec in self._records.items() if rec.state == SLOT_RETIRED]
        for sid in gone:
            del self._records[sid]
        return len(gone)
