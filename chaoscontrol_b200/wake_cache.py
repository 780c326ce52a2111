"""Wake-phase caches that feed the sleep cycle.

``WakeCache`` keeps the ``max_moments`` most surprising training moments (all
tensors detached and parked on the host) plus a rolling buffer of hidden states
and a running histogram of routing buckets
(cf. src/chaoscontrol/wake_cache.py:14-163).  ``TransactionalWakeCache`` adds a
multi-version layer: a batch opens a transaction with a read cutoff, stages its
writes, and publishes them on commit under strictly newer event ids, so a
counterfactual comparison never sees its own batch
(cf. src/chaoscontrol/wake_cache_txn.py:21-201).

Eviction is "replace the least surprising entry if the newcomer beats it"; the
index of that entry comes from one ``min`` over a parallel list of magnitudes.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

__all__ = ["WakeCache", "CausalEventClock", "CacheTxn", "TransactionalWakeCache"]


def _make_moment(surprise, inputs, targets, hidden, bucket_ids, slot_cues) -> dict[str, Any]:
    m: dict[str, Any] = {"surprise": float(surprise), "inputs": inputs.detach().cpu(),
                         "targets": targets.detach().cpu(), "hidden": hidden.detach().cpu()}
    if bucket_ids is not None:
        m["bucket_ids"] = bucket_ids.detach().cpu()
    if slot_cues is not None:
        m["slot_cues"] = slot_cues.detach().cpu()
    return m


class WakeCache:
    def __init__(self, max_moments: int = 32, max_hidden_buffer: int = 64) -> None:
        self.max_moments = max_moments
        self.max_hidden_buffer = max_hidden_buffer
        self.moments: list[dict[str, Any]] = []
        self.hidden_buffer: deque = deque(maxlen=max_hidden_buffer)
        self._bucket_counts: Optional[torch.Tensor] = None

    def _admit(self, moment: dict[str, Any]) -> None:
        if len(self.moments) < self.max_moments:
            self.moments.append(moment)
            return
        mags = [abs(float(m["surprise"])) for m in self.moments]
        weakest = min(range(len(mags)), key=mags.__getitem__)
        if abs(float(moment["surprise"])) > mags[weakest]:
            self.moments[weakest] = moment

    def record_moment(self, *, surprise: float, inputs: torch.Tensor, targets: torch.Tensor, hidden: torch.Tensor,
                      bucket_ids: Optional[torch.Tensor] = None, slot_cues: Optional[torch.Tensor] = None) -> None:
        self._admit(_make_moment(surprise, inputs, targets, hidden, bucket_ids, slot_cues))

    def push_hidden(self, hidden: torch.Tensor) -> None:
        self.hidden_buffer.append(hidden.detach().cpu())

    def update_bucket_counts(self, bucket_ids: torch.Tensor) -> None:
        counts = torch.bincount(bucket_ids.detach().cpu().long().reshape(-1))
        if self._bucket_counts is None:
            self._bucket_counts = counts
            return
        n = max(counts.numel(), self._bucket_counts.numel())
        total = torch.zeros(n, dtype=counts.dtype)
        total[: self._bucket_counts.numel()] += self._bucket_counts
        total[: counts.numel()] += counts
        self._bucket_counts = total

    def bucket_distribution(self, n_buckets: int) -> torch.Tensor:
        """Observed bucket frequencies over ``n_buckets`` (uniform before any data)."""
        uniform = torch.ones(n_buckets) / n_buckets
        if self._bucket_counts is None:
            return uniform
        c = torch.zeros(n_buckets, dtype=self._bucket_counts.dtype)
        k = min(n_buckets, self._bucket_counts.numel())
        c[:k] = self._bucket_counts[:k]
        return c.float() / c.sum().float() if c.sum() > 0 else uniform

    def filter_moments_by_partition(self, partition: Any) -> list[dict]:
        """Moments whose dominant bucket belongs to ``partition``."""
        out = []
        for m in self.moments:
            b = m.get("bucket_ids")
            if b is not None and partition.owns_bucket(int(b.reshape(-1).mode().values.item())):
                out.append(m)
        return out

    def clear(self) -> None:
        self.moments.clear()
        self.hidden_buffer.clear()
        self._bucket_counts = None


@dataclass
class CausalEventClock:
    """Monotone event-id source shared by cache commits and slot writers."""
    current: int = 0

    def next(self) -> int:
        self.current += 1
        return self.current


@dataclass
class CacheTxn:
    read_cutoff: int
    staged_moments: list[dict[str, Any]] = field(default_factory=list)
    staged_hidden: list[torch.Tensor] = field(default_factory=list)
    committed: bool = False
    rolled_back: bool = False

    def _check_open(self, what: str) -> None:
        if self.committed:
            raise RuntimeError("CacheTxn has already been committed" if what == "close"
                               else "cannot stage writes on a closed CacheTxn")
        if self.rolled_back:
            raise RuntimeError("CacheTxn has already been rolled back" if what == "close"
                               else "cannot stage writes on a closed CacheTxn")


class TransactionalWakeCache:
    """Entries of a wrapped, already-populated cache carry no event id and count
    as event 0: visible to every transaction."""

    def __init__(self, base: WakeCache | None = None, *, max_moments: int = 32, max_hidden_buffer: int = 64,
                 clock: CausalEventClock | None = None) -> None:
        self.base = base or WakeCache(max_moments=max_moments, max_hidden_buffer=max_hidden_buffer)
        self.clock = clock or CausalEventClock()

    @property
    def moments(self) -> list[dict[str, Any]]:
        return self.base.moments

    @property
    def hidden_buffer(self):
        return self.base.hidden_buffer

    def begin_batch(self) -> CacheTxn:
        return CacheTxn(read_cutoff=int(self.clock.current))

    def _publish_moment(self, moment: dict[str, Any]) -> None:
        stamped = dict(moment)
        stamped["_event_id"] = self.clock.next()
        self.base._admit(stamped)

    def _publish_hidden(self, hidden: torch.Tensor) -> None:
        h = hidden.detach().cpu()
        setattr(h, "_event_id", self.clock.next())
        self.base.hidden_buffer.append(h)

    def commit(self, txn: CacheTxn) -> None:
        txn._check_open("close")
        for m in txn.staged_moments:
            self._publish_moment(m)
        for h in txn.staged_hidden:
            self._publish_hidden(h)
        txn.committed = True

    def rollback(self, txn: CacheTxn) -> None:
        txn._check_open("close")
        txn.staged_moments.clear()
        txn.staged_hidden.clear()
        txn.rolled_back = True

    def reserve_event_ids(self, n: int, *, device=None) -> torch.Tensor:
        """Event ids for an external slot writer, taken from the same clock so the
        model-side slot visibility and the cache-side cutoff share one timeline."""
        if int(n) < 0:
            raise ValueError(f"cannot reserve a negative number of event ids: {n}")
        return torch.tensor([self.clock.next() for _ in range(int(n))], dtype=torch.long, device=device)

    def record_moment(self, *, surprise: float, inputs, targets, hidden, bucket_ids=None, slot_cues=None,
                      txn: CacheTxn | None = None) -> None:
        m = _make_moment(surprise, inputs, targets, hidden, bucket_ids, slot_cues)
        if txn is None:
            self._publish_moment(m)
        else:
            txn._check_open("stage")
            txn.staged_moments.append(m)

    def push_hidden(self, hidden: torch.Tensor, *, txn: CacheTxn | None = None) -> None:
        if txn is None:
            self._publish_hidden(hidden)
        else:
            txn._check_open("stage")
            txn.staged_hidden.append(hidden.detach().cpu())

    def visible_moments(self, read_cutoff: int | None) -> list[dict[str, Any]]:
        if read_cutoff is None:
            return list(self.base.moments)
        return [m for m in self.base.moments if int(m.get("_event_id", 0)) <= int(read_cutoff)]

    def visible_hidden(self, read_cutoff: int | None) -> list[torch.Tensor]:
        if read_cutoff is None:
            return list(self.base.hidden_buffer)
        return [h for h in self.base.hidden_buffer if int(getattr(h, "_event_id", 0)) <= int(read_cutoff)]

    def clear(self) -> None:
        self.base.clear()
        self.clock.current = 0
