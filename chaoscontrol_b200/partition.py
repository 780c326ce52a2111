"""Polyphasic sleep: semantic partitions, their layouts over routing buckets,
and the K-of-N rotation scheduler (cf. src/chaoscontrol/partition.py:9-181)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

__all__ = ["SemanticPartition", "PartitionTopology", "PolyphasicScheduler"]


@dataclass
class SemanticPartition:
    partition_id: int
    bucket_ids: set[int] = field(default_factory=set)
    mode: Literal["awake", "sleeping"] = "awake"

    @property
    def is_awake(self) -> bool:
        return self.mode == "awake"

    @property
    def is_sleeping(self) -> bool:
        return self.mode == "sleeping"

    def owns_bucket(self, bucket_id: int) -> bool:
        return bucket_id in self.bucket_ids


class PartitionTopology:
    def __init__(self, partitions: list[SemanticPartition]) -> None:
        self.partitions = partitions

    @classmethod
    def _from_sets(cls, sets) -> "PartitionTopology":
        return cls([SemanticPartition(partition_id=i, bucket_ids=set(s)) for i, s in enumerate(sets)])

    @classmethod
    def slot_striped(cls, n_partitions: int, k_max: int = 16) -> "PartitionTopology":
        """Round-robin buckets: uniform coverage, no semantic grouping (the control layout)."""
        return cls._from_sets(range(i, k_max, n_partitions) for i in range(n_partitions))

    @classmethod
    def bucket_owned(cls, n_partitions: int, k_max: int) -> "PartitionTopology":
        """Each partition owns ``k_max // n_partitions`` contiguous buckets."""
        per = k_max // n_partitions
        return cls._from_sets(range(i * per, (i + 1) * per) for i in range(n_partitions))

    @classmethod
    def bucket_striped(cls, n_partitions: int, k_max: int, group_size: int = 2) -> "PartitionTopology":
        """Partitions in the same group of ``group_size`` share one contiguous bucket family."""
        per = k_max // (n_partitions // group_size)
        return cls._from_sets(range((i // group_size) * per, (i // group_size + 1) * per)
                              for i in range(n_partitions))

    def slot_owner_map(self, total_slots: int) -> list[int]:
        n = len(self.partitions)
        return [i % n for i in range(total_slots)]

    def awake_partitions(self) -> list[SemanticPartition]:
        return [p for p in self.partitions if p.is_awake]

    def sleeping_partitions(self) -> list[SemanticPartition]:
        return [p for p in self.partitions if p.is_sleeping]

    def awake_bucket_ids(self) -> set[int]:
        out: set[int] = set()
        for p in self.awake_partitions():
            out |= p.bucket_ids
        return out


class PolyphasicScheduler:
    """``N - k_awake`` consecutive partitions of the ring sleep; every
    ``swap_interval`` steps the sleeping window advances by one."""

    def __init__(self, topology: PartitionTopology, k_awake: int, swap_interval: int = 256) -> None:
        n = len(topology.partitions)
        if not 0 < k_awake < n:
            raise ValueError(f"k_awake must be in (0, {n}), got {k_awake}")
        self.topology, self.k_awake, self.swap_interval = topology, k_awake, swap_interval
        self._step_count = 0
        self._sleep_cursor = 0
        self._apply()

    def _apply(self) -> None:
        n = len(self.topology.partitions)
        asleep = {(self._sleep_cursor + j) % n for j in range(n - self.k_awake)}
        for i, p in enumerate(self.topology.partitions):
            p.mode = "sleeping" if i in asleep else "awake"

    def awake(self) -> list[SemanticPartition]:
        return self.topology.awake_partitions()

    def sleeping(self) -> list[SemanticPartition]:
        return self.topology.sleeping_partitions()

    def step(self) -> bool:
        """Advances one step; True when the window moved."""
        self._step_count += 1
        if self._step_count % self.swap_interval:
            return False
        self._rotate()
        return True

    def _rotate(self) -> None:
        self._sleep_cursor = (self._sleep_cursor + 1) % len(self.topology.partitions)
        self._apply()
