"""Fixed-capacity, fingerprint-addressed episodic cache with utility-driven
eviction, and the token fingerprint it is keyed by.

Public surface of the reference's ``EpisodicCache`` / ``CacheEntry``
(src/chaoscontrol/optim/episodic_cache.py:45-595) and ``fingerprint_tokens``
(src/chaoscontrol/optim/episodic_writer.py:156-187).  Per-slot state is a
struct of flat tensors described by ONE field table, which drives
construction, reset, eviction, snapshot and (de)serialisation, so a new field
is one table row.  Eviction: an empty slot if there is one; else the lowest
``utility + protection`` among entries older than ``grace_steps``; else (cache
saturated during warm-up) the oldest write.

The fingerprint is the polynomial hash ``h <- (h * 1_000_003 + tok + 1) mod
(2^61 - 1)``.  The batch form evaluates it for all rows at once in uint64
arithmetic (the 81-bit products are folded with ``2^61 == 1 (mod p)``) and is
bit-identical to the scalar form and to the device kernel that packs write
events.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any

import numpy as np
import torch

__all__ = ["CacheEntry", "EpisodicCache", "fingerprint_tokens", "fingerprint_tokens_batch",
           "FINGERPRINT_MODULUS", "FINGERPRINT_BASE"]

FINGERPRINT_MODULUS = (1 << 61) - 1
FINGERPRINT_BASE = 1_000_003


def fingerprint_tokens(tokens: torch.Tensor) -> int:
    """Stable rolling hash of a 1-D token sequence, in ``[0, 2^61 - 1)``."""
    if tokens.dim() != 1:
        raise ValueError(f"fingerprint_tokens expects a 1-D tensor; got shape {tuple(tokens.shape)}")
    h = 0
    for tok in tokens.detach().to(dtype=torch.int64).cpu().tolist():
        h = (h * FINGERPRINT_BASE + int(tok) + 1) % FINGERPRINT_MODULUS
    return int(h)


def _mulbase_mod(h: np.ndarray) -> np.ndarray:
    """``h * BASE mod (2^61 - 1)`` for uint64 ``h < 2^61`` without overflow."""
    P = np.uint64(FINGERPRINT_MODULUS)
    B = np.uint64(FINGERPRINT_BASE)
    lo = (h & np.uint64(0xFFFFFFFF)) * B                      # < 2^52
    x = (h >> np.uint64(32)) * B                              # < 2^49;  needs * 2^32
    hi = (x >> np.uint64(29)) + ((x & np.uint64((1 << 29) - 1)) << np.uint64(32))   # 2^61 == 1
    s = lo + hi                                               # < 2^62
    s = (s & P) + (s >> np.uint64(61))
    return np.where(s >= P, s - P, s)


def fingerprint_tokens_batch(tokens: torch.Tensor) -> list[int]:
    """Fingerprints of every row of ``[N, W]`` token ids."""
    if tokens.dim() != 2:
        raise ValueError(f"fingerprint_tokens_batch expects 2-D [N, W]; got shape {tuple(tokens.shape)}")
    arr = tokens.detach().to(dtype=torch.int64).cpu().numpy().astype(np.uint64)
    P = np.uint64(FINGERPRINT_MODULUS)
    h = np.zeros(arr.shape[0], dtype=np.uint64)
    for j in range(arr.shape[1]):
        s = _mulbase_mod(h) + (arr[:, j] + np.uint64(1)) % P
        h = np.where(s >= P, s - P, s)
    return [int(v) for v in h.tolist()]


@dataclass(frozen=True)
class CacheEntry:
    slot: int
    key_fp: int
    key_rep: torch.Tensor
    value_tok_ids: torch.Tensor
    value_anchor_id: int
    utility_u: float
    last_fired_step: int
    write_step: int
    birth_embedding_version: int
    pressure_at_write: float = 0.0
    source_write_id: int = -1
    write_bucket: int = -1
    protection_score: float = 0.0


# name -> (trailing-shape attribute or None, dtype, value of an empty slot)
_FIELDS: dict[str, tuple[str | None, torch.dtype, Any]] = {
    "key_fp": (None, torch.int64, 0),
    "key_rep": ("key_rep_dim", torch.float32, 0),
    "value_tok_ids": ("span_length", torch.int64, 0),
    "value_anchor_id": (None, torch.int64, 0),
    "utility_u": (None, torch.float32, 0),
    "last_fired_step": (None, torch.int64, -1),
    "write_step": (None, torch.int64, -1),
    "birth_embedding_version": (None, torch.int64, 0),
    "occupied": (None, torch.bool, False),
    "pressure_at_write": (None, torch.float32, 0),
    "source_write_id": (None, torch.int64, -1),
    "write_bucket": (None, torch.int64, -1),
    "protection_score": (None, torch.float32, 0),
    "slot_state": ("slot_state_dim", torch.float16, 0),
    "simplex_edge_slot": ("simplex_k_max", torch.int64, -1),
    "simplex_edge_weight": ("simplex_k_max", torch.float16, 0),
}
# what evict() restores to the empty value (identity fields keep their last contents)
_EVICT_RESET = ("occupied", "last_fired_step", "write_step", "utility_u", "pressure_at_write", "source_write_id",
                "write_bucket", "protection_score", "slot_state", "simplex_edge_slot", "simplex_edge_weight")


class EpisodicCache:
    """Single-writer store; ``snapshot_to(device)`` hands readers a consistent copy.

    With ``eviction_trace_path`` every displacement appends one NDJSON row (the
    displaced slot's state before the overwrite and the displacing write's id)
    for offline behaviour-cloning of the eviction policy.
    """

    _CONFIG_FIELDS: tuple[str, ...] = ("capacity", "span_length", "key_rep_dim", "grace_steps", "utility_ema_decay",
                                       "fingerprint_window", "slot_state_dim", "simplex_k_max")
    _TENSOR_FIELDS: tuple[str, ...] = tuple(_FIELDS)

    def __init__(self, *, capacity: int, span_length: int = 8, key_rep_dim: int = 16, grace_steps: int = 200,
                 utility_ema_decay: float = 0.99, fingerprint_window: int = 8, slot_state_dim: int = 0,
                 simplex_k_max: int = 0, eviction_trace_path: str | None = None) -> None:
        for name, val in (("capacity", capacity), ("span_length", span_length), ("key_rep_dim", key_rep_dim),
                          ("fingerprint_window", fingerprint_window)):
            if val <= 0:
                raise ValueError(f"{name} must be positive; got {val}")
        if not 0.0 < utility_ema_decay < 1.0:
            raise ValueError(f"utility_ema_decay must be in (0, 1); got {utility_ema_decay}")
        for name, val in (("slot_state_dim", slot_state_dim), ("simplex_k_max", simplex_k_max)):
            if val < 0:
                raise ValueError(f"{name} must be non-negative; got {val}")
        self.capacity, self.span_length, self.key_rep_dim = int(capacity), int(span_length), int(key_rep_dim)
        self.grace_steps, self.utility_ema_decay = int(grace_steps), float(utility_ema_decay)
        self.fingerprint_window = int(fingerprint_window)
        self.slot_state_dim, self.simplex_k_max = int(slot_state_dim), int(simplex_k_max)
        self.eviction_trace_path = None if eviction_trace_path is None else str(eviction_trace_path)
        for name, (dim_attr, dtype, empty) in _FIELDS.items():
            shape = (self.capacity,) if dim_attr is None else (self.capacity, getattr(self, dim_attr))
            setattr(self, name, torch.full(shape, empty, dtype=dtype))
        self._fp_index: dict[int, int] = {}

    def __len__(self) -> int:
        return int(self.occupied.sum().item())

    @property
    def is_full(self) -> bool:
        return len(self) >= self.capacity

    def _check_slot(self, slot: int) -> None:
        if not 0 <= slot < self.capacity:
            raise IndexError(f"slot {slot} out of range for capacity {self.capacity}")

    def _allocate_slot(self, *, current_step: int) -> int:
        free = (~self.occupied).nonzero(as_tuple=True)[0]
        if free.numel():
            return int(free[0])
        past_grace = (current_step - self.write_step) >= self.grace_steps
        if past_grace.any():
            score = torch.where(past_grace, self.utility_u + self.protection_score,
                                torch.full_like(self.utility_u, float("inf")))
            return int(score.argmin())
        return int(self.write_step.argmin())

    def append(self, *, key_fp: int, key_rep: torch.Tensor, value_tok_ids: torch.Tensor, value_anchor_id: int,
               current_step: int, embedding_version: int, pressure_at_write: float = 0.0, source_write_id: int = -1,
               write_bucket: int = -1, displacing_candidate_id: int = -1, protection_score: float = 0.0) -> int:
        """Inserts one entry (utility starts at 1) and returns its slot."""
        if key_rep.shape != (self.key_rep_dim,):
            raise ValueError(f"key_rep must have shape ({self.key_rep_dim},); got {tuple(key_rep.shape)}")
        if value_tok_ids.shape != (self.span_length,):
            raise ValueError(f"value_tok_ids must have shape ({self.span_length},); got {tuple(value_tok_ids.shape)}")
        slot = self._allocate_slot(current_step=current_step)
        if bool(self.occupied[slot]):
            old_fp = int(self.key_fp[slot])
            if self._fp_index.get(old_fp) == slot:
                del self._fp_index[old_fp]
            if self.eviction_trace_path is not None:
                self._emit_eviction_trace_row(evicted_slot=slot, evicted_key_fp=old_fp, gpu_step=int(current_step),
                                              displacing_candidate_id=int(displacing_candidate_id),
                                              displacing_key_fp=int(key_fp))
        self.key_fp[slot] = int(key_fp)
        self.key_rep[slot] = key_rep.to(dtype=torch.float32)
        self.value_tok_ids[slot] = value_tok_ids.to(dtype=torch.int64)
        self.value_anchor_id[slot] = int(value_anchor_id)
        self.utility_u[slot] = 1.0
        self.last_fired_step[slot] = -1
        self.write_step[slot] = int(current_step)
        self.birth_embedding_version[slot] = int(embedding_version)
        self.occupied[slot] = True
        self.pressure_at_write[slot] = float(pressure_at_write)
        self.source_write_id[slot] = int(source_write_id)
        self.write_bucket[slot] = int(write_bucket)
        self.protection_score[slot] = float(protection_score)
        for name in ("slot_state", "simplex_edge_slot", "simplex_edge_weight"):
            getattr(self, name)[slot] = _FIELDS[name][2]
        self._fp_index[int(key_fp)] = slot
        return slot

    def query(self, key_fp: int) -> CacheEntry | None:
        """Exact-fingerprint lookup; read-only (call ``mark_fired`` if the entry is used)."""
        slot = self._fp_index.get(int(key_fp))
        if slot is None:
            return None
        if not bool(self.occupied[slot]):
            self._fp_index.pop(int(key_fp), None)
            return None
        return CacheEntry(
            slot=int(slot), key_fp=int(self.key_fp[slot]), key_rep=self.key_rep[slot].clone(),
            value_tok_ids=self.value_tok_ids[slot].clone(), value_anchor_id=int(self.value_anchor_id[slot]),
            utility_u=float(self.utility_u[slot]), last_fired_step=int(self.last_fired_step[slot]),
            write_step=int(self.write_step[slot]), birth_embedding_version=int(self.birth_embedding_version[slot]),
            pressure_at_write=float(self.pressure_at_write[slot]), source_write_id=int(self.source_write_id[slot]),
            write_bucket=int(self.write_bucket[slot]), protection_score=float(self.protection_score[slot]))

    def mark_fired(self, slot: int, current_step: int) -> None:
        self._check_slot(slot)
        if not bool(self.occupied[slot]):
            raise ValueError(f"slot {slot} is not occupied")
        self.last_fired_step[slot] = int(current_step)

    def update_utility(self, slot: int, ce_delta: float) -> None:
        """EMA of the retrieval-time CE improvement; feedback for an evicted slot is dropped."""
        self._check_slot(slot)
        if bool(self.occupied[slot]):
            d = self.utility_ema_decay
            self.utility_u[slot] = d * float(self.utility_u[slot]) + (1.0 - d) * float(ce_delta)

    def evict(self, slot: int) -> None:
        self._check_slot(slot)
        if not bool(self.occupied[slot]):
            return
        fp = int(self.key_fp[slot])
        if self._fp_index.get(fp) == slot:
            del self._fp_index[fp]
        for name in _EVICT_RESET:
            getattr(self, name)[slot] = _FIELDS[name][2]

    def reset(self) -> None:
        """Back to the freshly constructed state (shape parameters kept)."""
        for name, (_d, _t, empty) in _FIELDS.items():
            getattr(self, name).fill_(empty)
        self._fp_index.clear()

    def snapshot_to(self, device: torch.device) -> dict[str, torch.Tensor]:
        return {name: getattr(self, name).to(device, non_blocking=True) for name in _FIELDS}

    def to_dict(self) -> dict[str, Any]:
        blob: dict[str, Any] = {name: getattr(self, name) for name in self._CONFIG_FIELDS}
        blob.update({name: getattr(self, name).clone() for name in self._TENSOR_FIELDS})
        blob["fp_index"] = dict(self._fp_index)
        return blob

    @classmethod
    def from_dict(cls, blob: dict[str, Any]) -> "EpisodicCache":
        """Strict inverse of ``to_dict``: a missing key is an error, never a default,
        so a saved and a loaded cache cannot silently differ in shape."""
        missing = [n for n in (*cls._CONFIG_FIELDS, *cls._TENSOR_FIELDS, "fp_index") if n not in blob]
        if missing:
            raise KeyError(f"EpisodicCache.from_dict missing required key(s): {sorted(missing)}. The payload must "
                           f"carry every field emitted by EpisodicCache.to_dict.")
        cache = cls(**{n: blob[n] for n in cls._CONFIG_FIELDS})
        for n in cls._TENSOR_FIELDS:
            getattr(cache, n).copy_(blob[n])
        cache._fp_index = {int(k): int(v) for k, v in blob["fp_index"].items()}
        return cache

    def _emit_eviction_trace_row(self, *, evicted_slot: int, evicted_key_fp: int, gpu_step: int,
                                 displacing_candidate_id: int, displacing_key_fp: int) -> None:
        # column order is part of the schema: consumers read by position
        row = {"evicted_slot_id": int(evicted_slot), "evicted_key_fp": int(evicted_key_fp),
               "evicted_utility_at_eviction": float(self.utility_u[evicted_slot]),
               "evicted_write_step": int(self.write_step[evicted_slot]),
               "evicted_last_fired_step": int(self.last_fired_step[evicted_slot]),
               "evicted_protection_score": float(self.protection_score[evicted_slot]),
               "gpu_step": int(gpu_step), "displacing_candidate_id": int(displacing_candidate_id),
               "displacing_key_fp": int(displacing_key_fp)}
        with open(self.eviction_trace_path, "a", encoding="utf-8") as fh:
            fh.write(json.dumps(row, separators=(",", ":")) + "\n")
