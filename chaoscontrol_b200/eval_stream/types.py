"""Records and the three-axis run configuration of the streaming evaluator
(adapt set x persistence mode x delta modulation); field set follows
src/chaoscontrol/eval_stream/types.py:31-108 so JSON configs are interchangeable."""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Optional


@dataclass
class DocRecord:
    doc_id: int
    tokens: list[int]
    raw_bytes: int          # bits-per-byte denominator: a property of the text


@dataclass
class ChunkRecord:
    doc_id: int
    chunk_idx: int
    tokens: list[int]
    loss_before_adapt: float            # score-before-update loss
    loss_after_adapt: Optional[float]   # None when no weight TTT ran


@dataclass
class RunConfig:
    adapt_set: str = "none"
    persistence_mode: str = "reset"
    delta_scale: float = 1.0
    log_a_shift: float = 0.0
    chunk_size: int = 256               # -1 = whole document
    steps_per_chunk: int = 1
    eval_lr: float = 0.064
    persistent_muon_moments: bool = False
    warmup_steps: int = 20
    seed: int = 0
    max_docs: int = 50_000
    budget_seconds: float = 600.0
    score_floor_seconds: float = 0.0
    safety_margin_seconds: float = 0.0
    checkpoint_path: str = ""
    output_path: str = ""
    summary_path: str = ""
    episodic_cache_enabled: bool = False
    episodic_cache_reset_per_doc: bool = False
    episodic_cache_capacity: int = 4096
    episodic_span_length: int = 4
    episodic_key_rep_dim: int = -1
    episodic_grace_steps: int = 1000
    episodic_fingerprint_window: int = 8
    episodic_compute_replay_ce_pair: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "RunConfig":
        known = {f.name for f in fields(cls)}
        unknown = set(d) - known
        if unknown:
            raise ValueError(f"unknown RunConfig keys: {sorted(unknown)}")
        return cls(**d)
