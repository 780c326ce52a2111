"""Wall-clock accounting of an evaluation run under the score-floor framing
(cf. src/chaoscontrol/eval_stream/budget.py:9-218): scoring time is rent, what
is left after the floor and a safety margin may be spent on adaptation."""
from __future__ import annotations

import time
from typing import Optional

FULL_VALIDATION_DOCS = 50_000


class EvalDeadline:
    def __init__(self, budget_seconds: float) -> None:
        self.budget_seconds = float(budget_seconds)
        self._t0 = time.monotonic()

    def elapsed(self) -> float:
        return time.monotonic() - self._t0

    def remaining(self) -> float:
        return self.budget_seconds - self.elapsed()

    def is_expired(self) -> bool:
        return self.remaining() <= 0.0


def compute_usable_ttt_budget(*, total_budget_seconds: float, score_floor_seconds: float,
                              safety_margin_seconds: float) -> float:
    return max(0.0, total_budget_seconds - score_floor_seconds - safety_margin_seconds)


class BudgetTracker:
    def __init__(self, *, total_budget_seconds: float, score_floor_seconds: float = 0.0,
                 safety_margin_seconds: float = 0.0) -> None:
        self.total_budget_seconds = float(total_budget_seconds)
        self.configured_score_floor_seconds = max(0.0, float(score_floor_seconds))
        self.safety_margin_seconds = max(0.0, float(safety_margin_seconds))
        self.score_wall_seconds = 0.0
        self.adapt_wall_seconds = 0.0

    @property
    def usable_ttt_budget_seconds(self) -> float:
        return compute_usable_ttt_budget(total_budget_seconds=self.total_budget_seconds,
                                         score_floor_seconds=self.configured_score_floor_seconds,
                                         safety_margin_seconds=self.safety_margin_seconds)

    @property
    def slack_remaining_seconds(self) -> float:
        return max(0.0, self.usable_ttt_budget_seconds - self.adapt_wall_seconds)

    def can_adapt(self) -> bool:
        return self.slack_remaining_seconds > 0.0

    def add_score_time(self, seconds: float) -> None:
        self.score_wall_seconds += max(0.0, float(seconds))

    def add_adapt_time(self, seconds: float) -> None:
        self.adapt_wall_seconds += max(0.0, float(seconds))

    @staticmethod
    def result_status(*, requested_docs_complete: bool, full_validation_complete: bool,
                      record_eligible: bool, timed_out: bool, collapsed: bool) -> str:
        if record_eligible:
            return "record_eligible"
        if timed_out:
            return "incomplete_timeout"
        if collapsed:
            return "incomplete_collapsed"
        if not requested_docs_complete:
            return "incomplete_docs"
        if not full_validation_complete:
            return "exploratory_prefix_complete"
        return "full_validation_over_budget"

    def summary(self, *, docs_scored: int, chunks_scored: int, tokens_scored: int, adapt_steps: int,
                timed_out: bool, collapsed: bool, score_only_mode: bool, elapsed_seconds: float,
                ckpt_sha256: Optional[str] = None, ckpt_cfg_hash: Optional[str] = None,
                stream_seed: Optional[int] = None, gpu_name: Optional[str] = None,
                torch_version: Optional[str] = None, cuda_version: Optional[str] = None,
                chunk_size: Optional[int] = None, max_docs: Optional[int] = None) -> dict:
        floor = self.configured_score_floor_seconds
        if floor <= 0.0:
            floor = max(0.0, float(elapsed_seconds)) if score_only_mode else 0.0
        usable = compute_usable_ttt_budget(total_budget_seconds=self.total_budget_seconds,
                                           score_floor_seconds=floor,
                                           safety_margin_seconds=self.safety_margin_seconds)
        requested = (max_docs is not None and int(docs_scored) >= int(max_docs) and not timed_out
                     and not collapsed)
        full = (requested and int(docs_scored) >= FULL_VALIDATION_DOCS and
                int(max_docs) >= FULL_VALIDATION_DOCS)
        eligible = full and float(elapsed_seconds) <= self.total_budget_seconds
        return {
            "total_budget_seconds": self.total_budget_seconds,
            "elapsed_seconds": float(elapsed_seconds),
            "score_wall_seconds": self.score_wall_seconds,
            "adapt_wall_seconds": self.adapt_wall_seconds,
            "other_wall_seconds": max(0.0, float(elapsed_seconds) - self.score_wall_seconds -
                                      self.adapt_wall_seconds),
            "score_floor_seconds": floor,
            "safety_margin_seconds": self.safety_margin_seconds,
            "usable_ttt_budget_seconds": usable,
            "ttt_budget_used_seconds": self.adapt_wall_seconds,
            "slack_remaining_seconds": max(0.0, usable - self.adapt_wall_seconds),
            "docs_scored": int(docs_scored), "chunks_scored": int(chunks_scored),
            "tokens_scored": int(tokens_scored), "adapt_steps": int(adapt_steps),
            "timed_out": bool(timed_out), "collapsed": bool(collapsed),
            "score_only_mode": bool(score_only_mode),
            "requested_docs_complete": bool(requested), "full_validation_complete": bool(full),
            "record_eligible": bool(eligible),
            "result_status": self.result_status(requested_docs_complete=requested,
                                                full_validation_complete=full,
                                                record_eligible=eligible, timed_out=timed_out,
                                                collapsed=collapsed),
            "provenance": {"ckpt_sha256": ckpt_sha256, "ckpt_cfg_hash": ckpt_cfg_hash,
                           "stream_seed": stream_seed, "gpu_name": gpu_name,
                           "torch_version": torch_version, "cuda_version": cuda_version,
                           "chunk_size": chunk_size, "max_docs": max_docs},
        }
