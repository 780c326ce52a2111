"""Wall-clock ledger of an evaluation run.

Contract (the summary's key set and the status vocabulary are a result schema
shared with the reference's evaluation reports, src/chaoscontrol/eval_stream/
budget.py:9-218): the time a plain scoring pass needs is a fixed cost of the
run (the *score floor*); what remains of the budget after the floor and a
safety margin may be spent on test-time adaptation; a run counts for the record
only if it scored the whole validation set within the budget.

Layout here: the ledger is a dict of named phases, the booleans of a finished
run are derived in one place (:class:`_Outcome`), and the status string comes
from an ordered rule table.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

FULL_VALIDATION_DOCS = 50_000          # documents in the full validation set


def compute_usable_ttt_budget(*, total_budget_seconds: float, score_floor_seconds: float,
                              safety_margin_seconds: float) -> float:
    """Seconds that adaptation may use: budget minus floor minus margin, never negative."""
    left = float(total_budget_seconds) - float(score_floor_seconds) - float(safety_margin_seconds)
    return left if left > 0.0 else 0.0


class EvalDeadline:
    """Monotonic countdown started at construction."""

    def __init__(self, budget_seconds: float) -> None:
        self.budget_seconds = float(budget_seconds)
        self._started = time.monotonic()

    def elapsed(self) -> float:
        return time.monotonic() - self._started

    def remaining(self) -> float:
        return self.budget_seconds - self.elapsed()

    def is_expired(self) -> bool:
        return self.elapsed() >= self.budget_seconds


@dataclass(frozen=True)
class _Outcome:
    """What a finished run achieved, derived once from the counters."""
    requested_docs_complete: bool
    full_validation_complete: bool
    record_eligible: bool
    timed_out: bool
    collapsed: bool

    @classmethod
    def of(cls, *, docs_scored: int, max_docs: Optional[int], elapsed: float, budget: float, timed_out: bool,
           collapsed: bool) -> "_Outcome":
        clean = not (timed_out or collapsed)
        got_all = clean and max_docs is not None and docs_scored >= int(max_docs)
        whole_set = got_all and min(docs_scored, int(max_docs)) >= FULL_VALIDATION_DOCS
        return cls(got_all, whole_set, whole_set and elapsed <= budget, bool(timed_out), bool(collapsed))

    # first matching rule names the run
    _RULES = (
        ("record_eligible", lambda o: o.record_eligible),
        ("incomplete_timeout", lambda o: o.timed_out),
        ("incomplete_collapsed", lambda o: o.collapsed),
        ("incomplete_docs", lambda o: not o.requested_docs_complete),
        ("exploratory_prefix_complete", lambda o: not o.full_validation_complete),
    )

    @property
    def status(self) -> str:
        for name, rule in self._RULES:
            if rule(self):
                return name
        return "full_validation_over_budget"


class BudgetTracker:
    def __init__(self, *, total_budget_seconds: float, score_floor_seconds: float = 0.0,
                 safety_margin_seconds: float = 0.0) -> None:
        self.total_budget_seconds = float(total_budget_seconds)
        self.configured_score_floor_seconds = max(0.0, float(score_floor_seconds))
        self.safety_margin_seconds = max(0.0, float(safety_margin_seconds))
        self._spent = {"score": 0.0, "adapt": 0.0}

    # -- ledger ------------------------------------------------------------
    def _charge(self, phase: str, seconds: float) -> None:
        if seconds > 0.0:
            self._spent[phase] += float(seconds)

    def add_score_time(self, seconds: float) -> None:
        self._charge("score", seconds)

    def add_adapt_time(self, seconds: float) -> None:
        self._charge("adapt", seconds)

    @property
    def score_wall_seconds(self) -> float:
        return self._spent["score"]

    @property
    def adapt_wall_seconds(self) -> float:
        return self._spent["adapt"]

    # -- what adaptation may still use ---------------------------------------
    def _usable(self, floor: float) -> float:
        return compute_usable_ttt_budget(total_budget_seconds=self.total_budget_seconds, score_floor_seconds=floor,
                                         safety_margin_seconds=self.safety_margin_seconds)

    @property
    def usable_ttt_budget_seconds(self) -> float:
        return self._usable(self.configured_score_floor_seconds)

    @property
    def slack_remaining_seconds(self) -> float:
        return max(0.0, self.usable_ttt_budget_seconds - self.adapt_wall_seconds)

    def can_adapt(self) -> bool:
        return self.slack_remaining_seconds > 0.0

    @staticmethod
    def result_status(*, requested_docs_complete: bool, full_validation_complete: bool, record_eligible: bool,
                      timed_out: bool, collapsed: bool) -> str:
        return _Outcome(requested_docs_complete, full_validation_complete, record_eligible, timed_out,
                        collapsed).status

    # -- report ----------------------------------------------------------------
    def summary(self, *, docs_scored: int, chunks_scored: int, tokens_scored: int, adapt_steps: int,
                timed_out: bool, collapsed: bool, score_only_mode: bool, elapsed_seconds: float,
                ckpt_sha256: Optional[str] = None, ckpt_cfg_hash: Optional[str] = None,
                stream_seed: Optional[int] = None, gpu_name: Optional[str] = None,
                torch_version: Optional[str] = None, cuda_version: Optional[str] = None,
                chunk_size: Optional[int] = None, max_docs: Optional[int] = None) -> dict:
        elapsed = float(elapsed_seconds)
        # a score-only run with no configured floor IS the floor measurement
        floor = self.configured_score_floor_seconds or (max(0.0, elapsed) if score_only_mode else 0.0)
        usable = self._usable(floor)
        out = _Outcome.of(docs_scored=int(docs_scored), max_docs=max_docs, elapsed=elapsed,
                          budget=self.total_budget_seconds, timed_out=timed_out, collapsed=collapsed)
        clock = {
            "total_budget_seconds": self.total_budget_seconds,
            "elapsed_seconds": elapsed,
            "score_wall_seconds": self.score_wall_seconds,
            "adapt_wall_seconds": self.adapt_wall_seconds,
            "other_wall_seconds": max(0.0, elapsed - self.score_wall_seconds - self.adapt_wall_seconds),
            "score_floor_seconds": floor,
            "safety_margin_seconds": self.safety_margin_seconds,
            "usable_ttt_budget_seconds": usable,
            "ttt_budget_used_seconds": self.adapt_wall_seconds,
            "slack_remaining_seconds": max(0.0, usable - self.adapt_wall_seconds),
        }
        counts = {"docs_scored": int(docs_scored), "chunks_scored": int(chunks_scored),
                  "tokens_scored": int(tokens_scored), "adapt_steps": int(adapt_steps)}
        verdict = {"timed_out": out.timed_out, "collapsed": out.collapsed, "score_only_mode": bool(score_only_mode),
                   "requested_docs_complete": out.requested_docs_complete,
                   "full_validation_complete": out.full_validation_complete,
                   "record_eligible": out.record_eligible, "result_status": out.status}
        provenance = {"ckpt_sha256": ckpt_sha256, "ckpt_cfg_hash": ckpt_cfg_hash, "stream_seed": stream_seed,
                      "gpu_name": gpu_name, "torch_version": torch_version, "cuda_version": cuda_version,
                      "chunk_size": chunk_size, "max_docs": max_docs}
        return {**clock, **counts, **verdict, "provenance": provenance}
