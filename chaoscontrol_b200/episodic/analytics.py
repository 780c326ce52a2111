"""Queries over the per-replay NDJSON logs of a run directory (API of
src/chaoscontrol/episodic/analytics.py:39-116, where every query is still a
``NotImplementedError`` stub behind an optional DuckDB import).  Here the logs
are read with pandas and the four canonical queries are implemented.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np
import pandas as pd

LOG_GLOB = "episodic_replay_log_rank*.ndjson"

__all__ = ["ReplayLogQuery", "LOG_GLOB"]


@dataclass
class ReplayLogQuery:
    run_dir: Path
    table: pd.DataFrame

    @classmethod
    def open(cls, run_dir: Path | str) -> "ReplayLogQuery":
        """Loads every ``episodic_replay_log_rank*.ndjson`` under ``run_dir`` into one table
        (a ``rank`` column is added); ``FileNotFoundError`` when none matches."""
        run_dir = Path(run_dir)
        files = sorted(run_dir.glob(LOG_GLOB))
        if not files:
            raise FileNotFoundError(f"no {LOG_GLOB} under {run_dir}")
        frames = []
        for f in files:
            df = pd.read_json(f, lines=True)
            df["rank"] = int("".join(ch for ch in f.stem.rsplit("rank", 1)[-1] if ch.isdigit()) or 0)
            frames.append(df)
        return cls(run_dir, pd.concat(frames, ignore_index=True))

    def close(self) -> None:
        self.table = self.table.iloc[0:0]

    def __enter__(self) -> "ReplayLogQuery":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()

    # ------------------------------------------------------------------ canonical queries
    def cohort_replay_utility(self) -> pd.DataFrame:
        """Per write-bucket cohort: ``(write_bucket, n_replays, mean_cos_rare, mean_replay_loss,
        mean_utility_post)``."""
        g = self.table.groupby("write_bucket", dropna=False)
        return g.agg(n_replays=("step", "size"), mean_cos_rare=("replay_grad_cos_rare", "mean"),
                     mean_replay_loss=("replay_loss", "mean"),
                     mean_utility_post=("utility_post", "mean")).reset_index()

    def drift_trajectory_per_entry(self, *, window_steps: int = 512) -> pd.DataFrame:
        """Per entry ``(slot, write_step, key_fp)``: mean absolute change of ``utility_post`` between
        consecutive replays inside each ``window_steps`` window (``drift_norm_avg``)."""
        t = self.table.sort_values(["slot", "key_fp", "step"]).copy()
        key = ["slot", "write_step", "key_fp"]
        t["window"] = (t["step"] // max(int(window_steps), 1)).astype("int64")
        t["delta"] = t.groupby(key + ["window"])["utility_post"].diff().abs()
        out = t.groupby(key, dropna=False)["delta"].mean().rename("drift_norm_avg").reset_index()
        out["drift_norm_avg"] = out["drift_norm_avg"].fillna(0.0)
        return out

    def surprise_frontier(self, *, bucket_steps: int = 100) -> pd.DataFrame:
        """``(step_bucket, write_bucket)`` cells with mean write pressure, mean replay loss, their product
        (``frontier``) and the row count."""
        t = self.table.copy()
        t["step_bucket"] = (t["step"] // max(int(bucket_steps), 1)).astype("int64")
        g = t.groupby(["step_bucket", "write_bucket"], dropna=False)
        out = g.agg(mean_write_pressure=("write_pressure", "mean"), mean_replay_loss=("replay_loss", "mean"),
                    n=("step", "size")).reset_index()
        out["frontier"] = out["mean_write_pressure"] * out["mean_replay_loss"]
        return out

    def retrieval_utility_correlation(self) -> dict[str, float]:
        """Pearson correlation of the retrieval score with the replay's usefulness
        (``replay_grad_cos_rare`` and, as the always-available proxy, ``reward_shaped``)."""
        out: dict[str, float] = {}
        for col in ("replay_grad_cos_rare", "reward_shaped"):
            pair = self.table[["query_cosine", col]].apply(pd.to_numeric, errors="coerce").dropna()
            ok = len(pair) >= 2 and pair["query_cosine"].std() > 0 and pair[col].std() > 0
            out[col] = float(np.corrcoef(pair["query_cosine"], pair[col])[0, 1]) if ok else float("nan")
        out["n"] = float(len(self.table))
        return out
