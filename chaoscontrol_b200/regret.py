"""Counterfactual regret per routing bucket with regret matching
(cf. src/chaoscontrol/regret.py:12-53): actions not taken accumulate
``counterfactual - actual``; the exploration strategy is proportional to the
positive part.  Single agent, so regret steers exploration, not equilibrium."""
from __future__ import annotations

import torch

__all__ = ["RegretTable"]


class RegretTable:
    def __init__(self, n_buckets: int, n_actions: int) -> None:
        self.n_buckets, self.n_actions = n_buckets, n_actions
        self.cumulative_regret = torch.zeros(n_buckets, n_actions)

    def update(self, bucket_id: int, action_taken: int, counterfactual_values, actual_value: float) -> None:
        delta = torch.as_tensor(list(counterfactual_values), dtype=torch.float32) - float(actual_value)
        delta[action_taken] = 0.0
        self.cumulative_regret[bucket_id] += delta

    def get_regrets(self, bucket_id: int) -> torch.Tensor:
        return self.cumulative_regret[bucket_id].clone()

    def get_strategy(self, bucket_id: int) -> torch.Tensor:
        pos = self.cumulative_regret[bucket_id].clamp(min=0)
        total = pos.sum()
        return pos / total if total > 0 else torch.full((self.n_actions,), 1.0 / self.n_actions)

    def reset_bucket(self, bucket_id: int) -> None:
        self.cumulative_regret[bucket_id] = 0
