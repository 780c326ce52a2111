"""Fatigue dynamics that decide when the model should sleep
(cf. src/chaoscontrol/fatigue.py:13-132).

Per step, with ``f`` the fatigue in [0, 1]::

    pressure = (1 - improvement_rate) * memory_pressure
    f += accumulation_rate * pressure * (1 - f)      # logistic-style soft ceiling
         - surprise_suppression * surprise * f       # alertness pulls fatigue down
         - wake_decay_rate * f                       # slow passive recovery
"""
from __future__ import annotations

__all__ = ["FatigueTracker"]


class FatigueTracker:
    def __init__(self, accumulation_rate: float = 0.02, wake_decay_rate: float = 0.005,
                 sleep_decay_rate: float = 0.3, surprise_suppression: float = 1.0) -> None:
        self.accumulation_rate = accumulation_rate
        self.wake_decay_rate = wake_decay_rate
        self.sleep_decay_rate = sleep_decay_rate
        self.surprise_suppression = surprise_suppression
        self._fatigue = 0.0

    @property
    def score(self) -> float:
        return self._fatigue

    def step(self, surprise: float, improvement_rate: float, memory_pressure: float) -> float:
        f = self._fatigue
        pressure = (1.0 - improvement_rate) * memory_pressure
        f += (self.accumulation_rate * pressure * (1.0 - f)
              - self.surprise_suppression * surprise * f
              - self.wake_decay_rate * f)
        self._fatigue = min(1.0, max(0.0, f))
        return self._fatigue

    def apply_sleep_recovery(self, sleep_quality: float) -> float:
        self._fatigue = max(0.0, self._fatigue - self.sleep_decay_rate * sleep_quality)
        return self._fatigue

    def sleep_steps(self, base_sleep: int = 128) -> int:
        """0.5x the base duration when rested, 2x when exhausted, linear between."""
        return int(base_sleep * (0.5 + 1.5 * self._fatigue))
