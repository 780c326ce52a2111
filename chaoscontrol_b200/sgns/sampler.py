"""Unigram^power negative sampling (src/chaoscontrol/sgns/sampler.py:4-23)."""
from __future__ import annotations

import torch


def unigram_probs_from_counts(counts: torch.Tensor, power: float = 0.75) -> torch.Tensor:
    """``counts ** power`` normalised (uniform for ``power == 0``)."""
    if power == 0.0:
        return torch.full_like(counts, 1.0 / len(counts), dtype=torch.float32)
    w = counts.clamp(min=0).float().pow(power)
    return w / w.sum()


class NegativeSampler:
    def __init__(self, probs: torch.Tensor) -> None:
        probs = probs.float()
        if not torch.isclose(probs.sum(), probs.new_tensor(1.0), atol=1e-4):
            raise AssertionError("negative-sampling probabilities must sum to 1")
        self.probs = probs

    def sample(self, batch_size: int, k: int) -> torch.Tensor:
        return torch.multinomial(self.probs, batch_size * k, replacement=True).view(batch_size, k)
