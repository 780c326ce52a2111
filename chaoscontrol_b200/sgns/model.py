"""Two-table skip-gram model and its negative-sampling loss
(src/chaoscontrol/sgns/model.py:6-46)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class SGNSModel(nn.Module):
    """``input_embed`` (centre words, N(0, 0.01) init) is the product; ``output_embed``
    (contexts / negatives, zero init) is discarded after training."""

    def __init__(self, vocab_size: int, dim: int) -> None:
        super().__init__()
        self.input_embed = nn.Embedding(vocab_size, dim)
        self.output_embed = nn.Embedding(vocab_size, dim)
        nn.init.normal_(self.input_embed.weight, mean=0.0, std=0.01)
        nn.init.zeros_(self.output_embed.weight)

    def score_pairs(self, center: torch.Tensor, context: torch.Tensor) -> torch.Tensor:
        return (self.input_embed(center) * self.output_embed(context)).sum(-1)


def nce_loss(model: SGNSModel, center: torch.Tensor, context: torch.Tensor, negatives: torch.Tensor) -> torch.Tensor:
    """``mean_b [ -log sigma(<c_b, o_b>) - sum_k log sigma(-<c_b, n_bk>) ]`` for ``center`` /
    ``context`` ``[B]`` and ``negatives`` ``[B, K]``.  The positive is scored as column 0 of one
    batched product with the negatives."""
    c = model.input_embed(center)                                                # [B, D]
    others = model.output_embed(torch.cat([context.unsqueeze(1), negatives], 1))  # [B, 1 + K, D]
    scores = torch.bmm(others, c.unsqueeze(-1)).squeeze(-1)                      # [B, 1 + K]
    sign = torch.ones_like(scores)
    sign[:, 1:] = -1.0
    return -F.logsigmoid(sign * scores).sum(-1).mean()
