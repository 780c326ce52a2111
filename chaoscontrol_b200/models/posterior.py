"""Error-driven posterior corrections added to the hidden stream: one global
delta, one delta per routing bucket, or a cosine-addressed cache of past
corrections (cf. src/chaoscontrol/posterior.py:22-178)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class GlobalDelta(nn.Module):
    def __init__(self, model_dim: int, lr: float = 0.01) -> None:
        super().__init__()
        self.model_dim, self.lr = model_dim, lr
        self.register_buffer("delta", torch.zeros(1, model_dim))

    def read(self, batch_size: int) -> torch.Tensor:
        return self.delta.expand(batch_size, -1)

    def update(self, prediction_error_grad: torch.Tensor) -> None:
        g = prediction_error_grad.detach().reshape(1, -1)
        self.delta = (self.delta + self.lr * g).detach()

    def reset(self) -> None:
        self.delta.zero_()


class BucketDelta(nn.Module):
    def __init__(self, k_max: int, model_dim: int, lr: float = 0.01) -> None:
        super().__init__()
        self.k_max, self.model_dim, self.lr = k_max, model_dim, lr
        self.register_buffer("deltas", torch.zeros(k_max, model_dim))

    def read(self, bucket_id: int, batch_size: int) -> torch.Tensor:
        return self.deltas[bucket_id].unsqueeze(0).expand(batch_size, -1)

    def update(self, bucket_id: int, prediction_error_grad: torch.Tensor) -> None:
        self.deltas[bucket_id] = (self.deltas[bucket_id] + self.lr * prediction_error_grad.detach().reshape(-1)).detach()

    def reset(self) -> None:
        self.deltas.zero_()


class ResidualCache(nn.Module):
    """FIFO store of ``(context key, correction)`` pairs; a read is the softmax-
    weighted sum of the ``k`` corrections whose keys are most cosine-similar."""

    def __init__(self, model_dim: int, k: int = 4, max_entries: int = 256) -> None:
        super().__init__()
        self.model_dim, self.k, self.max_entries = model_dim, k, max_entries
        self._keys: list[torch.Tensor] = []
        self._values: list[torch.Tensor] = []

    def read(self, query: torch.Tensor) -> torch.Tensor:
        if not self._keys:
            return torch.zeros(query.shape[0], self.model_dim, device=query.device, dtype=query.dtype)
        keys, vals = torch.cat(self._keys, 0).to(query), torch.cat(self._values, 0).to(query)
        sim = F.normalize(query.detach(), dim=-1) @ F.normalize(keys, dim=-1).T
        top, idx = sim.topk(min(self.k, sim.shape[1]), dim=-1)
        return (F.softmax(top, dim=-1).unsqueeze(-1) * vals[idx]).sum(dim=1)

    def store(self, context_key: torch.Tensor, correction_value: torch.Tensor) -> None:
        self._keys.append(context_key.detach().reshape(1, -1))
        self._values.append(correction_value.detach().reshape(1, -1))
        if len(self._keys) > self.max_entries:
            self._keys = self._keys[-self.max_entries:]
            self._values = self._values[-self.max_entries:]

    def reset(self) -> None:
        self._keys.clear()
        self._values.clear()
