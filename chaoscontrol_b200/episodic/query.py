"""Top-K retrieval from the episodic cache
(modes of src/chaoscontrol/episodic/query.py:33-103).

``cosine_utility_weighted``  ``score(i) = cos(query, key_rep[i]) * utility_u[i]``
``pressure_only``            ``score(i) = pressure_at_write[i]`` (the control arm
                             that ignores similarity and learned utility)

Unoccupied slots never appear.  ``query_topk_batch`` scores many queries in
one matmul against a device snapshot of the cache.
"""
from __future__ import annotations

import torch

from .cache import EpisodicCache

__all__ = ["query_topk", "query_topk_batch"]

_VALID_SCORE_MODES = ("cosine_utility_weighted", "pressure_only")


def _check_mode(score_mode: str) -> None:
    if score_mode not in _VALID_SCORE_MODES:
        raise ValueError(f"score_mode must be one of {_VALID_SCORE_MODES}; got {score_mode!r}")


def query_topk(query_residual: torch.Tensor, cache: EpisodicCache, k: int,
               score_mode: str = "cosine_utility_weighted") -> torch.Tensor:
    """``[min(k, occupied)]`` int64 slot indices (into the cache), best first,
    on ``query_residual``'s device."""
    _check_mode(score_mode)
    dev = query_residual.device
    live = cache.occupied.to(dev).nonzero(as_tuple=True)[0]
    if live.numel() == 0 or k <= 0:
        return torch.empty(0, dtype=torch.int64, device=dev)
    if score_mode == "cosine_utility_weighted":
        keys = cache.key_rep.to(dev)[live]
        q = query_residual / (query_residual.norm() + 1e-8)
        scores = (keys / (keys.norm(dim=1, keepdim=True) + 1e-8)) @ q * cache.utility_u.to(dev)[live]
    else:
        scores = cache.pressure_at_write.to(dev)[live]
    return live[torch.topk(scores, min(int(k), live.numel()), largest=True).indices].to(torch.int64)


def query_topk_batch(queries: torch.Tensor, snapshot: dict[str, torch.Tensor], k: int,
                     score_mode: str = "cosine_utility_weighted"):
    """``(slots [Q, k], scores [Q, k])`` for ``queries [Q, D]`` against a
    ``cache.snapshot_to(device)`` dict.  Rows short of ``k`` live entries are
    padded with slot ``-1`` / score ``-inf``."""
    _check_mode(score_mode)
    occ = snapshot["occupied"]
    Q = queries.shape[0]
    if score_mode == "cosine_utility_weighted":
        keys = snapshot["key_rep"].to(queries.dtype)
        qn = queries / (queries.norm(dim=1, keepdim=True) + 1e-8)
        kn = keys / (keys.norm(dim=1, keepdim=True) + 1e-8)
        scores = (qn @ kn.T) * snapshot["utility_u"].to(queries.dtype)
    else:
        scores = snapshot["pressure_at_write"].to(queries.dtype).unsqueeze(0).expand(Q, -1)
    scores = scores.masked_fill(~occ.unsqueeze(0), float("-inf"))
    kk = min(int(k), scores.shape[1])
    top, idx = torch.topk(scores, kk, dim=1)
    idx = torch.where(torch.isinf(top), torch.full_like(idx, -1), idx)
    if kk < k:
        pad = k - kk
        idx = torch.cat([idx, idx.new_full((Q, pad), -1)], 1)
        top = torch.cat([top, top.new_full((Q, pad), float("-inf"))], 1)
    return idx, top
