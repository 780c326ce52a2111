"""Intrinsic checks of an embedding table: cosine neighbours and k-means
(src/chaoscontrol/sgns/intrinsic.py:4-30)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def nearest_neighbors(embed: torch.Tensor, query_ids: list[int], k: int = 5) -> dict[int, list[int]]:
    """Top-``k`` cosine neighbours (self excluded) of every query id: one matmul for all queries."""
    if not query_ids:
        return {}
    normed = F.normalize(embed.float(), dim=-1)
    q = torch.as_tensor(query_ids, device=embed.device, dtype=torch.long)
    sims = normed[q] @ normed.T
    sims[torch.arange(len(query_ids), device=embed.device), q] = float("-inf")
    top = torch.topk(sims, k, dim=-1).indices.tolist()
    return {int(i): row for i, row in zip(query_ids, top)}


def kmeans_clusters(embed: torch.Tensor, k: int, n_iter: int = 20) -> torch.Tensor:
    """Lloyd's algorithm from a seed-0 random choice of rows; returns one label per row.  Empty
    clusters keep their centroid."""
    x = embed.float()
    n = x.shape[0]
    gen = torch.Generator(device="cpu").manual_seed(0)
    cent = x[torch.randperm(n, generator=gen)[:k].to(x.device)].clone()
    labels = torch.zeros(n, dtype=torch.long, device=x.device)
    for _ in range(n_iter):
        labels = torch.cdist(x, cent).argmin(-1)
        sums = torch.zeros_like(cent).index_add_(0, labels, x)
        cnt = torch.bincount(labels, minlength=k).to(x.dtype).unsqueeze(-1)
        cent = torch.where(cnt > 0, sums / cnt.clamp_min(1.0), cent)
    return labels
