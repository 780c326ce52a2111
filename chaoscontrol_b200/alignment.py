"""Losses that couple the learned tokenizer's codebook to the Wernicke
codebook (cf. src/chaoscontrol/alignment.py:18-153).  Tokenizer codes are
projected to model width before they get here.

``contrastive``   InfoNCE: the mean projected code routed to bucket j should be
                  nearer to Wernicke entry j than to any other entry.
``diversity``     mean |cosine| between the two codebooks (push them apart).
``distillation``  1 - mean cosine(mean code of bucket j, Wernicke entry j).

Buckets without a routed code in the batch are skipped.  The per-bucket means
come from one ``index_add_`` each (shared helper).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

__all__ = ["no_alignment", "contrastive_alignment", "diversity_alignment", "distillation_alignment",
           "compute_alignment_loss"]


def _bucket_means(embeds: torch.Tensor, assigns: torch.Tensor, K: int):
    """``(means [A, D], bucket ids [A])`` over the buckets that received a code."""
    flat = embeds.reshape(-1, embeds.size(-1))
    ids = assigns.reshape(-1).long()
    sums = torch.zeros(K, flat.size(-1), device=flat.device, dtype=flat.dtype).index_add_(0, ids, flat)
    cnt = torch.zeros(K, device=flat.device, dtype=flat.dtype).index_add_(0, ids, torch.ones_like(ids, dtype=flat.dtype))
    live = torch.where(cnt > 0)[0]
    return sums[live] / cnt[live].unsqueeze(-1), live


def no_alignment(**_kwargs) -> torch.Tensor:
    return torch.tensor(0.0)


def contrastive_alignment(projected_tok_embeds: torch.Tensor, wernicke_entries: torch.Tensor,
                          wernicke_assignments: torch.Tensor, temperature: float = 0.1) -> torch.Tensor:
    means, live = _bucket_means(projected_tok_embeds, wernicke_assignments, wernicke_entries.size(0))
    if live.numel() == 0:
        return torch.tensor(0.0, device=projected_tok_embeds.device)
    logits = F.normalize(means, dim=-1) @ F.normalize(wernicke_entries, dim=-1).T / temperature
    return F.cross_entropy(logits, live)          # == -mean(pos/tau - logsumexp)


def diversity_alignment(projected_tok_entries: torch.Tensor, wernicke_entries: torch.Tensor) -> torch.Tensor:
    return (F.normalize(projected_tok_entries, dim=-1) @ F.normalize(wernicke_entries, dim=-1).T).abs().mean()


def distillation_alignment(projected_tok_embeds: torch.Tensor, wernicke_entries: torch.Tensor,
                           wernicke_assignments: torch.Tensor) -> torch.Tensor:
    means, live = _bucket_means(projected_tok_embeds, wernicke_assignments, wernicke_entries.size(0))
    if live.numel() == 0:
        return torch.tensor(0.0, device=projected_tok_embeds.device)
    return 1.0 - F.cosine_similarity(means, wernicke_entries[live], dim=-1).mean()


_ALIGNMENT_FNS = {"none": no_alignment, "contrastive": contrastive_alignment,
                  "diversity": diversity_alignment, "distillation": distillation_alignment}


def compute_alignment_loss(align_type: str, **kwargs) -> torch.Tensor:
    if align_type not in _ALIGNMENT_FNS:
        raise ValueError(f"Unknown alignment type {align_type!r}. Expected one of {list(_ALIGNMENT_FNS.keys())}")
    return _ALIGNMENT_FNS[align_type](**kwargs)
