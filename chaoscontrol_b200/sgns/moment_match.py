"""Transforms that carry the statistics of one embedding table onto another, and
the shuffled / synthetic controls that go with them
(src/chaoscontrol/sgns/moment_match.py:22-182)."""
from __future__ import annotations

import unicodedata
from collections.abc import Sequence
from typing import Optional

import torch
import torch.nn.functional as F


def _gen(seed: int, device: Optional[torch.device] = None) -> torch.Generator:
    if device is not None:
        try:
            return torch.Generator(device=device).manual_seed(seed)
        except (RuntimeError, TypeError):
            pass
    return torch.Generator().manual_seed(seed)


def _need_2d(t: torch.Tensor) -> None:
    if t.dim() != 2:
        raise ValueError(f"expected a 2D tensor, got shape={tuple(t.shape)}")


def match_row_norm_moments(src: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Rescales every row of ``src`` (direction untouched) so that the row norms have the mean and
    standard deviation of ``target``'s row norms."""
    sn, tn = src.norm(dim=-1), target.norm(dim=-1)
    z = (sn - sn.mean()) / sn.std().clamp(min=1e-8)
    return src * ((z * tn.std() + tn.mean()) / sn.clamp(min=1e-12)).unsqueeze(-1)


def _chol_cov(x: torch.Tensor) -> torch.Tensor:
    eye = torch.eye(x.shape[1], device=x.device, dtype=x.dtype)
    return torch.linalg.cholesky(torch.cov(x.T) + 1e-6 * eye)


def match_full_covariance(src: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Whitens ``src`` with the Cholesky factor of its covariance, re-colours with ``target``'s and
    moves to ``target``'s mean."""
    sc = src - src.mean(0)
    white = torch.linalg.solve_triangular(_chol_cov(sc), sc.T, upper=False).T
    return white @ _chol_cov(target - target.mean(0)).T + target.mean(0)


def shuffle_rows(src: torch.Tensor, seed: int) -> torch.Tensor:
    """Seeded row permutation: same marginals, id -> vector map destroyed."""
    return src[torch.randperm(src.shape[0], generator=_gen(seed, src.device), device=src.device)].clone()


def sample_with_row_norms(reference: torch.Tensor, *, seed: int, shuffle_norms_seed: Optional[int] = None
                          ) -> torch.Tensor:
    """Random unit directions scaled by ``reference``'s row norms (optionally permuted across ids)."""
    _need_2d(reference)
    dirs = F.normalize(torch.randn(reference.shape, generator=_gen(seed, reference.device), device=reference.device,
                                   dtype=reference.dtype), dim=-1)
    norms = reference.norm(dim=-1)
    if shuffle_norms_seed is not None:
        norms = norms[torch.randperm(norms.shape[0], generator=_gen(shuffle_norms_seed, reference.device),
                                     device=reference.device)]
    return dirs * norms.unsqueeze(-1)


def shuffle_rows_within_buckets(src: torch.Tensor, bucket_ids: torch.Tensor, *, seed: int) -> torch.Tensor:
    """Permutes rows only among ids of the same bucket: one sort by (bucket, random key)."""
    _need_2d(src)
    if bucket_ids.dim() != 1 or bucket_ids.shape[0] != src.shape[0]:
        raise ValueError("bucket_ids must be a 1D tensor with one entry per source row; "
                         f"got bucket_ids={tuple(bucket_ids.shape)} src={tuple(src.shape)}")
    b = bucket_ids.to(src.device)
    n = src.shape[0]
    key = torch.rand(n, generator=_gen(seed, src.device), device=src.device)
    # positions of each bucket in id order, and the same positions in a random order within the bucket
    place = torch.argsort(b, stable=True)
    donor = place[torch.argsort(b[place].double() * 2.0 + key[place].double(), stable=True)]
    out = src.clone()
    out[place] = src[donor]
    return out


def frequency_bucket_ids(counts: torch.Tensor, *, num_buckets: int) -> torch.Tensor:
    """Equal-size buckets by descending count rank (bucket 0 = most frequent)."""
    if counts.dim() != 1:
        raise ValueError(f"counts must be 1D, got shape={tuple(counts.shape)}")
    if num_buckets <= 0:
        raise ValueError(f"num_buckets must be positive, got {num_buckets}")
    n = counts.shape[0]
    out = torch.empty(n, dtype=torch.long, device=counts.device)
    if n:
        order = torch.argsort(counts.float(), descending=True, stable=True)
        out[order] = (torch.arange(n, device=counts.device) * num_buckets // n).clamp(max=num_buckets - 1)
    return out


def token_class_bucket_ids(pieces: Sequence[str]) -> torch.Tensor:
    """0 leading-space / whitespace, 1 punctuation, 2 numeric, 3 alphabetic, 4 other."""
    def cls(text: str) -> int:
        if text.startswith("▁") or text.strip() == "":
            return 0
        if text and all(unicodedata.category(ch).startswith("P") for ch in text):
            return 1
        if text.isnumeric():
            return 2
        return 3 if text.isalpha() else 4
    return torch.tensor([cls(str(p)) for p in pieces], dtype=torch.long)


def sample_full_covariance(reference: torch.Tensor, *, seed: int) -> torch.Tensor:
    """Gaussian cloud with ``reference``'s mean and covariance."""
    _need_2d(reference)
    noise = torch.randn(reference.shape, generator=_gen(seed, reference.device), device=reference.device,
                        dtype=reference.dtype)
    return match_full_covariance(noise, reference)
