"""Token data helpers: shard loading, LM window sampling, synthetic corpora.

``build_lm_starts`` / ``batch_from_starts`` / ``choose_eval_starts`` follow
src/chaoscontrol/data.py:316-347; ``load_fineweb_tokens`` reads the flat
little-endian uint16 shard format (data.py:120-145).  The synthetic generators
produce the Zipf / lognormal-length corpora used by the benchmarks when no
dataset is available.
"""
from __future__ import annotations

import os
import random
from pathlib import Path
from typing import Optional, Sequence

import numpy as np
import torch


def build_lm_starts(num_tokens: int, seq_len: int, stride: int) -> list[int]:
    stop = num_tokens - seq_len - 1
    if stop <= 0:
        return []
    return list(range(0, stop, stride))


def batch_from_starts(tokens: torch.Tensor, starts: Sequence[int], seq_len: int,
                      device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    windows = [tokens[s: s + seq_len + 1] for s in starts]
    batch = torch.stack(windows).to(device=device, dtype=torch.long)
    return batch[:, :-1], batch[:, 1:]


def batch_from_start_tensor(tokens: torch.Tensor, starts: torch.Tensor, seq_len: int,
                            device: torch.device, *, vocab_size: Optional[int] = None,
                            pin: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Vectorised window gather: int32 inputs and int64 targets
    (cf. experiments/23_fast_path/fast_path.py:159-186)."""
    idx = starts.view(-1, 1).long() + torch.arange(seq_len + 1).view(1, -1)
    win = tokens[idx]
    if vocab_size is not None:
        win = win.clamp(0, vocab_size - 1)
    inputs = win[:, :-1].to(torch.int32)
    targets = win[:, 1:].to(torch.int64)
    if pin and torch.cuda.is_available():
        inputs, targets = inputs.pin_memory(), targets.pin_memory()
    return (inputs.to(device, non_blocking=True), targets.to(device, non_blocking=True))


def choose_eval_starts(starts: list[int], *, batch_size: int, eval_batches: int, seed: int) -> list[int]:
    needed = batch_size * eval_batches
    if not starts:
        return []
    if len(starts) <= needed:
        return starts[:needed]
    return random.Random(seed).sample(starts, needed)


def load_fineweb_tokens(data_dir: str | os.PathLike, split: str = "train",
                        max_shards: Optional[int] = None) -> torch.Tensor:
    """Concatenate ``*{split}*.bin`` shards of flat uint16 tokens into one int16-viewed
    tensor (memory-mapped, no header)."""
    paths = sorted(Path(data_dir).glob(f"*{split}*.bin"))
    if max_shards is not None:
        paths = paths[:max_shards]
    if not paths:
        raise FileNotFoundError(f"no '*{split}*.bin' shards under {data_dir}")
    arrs = [np.memmap(p, dtype=np.uint16, mode="r") for p in paths]
    cat = arrs[0] if len(arrs) == 1 else np.concatenate(arrs)
    return torch.from_numpy(np.asarray(cat).view(np.int16))


def zipf_tokens(n: int, vocab: int, *, s: float = 1.1, seed: int = 0,
                dtype: torch.dtype = torch.int64) -> torch.Tensor:
    """``n`` iid tokens with ``P(k) ~ (k+1)^-s`` over ``vocab`` ids (inverse-CDF sampling)."""
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    rng = np.random.default_rng(seed)
    ids = np.searchsorted(cdf, rng.random(n), side="left").clip(0, vocab - 1)
    return torch.from_numpy(ids).to(dtype)


def lognormal_doc_lengths(n_docs: int, *, median: float = 700.0, sigma: float = 1.0,
                          lo: int = 32, hi: int = 32768, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    lens = rng.lognormal(mean=np.log(median), sigma=sigma, size=n_docs)
    return np.clip(lens, lo, hi).astype(np.int64)
