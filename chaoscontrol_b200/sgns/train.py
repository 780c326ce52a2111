"""One SGNS epoch over a token stream (src/chaoscontrol/sgns/train.py:9-75).

Pairs are never materialised as a whole: each (offset, direction) is a pair of
views of the stream, visited in random order, and only the batch order inside a
view is shuffled.  The epoch loss is accumulated on the device and read once."""
from __future__ import annotations

from collections.abc import Iterator
from typing import Optional

import torch
from torch.optim import Optimizer

from .model import SGNSModel, nce_loss
from .sampler import NegativeSampler


def iter_center_context_batches(stream: torch.Tensor, window: int, batch_size: int
                                ) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
    n = int(stream.numel())
    if window <= 0 or n <= 1:
        return
    reach = min(window, n - 1)
    views = [(o, fwd) for fwd in (True, False) for o in range(1, reach + 1)]
    for vi in torch.randperm(len(views)).tolist():
        o, fwd = views[vi]
        centers, contexts = (stream[o:], stream[:-o]) if fwd else (stream[:-o], stream[o:])
        pairs = int(centers.numel())
        for b in torch.randperm((pairs + batch_size - 1) // batch_size).tolist():
            s = b * batch_size
            yield centers[s:s + batch_size], contexts[s:s + batch_size]


_iter_center_context_batches = iter_center_context_batches


def train_one_epoch(model: SGNSModel, stream: torch.Tensor, sampler: NegativeSampler, window: int, k: int,
                    batch_size: int, opt: Optimizer, max_batches: Optional[int] = None) -> float:
    """Mean loss over the processed batches."""
    total = torch.zeros((), device=model.input_embed.weight.device)
    done = 0
    for c, ctx in iter_center_context_batches(stream, window, batch_size):
        if max_batches is not None and done >= max_batches:
            break
        neg = sampler.sample(batch_size=len(c), k=k).to(c.device)
        loss = nce_loss(model, c, ctx, neg)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        total += loss.detach()
        done += 1
    return float(total) / max(done, 1)
