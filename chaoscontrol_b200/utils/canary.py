"""Out-of-bounds write detection for kernels without a sanitizer: output tensors are carved out of
a larger allocation whose margins hold a known byte pattern, and the margins are checked after the
launch.  (The reference has no sanitizer use at all; this, the determinism re-runs and the
small-shape sweeps against fp32 statements are this repository's race / bounds checks.)"""
from __future__ import annotations

from typing import Sequence

import torch

PATTERN = 0xA5
MARGIN_BYTES = 4096

__all__ = ["guarded_empty", "check_canaries", "PATTERN", "MARGIN_BYTES"]

_GUARDS: list[tuple[torch.Tensor, int, int, str]] = []


def guarded_empty(shape: Sequence[int], *, dtype: torch.dtype, device, name: str = "") -> torch.Tensor:
    """A contiguous tensor of ``shape`` with ``MARGIN_BYTES`` of pattern bytes before and after it
    (the data start keeps 256-byte alignment)."""
    numel = 1
    for s in shape:
        numel *= int(s)
    item = torch.empty((), dtype=dtype).element_size()
    nbytes = numel * item
    pad_after = (-nbytes) % 256 + MARGIN_BYTES
    raw = torch.full((MARGIN_BYTES + nbytes + pad_after,), PATTERN, dtype=torch.uint8, device=device)
    _GUARDS.append((raw, MARGIN_BYTES, nbytes, name or f"guard{len(_GUARDS)}"))
    return raw[MARGIN_BYTES:MARGIN_BYTES + nbytes].view(dtype).view(*shape)


def check_canaries(*, clear: bool = True) -> None:
    """Raises ``AssertionError`` naming the first tensor whose margins were written to."""
    bad = []
    for raw, lo, n, name in _GUARDS:
        before, after = raw[:lo], raw[lo + n:]
        if bool((before != PATTERN).any()) or bool((after != PATTERN).any()):
            nb = int((before != PATTERN).sum())
            na = int((after != PATTERN).sum())
            bad.append(f"{name}: {nb} bytes before / {na} bytes after the tensor were overwritten")
    if clear:
        _GUARDS.clear()
    if bad:
        raise AssertionError("out-of-bounds writes detected: " + "; ".join(bad))
