"""Mixed-precision policy: ``autocast_context`` and the linear-promotion helpers
(API of src/chaoscontrol/precision.py:100-301 in the reference).

``fp8`` here is the library's own delayed-scaling e4m3/e5m2 path (no Transformer
Engine): ``"fp8"`` and ``"fp8_fused"`` both mean bf16 ambient autocast with
eligible ``nn.Linear`` modules swapped for :class:`..ops.fp8_linear.FusedFP8Linear`.
"""
from __future__ import annotations

import contextlib

import torch
import torch.nn as nn

_SUPPORTED = ("fp32", "bf16", "fp8", "fp8_fused")


@contextlib.contextmanager
def autocast_context(dtype: str, device_type: str = "cuda"):
    if dtype not in _SUPPORTED:
        raise ValueError(f"Unsupported precision dtype: {dtype!r}. "
                         "Expected one of {'fp32', 'bf16', 'fp8', 'fp8_fused'}.")
    if dtype == "fp32" or device_type != "cuda":
        with contextlib.nullcontext():
            yield
        return
    with torch.amp.autocast(device_type=device_type, dtype=torch.bfloat16):
        yield


def _eligible(name: str, mod: nn.Module) -> bool:
    if not isinstance(mod, nn.Linear) or type(mod) is not nn.Linear:
        return False
    if "lm_head" in name:
        return False
    return mod.in_features % 16 == 0 and mod.out_features % 16 == 0


def maybe_promote_linears_to_fused_fp8(model: nn.Module, enabled: bool, *, scaling: str = "tensor") -> int:
    """Swap eligible ``nn.Linear`` modules (16-aligned, not the LM head) for the
    fp8 linear; returns how many were promoted.

    ``scaling="tensor"`` is the reference's recipe (per-tensor delayed scaling, e4m3
    forward / e5m2 gradients).  ``scaling="block"`` uses e4m3 with 1 x 128 activation and
    128 x 128 weight scales (``in_features`` must then be a multiple of 128) and makes
    every RMSNorm of the model emit the quantised row for the linears it feeds."""
    if not enabled:
        return 0
    if scaling not in ("tensor", "block"):
        raise ValueError(f"scaling must be 'tensor' or 'block', got {scaling!r}")
    from .ops.fp8_block import BlockFP8Linear
    from .ops.fp8_linear import FusedFP8Linear
    count = 0
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            full = f"{parent_name}.{child_name}" if parent_name else child_name
            if not _eligible(full, child):
                continue
            if scaling == "block":
                if child.in_features % 128:
                    continue
                setattr(parent, child_name, BlockFP8Linear.from_nn_linear(child))
            else:
                setattr(parent, child_name, FusedFP8Linear.from_nn_linear(child))
            count += 1
    if scaling == "block" and count:
        from .models.core import RMSNorm
        for m in model.modules():
            if isinstance(m, RMSNorm):
                m.emit_fp8_blocks = True
    return count


def maybe_promote_linears_to_te(model: nn.Module, enabled: bool) -> int:
    """Kept for API parity: the Transformer-Engine recipe is served by the same
    in-tree fp8 linear."""
    return maybe_promote_linears_to_fused_fp8(model, enabled)
