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


def maybe_promote_linears_to_fused_fp8(model: nn.Module, enabled: bool) -> int:
    """Swap eligible ``nn.Linear`` modules (16-aligned, not the LM head) for the
    fp8 linear; returns how many were promoted."""
    if not enabled:
        return 0
    from .ops.fp8_linear import FusedFP8Linear
    count = 0
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            full = f"{parent_name}.{child_name}" if parent_name else child_name
            if _eligible(full, child):
                setattr(parent, child_name, FusedFP8Linear.from_nn_linear(child))
                count += 1
    return count


def maybe_promote_linears_to_te(model: nn.Module, enabled: bool) -> int:
    """Kept for API parity: the Transformer-Engine recipe is served by the same
    in-tree fp8 linear."""
    return maybe_promote_linears_to_fused_fp8(model, enabled)
