"""Autograd-level LM-head / loss ops with the reference's public names
(src/chaoscontrol/kernels/_lm_head_loss/__init__.py:1020-1560):
``fused_rms_norm``, ``fused_linear_cross_entropy[_with_ce]`` and the weighted
forms, ``fused_rms_linear_cross_entropy``, ``fused_lm_head_forward_with_ce_entropy``.

On CUDA (bf16, dim 256, vocab % 128 == 0) these run the tcgen05 kernels of
``csrc/lmhead.cu``; the ``backend`` / ``tile_size`` arguments are accepted for
compatibility (there is one implementation: streaming, logits never stored).
Other shapes and CPU tensors take the exact PyTorch expression.  Unknown
backend names raise instead of silently falling back.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import _lib
from ..ops import lm_head as LH
from ..ops.trunk import splitk_reduce

_BACKENDS = {"auto", "v1", "streaming", "streaming_v2", "streaming_cached"}


def _check_backend(backend: str) -> None:
    if str(backend).strip().lower() not in _BACKENDS:
        raise ValueError(f"unknown fused linear+CE backend {backend!r}; expected one of {sorted(_BACKENDS)}")


# ---------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------
class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D).contiguous()
        R = x2.shape[0]
        w = weight.to(torch.bfloat16).contiguous()
        y = torch.empty_like(x2)
        inv = torch.empty(R, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().ccb_rmsnorm_fwd(x2.data_ptr(), None, w.data_ptr(), y.data_ptr(), None,
                                              inv.data_ptr(), R, D, float(eps), _lib.stream_ptr()),
                   "rmsnorm_fwd")
        ctx.save_for_backward(x2, w, inv)
        ctx.shp = shp
        ctx.wdtype = weight.dtype
        return y.view(shp)

    @staticmethod
    def backward(ctx, go):
        x2, w, inv = ctx.saved_tensors
        R, D = x2.shape
        go2 = go.reshape(-1, D).contiguous().to(torch.bfloat16)
        gx = torch.empty_like(x2)
        nb = int(_lib.lib().ccb_rmsnorm_bwd_blocks(R))
        part = torch.empty(nb, D, dtype=torch.float32, device=x2.device)
        gw = torch.empty(D, dtype=torch.float32, device=x2.device)
        _lib.check(_lib.lib().ccb_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), go2.data_ptr(),
                                              inv.data_ptr(), gx.data_ptr(), part.data_ptr(),
                                              gw.data_ptr(), R, D, _lib.stream_ptr()), "rmsnorm_bwd")
        return gx.view(ctx.shp), gw.to(ctx.wdtype), None


def fused_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight`` with fp32 statistics."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 2 == 0 and _lib.available():
        return _RmsNormFn.apply(x, weight, eps)
    normed = F.rms_norm(x.float(), (x.size(-1),), eps=eps)
    return (normed * weight.float()).to(x.dtype) if x.dtype != torch.float32 else normed * weight


# ---------------------------------------------------------------------------
# linear + CE
# ---------------------------------------------------------------------------
class _LinearCeFn(torch.autograd.Function):
    """(x [R,D], weight [V,D], targets [R], row_weight or None) -> (loss_sum_weighted, per-row CE)."""

    @staticmethod
    def forward(ctx, x, weight, targets, row_weight):
        loss_rows, lse = LH.lm_head_lse(x, None, weight, targets)
        ctx.save_for_backward(x, weight, targets, lse, row_weight if row_weight is not None
                              else torch.empty(0, device=x.device))
        ctx.has_w = row_weight is not None
        total = (loss_rows * row_weight.float()).sum() if row_weight is not None else loss_rows.sum()
        ctx.mark_non_differentiable(loss_rows)
        return total, loss_rows

    @staticmethod
    def backward(ctx, gtotal, _gl):
        x, weight, targets, lse, rw = ctx.saved_tensors
        roww = rw.float().contiguous() if ctx.has_w else None
        _, _, dX, part = LH.lm_head_train(x, None, weight, targets, gscale=1.0, rowweight=roww, lse=lse)
        dW, _ = splitk_reduce(part)
        return dX * gtotal.to(dX.dtype), (dW * gtotal).to(weight.dtype), None, None


def _linear_ce(x, weight, targets, row_weight=None):
    """Returns (weighted sum of per-row CE, per-row CE)."""
    if LH.kernel_supported(x, weight) and _lib.available():
        return _LinearCeFn.apply(x.contiguous(), weight.contiguous(), targets.reshape(-1), row_weight)
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        # the kernels' own dtype with a shape they do not take: refuse, like the reference's dispatcher;
        # other dtypes (fp32 debugging runs) and CPU tensors are outside the kernels' domain
        raise TypeError(f"fused linear+CE: no kernel takes x {tuple(x.shape)} with weight {tuple(weight.shape)} "
                        "(model dim a multiple of 8 and at most 512, vocabulary a multiple of 8)")
    logits = F.linear(x, weight).float()
    rows = F.cross_entropy(logits, targets.reshape(-1).long(), reduction="none")
    total = (rows * row_weight.float()).sum() if row_weight is not None else rows.sum()
    return total, rows.detach()


def _reduce(total, n_rows: int, reduction: str):
    if reduction == "mean":
        return total / n_rows
    if reduction == "sum":
        return total
    raise ValueError(f"reduction must be 'mean' or 'sum', got {reduction!r}")


def fused_linear_cross_entropy(x, weight, targets, *, reduction: str = "mean", tile_size: int = 1024,
                               backend: str = "auto"):
    _check_backend(backend)
    total, _ = _linear_ce(x.reshape(-1, x.shape[-1]), weight, targets)
    return _reduce(total, targets.numel(), reduction)


def fused_linear_cross_entropy_with_ce(x, weight, targets, *, reduction: str = "mean",
                                       tile_size: int = 1024, backend: str = "auto"):
    _check_backend(backend)
    total, rows = _linear_ce(x.reshape(-1, x.shape[-1]), weight, targets)
    return _reduce(total, targets.numel(), reduction), rows


def fused_linear_cross_entropy_weighted(x, weight, targets, row_weight, *, normalizer=None,
                                        tile_size: int = 1024, backend: str = "auto"):
    """``sum_r w_r * CE_r / max(normalizer, 1)`` (normalizer defaults to ``sum w``)."""
    _check_backend(backend)
    total, rows = _linear_ce(x.reshape(-1, x.shape[-1]), weight, targets, row_weight.reshape(-1))
    norm = row_weight.float().sum() if normalizer is None else torch.as_tensor(
        normalizer, dtype=torch.float32, device=x.device)
    return total / norm.clamp_min(1.0), rows


def fused_rms_linear_cross_entropy(x, norm_weight, linear_weight, targets, *, eps: float = 1e-6,
                                   reduction: str = "mean", tile_size: int = 1024,
                                   backend: str = "auto"):
    return fused_linear_cross_entropy(fused_rms_norm(x, norm_weight, eps), linear_weight, targets,
                                      reduction=reduction, tile_size=tile_size, backend=backend)


def fused_rms_linear_cross_entropy_with_ce(x, norm_weight, linear_weight, targets, *, eps: float = 1e-6,
                                           reduction: str = "mean", tile_size: int = 1024,
                                           backend: str = "auto"):
    return fused_linear_cross_entropy_with_ce(fused_rms_norm(x, norm_weight, eps), linear_weight,
                                              targets, reduction=reduction, tile_size=tile_size,
                                              backend=backend)


@torch.no_grad()
def fused_lm_head_forward_with_ce_entropy(x, weight, target, *, tile_size: int = 8192):
    """Forward only: ``(mean loss, lse, per-token CE, per-token entropy)``."""
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    # the entropy by-product exists in the single-kernel head (model dim 256) only; other dims take the
    # PyTorch statement in bounded row chunks, which this forward-only diagnostic asks for explicitly
    rows, lse, ent = LH.lm_head_lse(x2, None, weight.contiguous(), target.reshape(-1), want_entropy=True,
                                    allow_materialized=True)
    return rows.mean(), lse, rows, ent
