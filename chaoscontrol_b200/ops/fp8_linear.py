"""fp8 linear layer with delayed per-tensor scaling on tcgen05 ``kind::f8f6f4``.

Same module contract as the reference's ``FusedFP8Linear``
(src/chaoscontrol/kernels/fp8_linear.py:171-432): master weight in bf16,
activations and weights quantised to e4m3, output gradients to e5m2, scales
READ from ``x_scale`` / ``w_scale`` / ``gy_scale`` buffers that
``flush_amax_history()`` refreshes once per optimizer step from a 16-entry amax
history; every cast folds its observed ``max|t|`` into a ``*_amax_pending``
buffer with one integer ``atomicMax`` and never synchronises with the host.
Before the first flush every scale is 1 (casts saturate at the format's range).

GEMM plan (all operands K-major, so no tensor-core transpose modes are needed):

* forward   ``y  = x8 @ w8.T``             ``x8 [M,K]``, ``w8 [N,K]``
* dgrad     ``dx = gy8 @ w8t.T``           ``gy8 [M,N]``, ``w8t [K,N]`` (transposing cast of ``W``)
* wgrad     ``dW = gy8t @ x8t.T``          ``gy8t [N,M]``, ``x8t [K,M]`` (transposing casts; the ``gy``
                                           one also emits the bias gradient column sum)

``x8t`` is produced in the forward pass while ``x`` is hot and saved instead of ``x``.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.nn as nn

from . import _lib
from .gemm import gemm_fp8

__all__ = ["FusedFP8Linear", "fused_fp8_flush_all", "fp8_cast", "fp8_cast_transpose", "fp8_flush_amax",
           "fp8_linear_reference", "E4M3_MAX", "E5M2_MAX"]

E4M3_MAX = 448.0
E5M2_MAX = 57344.0
_DEFAULT_AMAX_HISTORY_LEN = 16
_FMT = {torch.float8_e4m3fn: 1, torch.float8_e5m2: 2}
_MAXREP = {torch.float8_e4m3fn: E4M3_MAX, torch.float8_e5m2: E5M2_MAX}


def _pad16(n: int) -> int:
    return (n + 15) // 16 * 16


def fp8_cast(x: torch.Tensor, scale: torch.Tensor, pending: Optional[torch.Tensor], dtype: torch.dtype) -> torch.Tensor:
    """``(x / scale)`` saturated to ``dtype``; ``pending = max(pending, max|x|)``."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        _lib.check(_lib.lib().ccb_fp8_cast_amax(x.data_ptr(), out.data_ptr(), scale.data_ptr(), _lib.ptr(pending),
                                                x.numel(), _FMT[dtype], _lib.stream_ptr()), "fp8_cast_amax")
        return out
    if x.is_cuda:
        return fp8_cast(x.to(torch.bfloat16).contiguous(), scale, pending, dtype)
    xf = x.float()
    if pending is not None:
        pending.copy_(torch.maximum(pending, xf.abs().max().reshape(1)))
    m = _MAXREP[dtype]
    return (xf / scale.float()).clamp(-m, m).to(dtype)


def fp8_cast_transpose(x: torch.Tensor, scale: torch.Tensor, pending: Optional[torch.Tensor], dtype: torch.dtype,
                       colsum: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Transposed cast of ``x [R, C]``: returns a ``[C, R]`` view whose row stride is padded
    to 16 bytes.  ``colsum [C]`` (fp32), when given, accumulates ``x.sum(0)``."""
    R, Cc = x.shape
    if x.is_cuda:
        if x.dtype != torch.bfloat16 or x.stride(1) != 1:
            x = x.to(torch.bfloat16).contiguous()
        ldo = _pad16(R)
        buf = torch.empty((Cc, ldo), dtype=dtype, device=x.device)
        if ldo != R:
            buf.view(torch.uint8)[:, R:].zero_()          # padding feeds the GEMM's K tail
        _lib.check(_lib.lib().ccb_fp8_cast_transpose_amax(
            x.data_ptr(), buf.data_ptr(), scale.data_ptr(), _lib.ptr(pending), _lib.ptr(colsum), R, Cc,
            x.stride(0), ldo, _FMT[dtype], _lib.stream_ptr()), "fp8_cast_transpose_amax")
        return buf[:, :R]
    xf = x.float()
    if pending is not None:
        pending.copy_(torch.maximum(pending, xf.abs().max().reshape(1)))
    if colsum is not None:
        colsum.add_(xf.sum(0))
    m = _MAXREP[dtype]
    return (xf.T / scale.float()).clamp(-m, m).contiguous().to(dtype)


def fp8_flush_amax(history: torch.Tensor, pending: torch.Tensor, scale: Optional[torch.Tensor], max_rep: float) -> None:
    """Roll ``history`` left, append ``pending``, ``scale = max(history) / max_rep``
    (1 while the history is empty), zero ``pending``.  ``scale=None`` only rolls."""
    if history.is_cuda:
        _lib.check(_lib.lib().ccb_fp8_flush_amax(history.data_ptr(), history.numel(), pending.data_ptr(),
                                                 _lib.ptr(scale), float(max_rep), _lib.stream_ptr()), "fp8_flush_amax")
        return
    with torch.no_grad():
        history.copy_(torch.roll(history, -1))
        history[-1] = pending.squeeze()
        if scale is not None:
            m = history.max()
            scale.copy_(torch.where(m > 0, m / max_rep, torch.ones_like(m)).reshape(1))
        pending.zero_()


def fp8_linear_reference(x, weight, bias, x_scale, w_scale):
    """fp32 oracle of the forward pass: quantise, dequantise, matmul."""
    xq = (x.float() / x_scale.float()).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float() * x_scale.float()
    wq = (weight.float() / w_scale.float()).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float() * w_scale.float()
    y = xq @ wq.T
    return y if bias is None else y + bias.float()


def _k_view(t8: torch.Tensor) -> torch.Tensor:
    """K-major operand whose row stride obeys the 16-byte rule (copy only if it does not)."""
    if t8.stride(-1) == 1 and t8.stride(0) % 16 == 0:
        return t8
    R, K = t8.shape
    buf = torch.zeros((R, _pad16(K)), dtype=torch.uint8, device=t8.device).view(t8.dtype)
    buf[:, :K].copy_(t8)
    return buf[:, :K]


class _FusedFP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x, weight, bias, x_scale, w_scale, gy_scale, x_pending, w_pending, gy_pending, gx_pending):
        e4 = torch.float8_e4m3fn
        x8 = _k_view(fp8_cast(x, x_scale, x_pending, e4))
        w8 = _k_view(fp8_cast(weight, w_scale, w_pending, e4))
        y = gemm_fp8(x8, w8, scale_a=x_scale, scale_b=w_scale, bias=bias, out_dtype=torch.bfloat16
                     if x.is_cuda else x.dtype)
        need_w = weight.requires_grad
        x8t = fp8_cast_transpose(x, x_scale, None, e4) if need_w else None
        ctx.save_for_backward(x8t, weight, x_scale, w_scale, gy_scale, gy_pending, gx_pending)
        ctx.has_bias = bias is not None
        ctx.in_dtype = x.dtype
        return y

    @staticmethod
    def backward(ctx: Any, gy):
        x8t, weight, x_scale, w_scale, gy_scale, gy_pending, gx_pending = ctx.saved_tensors
        e4, e5 = torch.float8_e4m3fn, torch.float8_e5m2
        gy = gy.contiguous()
        odt = torch.bfloat16 if gy.is_cuda else ctx.in_dtype
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gy8 = _k_view(fp8_cast(gy, gy_scale, gy_pending, e5))
            w8t = fp8_cast_transpose(weight, w_scale, None, e4)
            gx = gemm_fp8(gy8, w8t, scale_a=gy_scale, scale_b=w_scale, out_dtype=odt)
            with torch.no_grad():                         # diagnostic only: never feeds a scale
                gx_pending.copy_(torch.maximum(gx_pending, gx.detach().abs().max().float().reshape(1)))
        if ctx.needs_input_grad[1]:
            colsum = torch.zeros(gy.shape[1], dtype=torch.float32, device=gy.device) if ctx.has_bias else None
            pend = None if ctx.needs_input_grad[0] else gy_pending     # count gy's amax once
            gy8t = fp8_cast_transpose(gy, gy_scale, pend, e5, colsum=colsum)
            gw = gemm_fp8(gy8t, x8t, scale_a=gy_scale, scale_b=x_scale, out_dtype=odt).to(weight.dtype)
            if ctx.has_bias:
                gb = colsum.to(weight.dtype)
        elif ctx.has_bias:
            gb = gy.float().sum(0).to(weight.dtype)
        return gx, gw, gb, None, None, None, None, None, None, None


class FusedFP8Linear(nn.Module):
    """Drop-in ``nn.Linear`` whose three GEMMs run in 8-bit floats.

    Call ``flush_amax_history()`` (or ``fused_fp8_flush_all(model)``) once per
    optimizer step, after ``optimizer.step()``; skipping it keeps the scales stale
    but the maths valid.  All scaling state is persistent (checkpointed).
    """

    def __init__(self, in_features: int, out_features: int, *, bias: bool = True, device=None,
                 dtype: torch.dtype = torch.bfloat16, amax_history_len: int = _DEFAULT_AMAX_HISTORY_LEN) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty((out_features, in_features), device=device, dtype=dtype))
        if bias:
            self.bias = nn.Parameter(torch.zeros((out_features,), device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        kw = dict(dtype=torch.float32, device=device)
        for t in ("x", "w", "gy", "gx"):
            self.register_buffer(f"{t}_amax_history", torch.zeros(amax_history_len, **kw), persistent=True)
            self.register_buffer(f"{t}_amax_pending", torch.zeros(1, **kw), persistent=True)
        for t in ("x", "w", "gy"):
            self.register_buffer(f"{t}_scale", torch.ones(1, **kw), persistent=True)

    @classmethod
    def from_nn_linear(cls, m: nn.Linear) -> "FusedFP8Linear":
        out = cls(m.in_features, m.out_features, bias=m.bias is not None, device=m.weight.device,
                  dtype=m.weight.dtype)
        with torch.no_grad():
            out.weight.copy_(m.weight)
            if m.bias is not None:
                out.bias.copy_(m.bias)
        return out

    def flush_amax_history(self) -> None:
        fp8_flush_amax(self.x_amax_history, self.x_amax_pending, self.x_scale, E4M3_MAX)
        fp8_flush_amax(self.w_amax_history, self.w_amax_pending, self.w_scale, E4M3_MAX)
        fp8_flush_amax(self.gy_amax_history, self.gy_amax_pending, self.gy_scale, E5M2_MAX)
        fp8_flush_amax(self.gx_amax_history, self.gx_amax_pending, None, 1.0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        xf = x.reshape(-1, self.in_features)
        if xf.dtype != self.weight.dtype:
            xf = xf.to(self.weight.dtype)
        y = _FusedFP8LinearFn.apply(xf, self.weight, self.bias, self.x_scale, self.w_scale, self.gy_scale,
                                    self.x_amax_pending, self.w_amax_pending, self.gy_amax_pending,
                                    self.gx_amax_pending)
        return y.reshape(*lead, self.out_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


def fused_fp8_flush_all(model: nn.Module) -> int:
    """Flushes every ``FusedFP8Linear`` under ``model``; returns how many there were."""
    n = 0
    for m in model.modules():
        if isinstance(m, FusedFP8Linear):
            m.flush_amax_history()
            n += 1
    return n
