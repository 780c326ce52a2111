"""Diagonal-SSM scan ops.

Two families:

* the *fused* scan used by the trunk (``scan_fused_fwd`` / ``scan_fused_bwd``):
  consumes the packed raw projection ``P = (select | candidate | gate | delta)``
  and never materialises decay / update / gate;
* ``ssm_scan(decay, update)``: the reference's public op
  (src/chaoscontrol/kernels/_ssm_scan/__init__.py:309-338), kept for API parity,
  extended with an optional initial state.

Each has a plain PyTorch fp32 statement used on CPU and as the test oracle.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

__all__ = [
    "scan_fused_reference", "scan_fused_fwd", "scan_fused_bwd", "ssm_scan", "diag_recurrence_reference",
    "diag_recurrence_chunked",
]


# ---------------------------------------------------------------------------
# references
# ---------------------------------------------------------------------------
def diag_recurrence_reference(decay: torch.Tensor, update: torch.Tensor,
                              h0: Optional[torch.Tensor] = None) -> torch.Tensor:
    """state[t] = decay[t] * state[t-1] + update[t]; serial fp32 loop (oracle)."""
    B, T, D = update.shape
    s = torch.zeros(B, D, dtype=torch.float32, device=update.device) if h0 is None else h0.float()
    out = []
    dec = decay.float()
    upd = update.float()
    for t in range(T):
        s = dec[:, t] * s + upd[:, t]
        out.append(s)
    return torch.stack(out, dim=1)


def diag_recurrence_chunked(decay: torch.Tensor, update: torch.Tensor, chunk: int = 32,
                            h0: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Chunked parallel form of the same recurrence (fp64 inside a chunk), the vectorised CPU
    path (cf. src/chaoscontrol/core.py:46-119).

    Inside a chunk ``h[t] = sum_{j<=t} exp(L[t] - L[j]) u[j] + exp(L[t]) carry`` with ``L`` the
    running sum of ``log decay``.  Every exponent is <= 0, so nothing overflows or divides by an
    underflowed product however small the decays get (a cumulative-product form ``cp * cumsum(u /
    cp)`` turns into 0 * inf once a chunk's product underflows, which strongly decaying channels
    reach after a few optimizer steps)."""
    B, T, D = update.shape
    dt = torch.float64
    dec = decay.to(dt)
    upd = update.to(dt)
    carry = torch.zeros(B, D, dtype=dt, device=update.device) if h0 is None else h0.to(dt)
    outs = []
    for t0 in range(0, T, chunk):
        d = dec[:, t0:t0 + chunk]
        u = upd[:, t0:t0 + chunk]
        c = d.shape[1]
        logp = torch.cumsum(torch.log(d.clamp_min(1e-300)), dim=1)           # [B, c, D]
        diff = logp.unsqueeze(2) - logp.unsqueeze(1)                          # [B, t, j, D] = L[t] - L[j]
        lower = torch.ones(c, c, dtype=torch.bool, device=update.device).tril()
        w = torch.exp(diff.masked_fill(~lower[None, :, :, None], float("-inf")))
        h = torch.einsum("btjd,bjd->btd", w, u) + torch.exp(logp) * carry.unsqueeze(1)
        outs.append(h)
        carry = h[:, -1]
    return torch.cat(outs, dim=1).to(torch.float32)


def scan_fused_reference(P: torch.Tensor, log_a: torch.Tensor, h0: Optional[torch.Tensor],
                         B: int, T: int, D: int):
    """fp32 statement of the fused scan.  ``P`` is ``[B*T, 4D]``.

    Returns ``(y, h, hT)`` as fp32 ``[B*T, D]``, ``[B*T, D]``, ``[B, D]``.
    Differentiable, so autograd through it is the oracle for the backward kernel.
    """
    Pf = P.float().view(B, T, 4 * D)
    s_raw, c_raw, g_raw, d_raw = Pf.split(D, dim=-1)
    a = torch.sigmoid(log_a.float())
    a = a[None, None, :] if a.dim() == 1 else a[:, None, :]      # shared, or one decay vector per batch row
    delta = F.softplus(d_raw).clamp_min(1e-4)
    decay = torch.exp(-delta * a)
    update = torch.sigmoid(s_raw) * torch.tanh(c_raw)
    s = torch.zeros(B, D, dtype=torch.float32, device=P.device) if h0 is None else h0.float()
    hs = []
    for t in range(T):
        s = decay[:, t] * s + update[:, t]
        hs.append(s)
    h = torch.stack(hs, dim=1)
    y = torch.sigmoid(g_raw) * h
    return y.reshape(B * T, D), h.reshape(B * T, D), s


# ---------------------------------------------------------------------------
# fused CUDA scan
# ---------------------------------------------------------------------------
def _log_a_batch_stride(log_a: torch.Tensor, B: int, D: int) -> int:
    if log_a.dim() == 1:
        assert log_a.numel() == D and log_a.is_contiguous()
        return 0
    assert log_a.shape == (B, D) and log_a.stride(1) == 1, "per-row log_a must be [B, D]"
    return int(log_a.stride(0))


def scan_fused_fwd(P: torch.Tensor, log_a_f32: torch.Tensor, h0: Optional[torch.Tensor], B: int,
                   T: int, D: int, *, save_h: bool = True, want_hT: bool = True):
    """Launch ``scan_fwd_kernel``.  ``P`` bf16 ``[B*T, >=4D]`` (row stride free),
    ``log_a_f32`` fp32 ``[D]`` (shared) or ``[B, D]`` (one decay vector per batch
    row), ``h0`` fp32 ``[B, D]`` or None."""
    assert P.dtype == torch.bfloat16 and log_a_f32.dtype == torch.float32
    la_bs = _log_a_batch_stride(log_a_f32, B, D)
    y = torch.empty(B * T, D, dtype=torch.bfloat16, device=P.device)
    h = torch.empty(B * T, D, dtype=torch.bfloat16, device=P.device) if save_h else None
    hT = torch.empty(B, D, dtype=torch.float32, device=P.device) if want_hT else None
    if h0 is not None:
        assert h0.dtype == torch.float32 and h0.is_contiguous()
    _lib.check(_lib.lib().ccb_scan_fwd(P.data_ptr(), P.stride(0), log_a_f32.data_ptr(), _lib.ptr(h0),
                                       y.data_ptr(), _lib.ptr(h), _lib.ptr(hT), B, T, D, la_bs,
                                       _lib.stream_ptr()), "scan_fwd")
    return y, h, hT


def scan_fused_bwd(P: torch.Tensor, log_a_f32: torch.Tensor, h0: Optional[torch.Tensor],
                   h: torch.Tensor, dy: torch.Tensor, dhT: Optional[torch.Tensor],
                   rowss: Optional[torch.Tensor], inv_dim: float, eps: float, B: int, T: int, D: int,
                   *, want_dh0: bool = False, dP: Optional[torch.Tensor] = None):
    """Launch ``scan_bwd_kernel``.  Returns ``(dP bf16 [B*T,4D], dlog_a fp32, dh0)``.

    When ``rowss`` is given, ``dP`` comes out pre-multiplied by the producing
    RMSNorm's row scale so the following GEMMs need no separate pass.  With a
    shared ``log_a`` (``[D]``) its gradient is summed over the batch; with one
    decay vector per batch row (``[B, D]``) the gradient keeps that shape.
    """
    la_bs = _log_a_batch_stride(log_a_f32, B, D)
    if dP is None:
        dP = torch.empty(B * T, 4 * D, dtype=torch.bfloat16, device=P.device)
    part = torch.empty(B, D, dtype=torch.float32, device=P.device)
    dh0 = torch.empty(B, D, dtype=torch.float32, device=P.device) if want_dh0 else None
    assert dy.dtype == torch.bfloat16 and dy.is_contiguous() and h.is_contiguous()
    _lib.check(_lib.lib().ccb_scan_bwd(
        P.data_ptr(), P.stride(0), log_a_f32.data_ptr(), _lib.ptr(h0), h.data_ptr(), dy.data_ptr(),
        _lib.ptr(dhT), _lib.ptr(rowss), inv_dim, eps, dP.data_ptr(), dP.stride(0), part.data_ptr(),
        _lib.ptr(dh0), B, T, D, la_bs, _lib.stream_ptr()), "scan_bwd")
    if log_a_f32.dim() == 2:
        return dP, part, dh0
    # deterministic second stage of the d log_a reduction
    dloga = torch.empty(D, dtype=torch.float32, device=P.device)
    _lib.check(_lib.lib().ccb_colsum(part.data_ptr(), B, D, dloga.data_ptr(), 0, _lib.stream_ptr()),
               "colsum")
    return dP, dloga, dh0


# ---------------------------------------------------------------------------
# public ssm_scan(decay, update) with autograd
# ---------------------------------------------------------------------------
_DT_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
#: (decay, update) dtype pairs the native scan takes as they are -- the reference op's whitelist
#: (src/chaoscontrol/kernels/_ssm_scan/__init__.py:104-113)
KERNEL_DTYPE_COMBOS = frozenset({
    (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float16), (torch.float16, torch.float16),
    (torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.float32, torch.float16),
})


class _SsmScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, decay, update, h0):
        B, T, D = update.shape
        states = torch.empty(B, T, D, dtype=torch.float32, device=update.device)
        h0c = None if h0 is None else h0.float().contiguous()
        _lib.check(_lib.lib().ccb_plain_scan_fwd(decay.data_ptr(), _DT_CODE[decay.dtype], update.data_ptr(),
                                                 _DT_CODE[update.dtype], _lib.ptr(h0c), states.data_ptr(),
                                                 B, T, D, _lib.stream_ptr()), "plain_scan_fwd")
        ctx.save_for_backward(decay, states, h0c if h0c is not None else torch.empty(0))
        ctx.has_h0 = h0 is not None
        ctx.update_dtype = update.dtype
        return states.to(update.dtype)

    @staticmethod
    def backward(ctx, g):
        decay, states, h0c = ctx.saved_tensors
        B, T, D = states.shape
        gs = g.to(ctx.update_dtype).contiguous()
        gdec = torch.empty_like(decay)                     # decay dtype
        gupd = torch.empty_like(gs)                        # update dtype
        gh0 = torch.empty(B, D, dtype=torch.float32, device=g.device) if ctx.has_h0 else None
        _lib.check(_lib.lib().ccb_plain_scan_bwd(decay.data_ptr(), _DT_CODE[decay.dtype], states.data_ptr(),
                                                 h0c.data_ptr() if ctx.has_h0 else None, gs.data_ptr(),
                                                 _DT_CODE[ctx.update_dtype], gdec.data_ptr(), gupd.data_ptr(),
                                                 _lib.ptr(gh0), B, T, D, _lib.stream_ptr()), "plain_scan_bwd")
        return gdec, gupd, gh0


def ssm_scan(decay: torch.Tensor, update: torch.Tensor,
             initial_state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``states[t] = decay[t] * states[t-1] + update[t]`` over ``(B, T, D)``.

    CUDA tensors run the native kernel (fp32 accumulator, result in
    ``update.dtype``); CPU tensors run the chunked fp64 form.  Non-contiguous
    inputs are rejected like the reference op does.
    """
    if decay.shape != update.shape or update.dim() != 3:
        raise ValueError("ssm_scan expects decay and update of identical (B, T, D) shape")
    if not decay.is_contiguous() or not update.is_contiguous():
        raise ValueError("ssm_scan requires contiguous inputs")
    if update.is_cuda:
        if (decay.dtype, update.dtype) not in KERNEL_DTYPE_COMBOS:
            raise TypeError(f"ssm_scan: (decay, update) dtypes ({decay.dtype}, {update.dtype}) are not among the "
                            f"pairs the native scan takes: {sorted(map(str, KERNEL_DTYPE_COMBOS))}; cast explicitly")
        return _SsmScanFn.apply(decay, update, initial_state)
    return diag_recurrence_chunked(decay, update, h0=initial_state).to(update.dtype)
