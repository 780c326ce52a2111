"""Hand-scheduled forward and backward of the diagonal-SSM trunk.

One layer is four GEMMs and one scan kernel in each direction; every
elementwise op of the block (both RMSNorms, the gate nonlinearities, SiLU, the
two residual adds) lives in a GEMM epilogue or in the scan kernel, so no
``[rows, dim]`` tensor is ever touched by a standalone elementwise pass:

forward (x: residual stream, ss = row sum of squares of x)::

    P   = rs1 * (x  @ Wp'^T)          Wp' = [select;in;gate;delta] * w_input_norm   (EPI_ROWSCALE)
    y,h = scan(P, log_a, h0)
    x2  = x  + y @ Wo^T , ss2         (EPI_RESID_SS)
    u,f = rs2 * (x2 @ Wfc'^T), silu   Wfc' = fc * w_ff_norm                         (EPI_ROWSCALE_SILU)
    x3  = x2 + f @ Wproj^T , ss3      (EPI_RESID_SS)

The RMSNorm weight is folded into the following linear's weight (tiny, once
per step) and the row scale ``rs = rsqrt(ss/D + eps)`` is applied to the GEMM
output, which is algebraically the reference block
(src/chaoscontrol/model.py:111-140, core.py:492-507, core.py:322-335).

backward mirrors it with the RMSNorm backward fused into the input-gradient
GEMM epilogue (EPI_RMSBWD) and weight gradients from split-K MN-major GEMMs.
Everything here also runs on CPU tensors (fp32) through the op stand-ins, which
is how the algebra is tested against autograd of the plain module.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _lib
from .gemm import (EPI_DSILU, EPI_RESID_SS, EPI_RMSBWD, EPI_ROWSCALE, EPI_ROWSCALE_SILU,
                   EPI_STORE, gemm, pick_splits)
from .scan import scan_fused_bwd, scan_fused_fwd, scan_fused_reference

EPS = 1e-6


# ---------------------------------------------------------------------------
# small op wrappers with CPU stand-ins
# ---------------------------------------------------------------------------
def fold_colscale(W: torch.Tensor, wn: torch.Tensor) -> torch.Tensor:
    """``W * wn[None, :]`` in the activation dtype (RMSNorm weight folded into W)."""
    if W.is_cuda and W.dtype == torch.bfloat16 and wn.dtype == torch.bfloat16 and W.is_contiguous():
        out = torch.empty_like(W)
        _lib.check(_lib.lib().ccb_fold_colscale(W.data_ptr(), wn.data_ptr(), out.data_ptr(),
                                                W.shape[0], W.shape[1], _lib.stream_ptr()), "fold")
        return out
    return (W.float() * wn.float()[None, :]).to(W.dtype)


def embed_fwd(tokens: torch.Tensor, E: torch.Tensor):
    """Gather rows of ``E`` and their sums of squares.  Returns ``(x [R,D], ss [R])``."""
    flat = tokens.reshape(-1)
    R, D = flat.numel(), E.shape[1]
    if E.is_cuda:
        assert E.dtype == torch.bfloat16 and E.is_contiguous()
        if flat.dtype not in (torch.int32, torch.int64):
            flat = flat.long()
        flat = flat.contiguous()
        x = torch.empty(R, D, dtype=E.dtype, device=E.device)
        ss = torch.empty(R, dtype=torch.float32, device=E.device)
        _lib.check(_lib.lib().ccb_embed_fwd(flat.data_ptr(), int(flat.dtype == torch.int64),
                                            E.data_ptr(), x.data_ptr(), ss.data_ptr(), R, D,
                                            E.shape[0], _lib.stream_ptr()), "embed_fwd")
        return x, ss
    x = E[flat.long()]
    return x, (x.float() ** 2).sum(-1)


def embed_bwd(tokens: torch.Tensor, dx: torch.Tensor, V: int,
              sort_cache: Optional[tuple] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 ``[V, D]`` gradient of the embedding table (sum of the ``dx`` rows of each token).

    On the GPU the rows are added in a fixed order derived from the stably sorted token array, so
    the same batch gives the same bits on every run and on every replica."""
    flat = tokens.reshape(-1).long()
    D = dx.shape[1]
    if out is not None:
        dE = out.zero_()
    else:
        dE = torch.zeros(V, D, dtype=torch.float32, device=dx.device)
    if dx.is_cuda and D in (256, 512, 1024):
        if sort_cache is None:
            sort_cache = torch.sort(flat, stable=True)
        st, perm = sort_cache
        L = _lib.lib()
        slots = torch.empty(int(L.ccb_embed_bwd_slots(flat.numel(), D, V)), dtype=torch.float32,
                            device=dx.device)
        _lib.check(L.ccb_embed_bwd_sorted(st.data_ptr(), perm.data_ptr(), dx.data_ptr(), dE.data_ptr(),
                                          slots.data_ptr(), flat.numel(), D, V, _lib.stream_ptr()),
                   "embed_bwd")
        return dE
    dE.index_add_(0, flat, dx.float())
    return dE


def splitk_reduce(part: torch.Tensor, *, colscale: Optional[torch.Tensor] = None,
                  W: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  dcol_out: Optional[torch.Tensor] = None):
    """Sum split-K partials ``[S, N, K]`` (or ``[N, K]``).

    Returns ``(dW [N,K] fp32, dcol [K] fp32 or None)`` with
    ``dW = colscale * sum`` and ``dcol = sum_n sum[n,k] * W[n,k]`` -- the
    gradients of ``W`` and of the RMSNorm weight folded into it.
    """
    if part.dim() == 2:
        part = part.unsqueeze(0)
    S, N, K = part.shape
    if part.is_cuda and (colscale is None or colscale.dtype == torch.bfloat16) and (
            W is None or (W.dtype == torch.bfloat16 and W.is_contiguous())):
        if out is None:
            out = torch.empty(N, K, dtype=torch.float32, device=part.device)
        assert out.dtype == torch.float32 and out.is_contiguous()
        nb = (N + 7) // 8
        colpart = torch.empty(nb, K, dtype=torch.float32, device=part.device) if W is not None else None
        dcol = None
        if W is not None:
            dcol = dcol_out if dcol_out is not None else torch.empty(K, dtype=torch.float32,
                                                                     device=part.device)
        _lib.check(_lib.lib().ccb_splitk_reduce(part.data_ptr(), S, part.stride(0), N, K,
                                                _lib.ptr(colscale), _lib.ptr(W), out.data_ptr(), 0,
                                                _lib.ptr(colpart), _lib.ptr(dcol), 0,
                                                _lib.stream_ptr()), "splitk_reduce")
        return out, dcol
    s = part.float().sum(0)
    dcol = (s * W.float()).sum(0) if W is not None else None
    if colscale is not None:
        s = s * colscale.float()[None, :]
    if out is not None:
        out.copy_(s)
        s = out
    if dcol is not None and dcol_out is not None:
        dcol_out.copy_(dcol)
        dcol = dcol_out
    return s, dcol


def _wgrad(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Split-K partials of ``dy^T @ x`` (``[S, N, K]`` fp32)."""
    M, N = dy.shape
    K = x.shape[1]
    S = pick_splits(N, K, M) if dy.is_cuda else 1
    out = gemm(dy, x, a_mn=True, b_mn=True, splits=S, out_dtype=torch.float32)
    return out if out.dim() == 3 else out.unsqueeze(0)


# ---------------------------------------------------------------------------
# per-layer weights as the kernels want them
# ---------------------------------------------------------------------------
@dataclass
class LayerWeights:
    Wp: torch.Tensor        # [4D, D]  select | in | gate | delta  (unscaled)
    Wo: torch.Tensor        # [D, D]
    Wfc: torch.Tensor       # [F, D]
    Wproj: torch.Tensor     # [D, F]
    wn1: torch.Tensor       # [D] input_norm.weight
    wn2: torch.Tensor       # [D] ff_norm.weight
    log_a: torch.Tensor     # [D]
    # derived per step
    Wp_f: torch.Tensor = field(default=None)     # Wp * wn1
    Wfc_f: torch.Tensor = field(default=None)    # Wfc * wn2
    log_a32: torch.Tensor = field(default=None)

    def prepare(self) -> "LayerWeights":
        self.Wp_f = fold_colscale(self.Wp, self.wn1)
        self.Wfc_f = fold_colscale(self.Wfc, self.wn2)
        self.log_a32 = self.log_a.float().contiguous()
        return self


@dataclass
class LayerCtx:
    x: torch.Tensor
    ss1: torch.Tensor
    P: torch.Tensor
    h: torch.Tensor
    y: torch.Tensor
    x2: torch.Tensor
    ss2: torch.Tensor
    u: torch.Tensor
    f: torch.Tensor
    h0: Optional[torch.Tensor]


@dataclass
class LayerGrads:
    dWp: torch.Tensor       # [4D, D] fp32
    dWo: torch.Tensor
    dWfc: torch.Tensor
    dWproj: torch.Tensor
    dwn1: torch.Tensor
    dwn2: torch.Tensor
    dlog_a: torch.Tensor
    dh0: Optional[torch.Tensor] = None


def _scan_fwd(P, log_a32, h0, B, T, D, save_h):
    if P.is_cuda:
        return scan_fused_fwd(P, log_a32, h0, B, T, D, save_h=save_h)
    y, h, hT = scan_fused_reference(P, log_a32, h0, B, T, D)
    return y.to(P.dtype), h.to(P.dtype), hT


def _scan_bwd(P, log_a32, h0, h, dy, dhT, rowss, inv_dim, eps, B, T, D, want_dh0):
    if P.is_cuda:
        return scan_fused_bwd(P, log_a32, h0, h, dy, dhT, rowss, inv_dim, eps, B, T, D,
                              want_dh0=want_dh0)
    with torch.enable_grad():
        Pr = P.detach().float().requires_grad_(True)
        la = log_a32.detach().clone().requires_grad_(True)
        h0r = h0.detach().clone().requires_grad_(True) if h0 is not None else None
        y, _, hT = scan_fused_reference(Pr, la, h0r, B, T, D)
        obj = (y * dy.float()).sum()
        if dhT is not None:
            obj = obj + (hT * dhT.float()).sum()
        ins = [Pr, la] + ([h0r] if (h0r is not None and want_dh0) else [])
        grads = torch.autograd.grad(obj, ins)
    dP = grads[0]
    if rowss is not None:
        dP = dP * torch.rsqrt(rowss.float() * inv_dim + eps)[:, None]
    return dP.to(P.dtype), grads[1], (grads[2] if len(grads) > 2 else None)


def layer_forward(x: torch.Tensor, ss1: torch.Tensor, w: LayerWeights, B: int, T: int,
                  h0: Optional[torch.Tensor] = None, *, save: bool = True):
    """One block.  Returns ``(x3, ss3, hT, ctx)``; ``ctx`` is None when ``save`` is False."""
    R, D = x.shape
    F_ = w.Wfc.shape[0]
    inv_d = 1.0 / D
    P = gemm(x, w.Wp_f, epi=EPI_ROWSCALE, rowss=ss1, inv_dim=inv_d, eps=EPS)
    y, h, hT = _scan_fwd(P, w.log_a32, h0, B, T, D, save)
    ss2 = torch.empty(R, dtype=torch.float32, device=x.device)
    x2 = gemm(y, w.Wo, epi=EPI_RESID_SS, r1=x, ss_out=ss2)
    f = torch.empty(R, F_, dtype=x.dtype, device=x.device)
    u = gemm(x2, w.Wfc_f, epi=EPI_ROWSCALE_SILU, rowss=ss2, inv_dim=inv_d, eps=EPS, c2=f)
    ss3 = torch.empty(R, dtype=torch.float32, device=x.device)
    x3 = gemm(f, w.Wproj, epi=EPI_RESID_SS, r1=x2, ss_out=ss3)
    ctx = LayerCtx(x, ss1, P, h, y, x2, ss2, u, f, h0) if save else None
    return x3, ss3, hT, ctx


def layer_backward(dx3: torch.Tensor, ctx: LayerCtx, w: LayerWeights, B: int, T: int,
                   dhT: Optional[torch.Tensor] = None, *, want_dh0: bool = False,
                   outs: Optional[dict] = None):
    """Backward of :func:`layer_forward`.  Returns ``(dx, LayerGrads)``.

    ``outs`` may map ``dWp / dWo / dWfc / dWproj / dwn1 / dwn2`` to preallocated
    fp32 tensors (views of a flat gradient buffer) that receive the results.
    """
    R, D = ctx.x.shape
    inv_d = 1.0 / D
    o = outs or {}
    # feed-forward half
    du = gemm(dx3, w.Wproj, b_mn=True, epi=EPI_DSILU, r1=ctx.u, rowss=ctx.ss2, inv_dim=inv_d, eps=EPS)
    dWproj, _ = splitk_reduce(_wgrad(dx3, ctx.f), out=o.get("dWproj"))
    dx2 = gemm(du, w.Wfc_f, b_mn=True, epi=EPI_RMSBWD, r1=ctx.x2, r2=dx3, rowss=ctx.ss2,
               inv_dim=inv_d, eps=EPS)
    dWfc, dwn2 = splitk_reduce(_wgrad(du, ctx.x2), colscale=w.wn2, W=w.Wfc, out=o.get("dWfc"),
                               dcol_out=o.get("dwn2"))
    # recurrence half
    dy = gemm(dx2, w.Wo, b_mn=True)
    dWo, _ = splitk_reduce(_wgrad(dx2, ctx.y), out=o.get("dWo"))
    dP, dlog_a, dh0 = _scan_bwd(ctx.P, w.log_a32, ctx.h0, ctx.h, dy, dhT, ctx.ss1, inv_d, EPS, B, T,
                                D, want_dh0)
    dx = gemm(dP, w.Wp_f, b_mn=True, epi=EPI_RMSBWD, r1=ctx.x, r2=dx2, rowss=ctx.ss1, inv_dim=inv_d,
              eps=EPS)
    dWp, dwn1 = splitk_reduce(_wgrad(dP, ctx.x), colscale=w.wn1, W=w.Wp, out=o.get("dWp"),
                              dcol_out=o.get("dwn1"))
    if "dlog_a" in o:
        o["dlog_a"].copy_(dlog_a)
    return dx, LayerGrads(dWp, dWo, dWfc, dWproj, dwn1, dwn2, dlog_a, dh0)
