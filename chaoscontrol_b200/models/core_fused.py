"""``FusedCareSSMBlock``: a drop-in ``CareSSMBlock`` (same parameter names, state dicts
round-trip) whose forward AND backward are the hand-scheduled kernel sequence of
``ops/trunk.py`` behind one autograd node, plus ``post_scan_fused`` for the
residual + RMSNorm + feed-forward + residual tail on its own (API of
src/chaoscontrol/core_fused.py:86-429).

The reference fuses only the post-scan tail, and does so by tracing it with a compiler
(core_fused.py:151-193).  Here the whole block is four tcgen05 GEMMs and one scan kernel in
each direction with every elementwise op in an epilogue, and it also takes an initial state
(the reference's fused block drops to the unfused path for carried state).  Configurations the
kernels do not take (CPU, fp32, non-diagonal A, rich-B, Jacobian statistics, low-rank delta)
run the plain module path, so the block is safe to use anywhere.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import gemm as G
from ..ops import trunk as T
from .core import CareSSMCore, FeedForward, RMSNorm

__all__ = ["FusedCareSSMBlock", "post_scan_fused", "post_scan_reference", "get_post_scan_backend"]


def get_post_scan_backend() -> dict[str, str]:
    """Which implementation ``post_scan_fused`` runs (core_fused.py:196-202 of the reference reports
    its compiled / eager choice; here there is no tracing compiler to fall back from)."""
    import torch as _t
    if _t.cuda.is_available():
        return {"backend": "tcgen05_gemm_epilogues",
                "note": "bf16 CUDA operands run two GEMMs with RMSNorm, SiLU and residual adds fused in their "
                        "epilogues; other operands run the PyTorch statement"}
    return {"backend": "eager", "note": "no CUDA device: PyTorch statement"}


def post_scan_reference(x_pre_residual, scan_out, ff_norm_weight, ff_norm_eps, ff_fc_weight, ff_proj_weight):
    """``x = x_pre + scan_out;  x + proj(silu(fc(RMSNorm(x))))`` in plain PyTorch."""
    x = x_pre_residual + scan_out
    normed = F.rms_norm(x.float(), (x.size(-1),), eps=ff_norm_eps).to(x.dtype) * ff_norm_weight
    return x + F.linear(F.silu(F.linear(normed, ff_fc_weight)), ff_proj_weight)


def _kernels_ok(x: torch.Tensor, *weights: torch.Tensor) -> bool:
    D = x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and D % 64 == 0 and D <= 512 and
            all(w.dtype == torch.bfloat16 for w in weights))


class _PostScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_pre, scan_out, wn2, eps, Wfc, Wproj):
        shp = x_pre.shape
        D = shp[-1]
        x2 = (x_pre + scan_out).reshape(-1, D).contiguous()
        ss2 = x2.float().square().sum(-1)
        Wfc_f = T.fold_colscale(Wfc.contiguous(), wn2.contiguous())
        f = torch.empty(x2.shape[0], Wfc.shape[0], dtype=x2.dtype, device=x2.device)
        u = G.gemm(x2, Wfc_f, epi=G.EPI_ROWSCALE_SILU, rowss=ss2, inv_dim=1.0 / D, eps=eps, c2=f)
        x3 = G.gemm(f, Wproj.contiguous(), epi=G.EPI_RESID_SS, r1=x2, ss_out=torch.empty_like(ss2))
        ctx.save_for_backward(x2, ss2, u, f, wn2, Wfc, Wproj, Wfc_f)
        ctx.eps, ctx.shp = eps, shp
        return x3.view(shp)

    @staticmethod
    def backward(ctx, go):
        x2, ss2, u, f, wn2, Wfc, Wproj, Wfc_f = ctx.saved_tensors
        D = x2.shape[1]
        dx3 = go.reshape(-1, D).contiguous()
        du = G.gemm(dx3, Wproj, b_mn=True, epi=G.EPI_DSILU, r1=u, rowss=ss2, inv_dim=1.0 / D, eps=ctx.eps)
        dWproj, _ = T.splitk_reduce(T._wgrad(dx3, f))
        dx2 = G.gemm(du, Wfc_f, b_mn=True, epi=G.EPI_RMSBWD, r1=x2, r2=dx3, rowss=ss2, inv_dim=1.0 / D, eps=ctx.eps)
        dWfc, dwn2 = T.splitk_reduce(T._wgrad(du, x2), colscale=wn2, W=Wfc)
        dx2 = dx2.view(ctx.shp)
        return dx2, dx2, dwn2.to(wn2.dtype), None, dWfc.to(Wfc.dtype), dWproj.to(Wproj.dtype)


def post_scan_fused(x_pre_residual, scan_out, ff_norm_weight, ff_norm_eps, ff_fc_weight, ff_proj_weight):
    """Two tcgen05 GEMMs with the RMSNorm, SiLU and both residual adds in their epilogues (forward and
    backward); the PyTorch statement elsewhere."""
    if _kernels_ok(x_pre_residual, ff_norm_weight, ff_fc_weight, ff_proj_weight) and scan_out.dtype == torch.bfloat16:
        return _PostScanFn.apply(x_pre_residual, scan_out, ff_norm_weight, float(ff_norm_eps), ff_fc_weight,
                                 ff_proj_weight)
    return post_scan_reference(x_pre_residual, scan_out, ff_norm_weight, ff_norm_eps, ff_fc_weight, ff_proj_weight)


class _BlockFn(torch.autograd.Function):
    """The whole block as one node: ``(x, h0?, 10 parameters) -> (x_out, h_T)``."""

    @staticmethod
    def forward(ctx, x, h0, sel, inp, gate, delta, out, fc, proj, wn1, wn2, log_a):
        B, Tn, D = x.shape
        w = T.LayerWeights(Wp=torch.cat([sel, inp, gate, delta], 0), Wo=out.contiguous(), Wfc=fc.contiguous(),
                           Wproj=proj.contiguous(), wn1=wn1.contiguous(), wn2=wn2.contiguous(), log_a=log_a).prepare()
        x2d = x.reshape(B * Tn, D).contiguous()
        ss1 = x2d.float().square().sum(-1)
        h0f = None if h0 is None else h0.float().contiguous()
        x3, _ss3, hT, c = T.layer_forward(x2d, ss1, w, B, Tn, h0f, save=True)
        ctx.w, ctx.c, ctx.dims = w, c, (B, Tn, D)
        ctx.has_h0 = h0 is not None
        ctx.dtypes = (wn1.dtype, log_a.dtype)
        ctx.mark_non_differentiable(hT)
        return x3.view(B, Tn, D), hT

    @staticmethod
    def backward(ctx, go, _ghT):
        B, Tn, D = ctx.dims
        dx, g = T.layer_backward(go.reshape(B * Tn, D).contiguous(), ctx.c, ctx.w, B, Tn, None,
                                 want_dh0=ctx.has_h0 and ctx.needs_input_grad[1])
        ctx.c = None
        wdt = ctx.w.Wo.dtype
        dsel, dinp, dgate, ddelta = (t.to(wdt) for t in g.dWp.split(D, 0))
        ndt, adt = ctx.dtypes
        return (dx.view(B, Tn, D), g.dh0 if ctx.has_h0 else None, dsel, dinp, dgate, ddelta, g.dWo.to(wdt),
                g.dWfc.to(wdt), g.dWproj.to(wdt), g.dwn1.to(ndt), g.dwn2.to(ndt), g.dlog_a.to(adt))


class FusedCareSSMBlock(nn.Module):
    def __init__(self, dim: int, ff_mult: int = 2, *, a_mode: str = "diag", a_full_rank: int = 8,
                 a_full_gamma: float = 0.05, ssm_delta_rank: int = 0) -> None:
        super().__init__()
        self.input_norm = RMSNorm(dim)
        self.ff_norm = RMSNorm(dim)
        self.ff = FeedForward(dim, ff_mult)
        self.core = CareSSMCore(dim, a_mode=a_mode, a_full_rank=a_full_rank, a_full_gamma=a_full_gamma,
                                delta_rank=ssm_delta_rank)
        self.rich_b: Optional[nn.Module] = None
        self._a_mode = a_mode

    @classmethod
    def from_unfused(cls, block: nn.Module) -> "FusedCareSSMBlock":
        """Same weights and dtype as ``block`` (diagonal A, no rich-B), loaded strictly."""
        core = block.core
        if core.a_mode != "diag":
            raise ValueError(f"FusedCareSSMBlock.from_unfused requires a_mode='diag', got {core.a_mode!r}")
        if block.rich_b is not None:
            raise ValueError("FusedCareSSMBlock.from_unfused requires rich_b=None")
        fused = cls(core.dim, block.ff.fc.out_features // core.dim, a_mode="diag",
                    ssm_delta_rank=int(getattr(core, "delta_rank", 0)))
        ref = block.ff.fc.weight
        fused = fused.to(device=ref.device, dtype=ref.dtype)
        fused.load_state_dict(block.state_dict(), strict=True)
        return fused

    def _kernel_path(self, x: torch.Tensor) -> bool:
        c = self.core
        return (self._a_mode == "diag" and int(getattr(c, "delta_rank", 0)) == 0 and x.dim() == 3 and
                _kernels_ok(x, *(p for p in self.parameters())))

    def step(self, x: torch.Tensor, state: torch.Tensor):
        y, new_state = self.core.step(self.input_norm(x), state, rich_b=None)
        x = x + y
        return x + self.ff(self.ff_norm(x)), new_state

    def forward(self, x: torch.Tensor, *, return_jacobian_stats: bool = False,
                initial_state: Optional[torch.Tensor] = None, return_final_state: bool = False):
        if return_jacobian_stats or not self._kernel_path(x):
            return self._forward_unfused(x, return_jacobian_stats=return_jacobian_stats, initial_state=initial_state,
                                         return_final_state=return_final_state)
        c, ff = self.core, self.ff
        y, hT = _BlockFn.apply(x, initial_state, c.select_proj.weight, c.in_proj.weight, c.gate_proj.weight,
                               c.delta_proj.weight, c.out_proj.weight, ff.fc.weight, ff.proj.weight,
                               self.input_norm.weight, self.ff_norm.weight, c.log_a)
        return (y, hT) if return_final_state else y

    def _forward_unfused(self, x, *, return_jacobian_stats=False, initial_state=None, return_final_state=False):
        res = self.core(self.input_norm(x), rich_b=self.rich_b, return_jacobian_stats=return_jacobian_stats,
                        initial_state=initial_state, return_final_state=return_final_state)
        extras = ()
        if return_jacobian_stats or return_final_state:
            y, *extras = res
        else:
            y = res
        x = post_scan_fused(x, y, self.ff_norm.weight, self.ff_norm.eps, self.ff.fc.weight, self.ff.proj.weight)
        return (x, *extras) if extras else x
