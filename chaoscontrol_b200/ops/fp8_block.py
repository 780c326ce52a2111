"""Block-scaled e4m3 linear layer (``csrc/fp8_block.cu``).

Activations and output gradients are quantised per row and 128-wide block of
the contraction dimension ("1 x 128"), weights per 128 x 128 block; master
weights stay bf16.  ``y = x @ W.T`` and ``dx = dy @ W`` run as block-scaled
tcgen05 GEMMs (the per-block scales are applied while the K-block partial
products are added up in the epilogue), ``dW = dy.T @ x`` stays bf16.

The cast is fused into the producer where one exists: :func:`rmsnorm_quant`
normalises a row, writes the bf16 result that autograd needs and the e4m3 row
with its scales in the same pass, and tags the returned tensor so that every
:class:`BlockFP8Linear` fed by it skips its own quantisation pass.

Finer-grained replacement of the reference's per-tensor cuBLASLt fp8 linear
(src/chaoscontrol/kernels/fp8_linear.py:171-265, 292-348); the per-tensor
delayed-scaling layer with the reference's exact contract is
``ops/fp8_linear.py``.  Everything also runs on CPU through a PyTorch emulation
of the same quantisation, which is what the CPU tests check.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from . import gemm as G

E4M3_MAX = 448.0
BLOCK = 128

__all__ = ["quant_rows", "quant_blocks", "block_gemm", "block_linear_reference", "rmsnorm_quant",
           "BlockFP8Linear", "QuantRows"]


class QuantRows:
    """e4m3 rows ``q`` [R, K] with scales ``s_t`` [K/128, R]."""
    __slots__ = ("q", "s_t")

    def __init__(self, q: torch.Tensor, s_t: torch.Tensor) -> None:
        self.q, self.s_t = q, s_t

    def dequant(self) -> torch.Tensor:
        R, K = self.q.shape
        return (self.q.float().view(R, K // BLOCK, BLOCK) * self.s_t.t().unsqueeze(-1)).view(R, K)


def _use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and _lib.available()


def _to_e4m3(v: torch.Tensor) -> torch.Tensor:
    return v.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def quant_rows(x: torch.Tensor, *, norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
               want_normed: bool = False):
    """``(QuantRows, inv_rms or None, normed bf16 or None)`` of ``x`` [R, K] (of
    ``RMSNorm(x) * norm_weight`` when a weight is given)."""
    R, K = x.shape
    if K % BLOCK:
        raise ValueError(f"quant_rows: K={K} must be a multiple of {BLOCK}")
    if _use_kernels(x) and K <= 2048 and x.stride(1) == 1 and x.stride(0) % 8 == 0:
        q = torch.empty(R, K, dtype=torch.float8_e4m3fn, device=x.device)
        s_t = torch.empty(K // BLOCK, R, dtype=torch.float32, device=x.device)
        inv = torch.empty(R, dtype=torch.float32, device=x.device) if norm_weight is not None else None
        y = torch.empty(R, K, dtype=torch.bfloat16, device=x.device) if want_normed else None
        w = norm_weight.to(torch.bfloat16).contiguous() if norm_weight is not None else None
        _lib.check(_lib.lib().ccb_fp8_quant_rows(x.data_ptr(), x.stride(0), _lib.ptr(w), float(eps), q.data_ptr(),
                                                 s_t.data_ptr(), _lib.ptr(inv), _lib.ptr(y), R, K,
                                                 _lib.stream_ptr()), "fp8_quant_rows")
        return QuantRows(q, s_t), inv, y
    v = x.float()
    inv = None
    if norm_weight is not None:
        inv = torch.rsqrt(v.square().mean(-1) + eps)
        v = v * inv[:, None] * norm_weight.to(torch.bfloat16).float()
    blocks = v.view(R, K // BLOCK, BLOCK)
    scale = blocks.abs().amax(-1).clamp_min(1e-12) / E4M3_MAX
    q = _to_e4m3(blocks / scale.unsqueeze(-1)).view(R, K)
    return QuantRows(q, scale.t().contiguous()), inv, (v.to(x.dtype) if want_normed else None)


def quant_blocks(w: torch.Tensor, *, want_transpose: bool = True):
    """``(q [N, K], qt [K, N] or None, s [ceil(N/128), ceil(K/128)])`` of a weight matrix."""
    N, K = w.shape
    nb, kb = (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK
    if _use_kernels(w) and w.is_contiguous():
        q = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=w.device)
        qt = torch.empty(K, N, dtype=torch.float8_e4m3fn, device=w.device) if want_transpose else None
        s = torch.empty(nb, kb, dtype=torch.float32, device=w.device)
        _lib.check(_lib.lib().ccb_fp8_quant_blocks(w.data_ptr(), q.data_ptr(), _lib.ptr(qt), s.data_ptr(), N, K,
                                                   _lib.stream_ptr()), "fp8_quant_blocks")
        return q, qt, s
    pad = F.pad(w.float(), (0, kb * BLOCK - K, 0, nb * BLOCK - N)).view(nb, BLOCK, kb, BLOCK)
    s = pad.abs().amax(dim=(1, 3)).clamp_min(1e-12) / E4M3_MAX
    q = _to_e4m3(pad / s[:, None, :, None]).view(nb * BLOCK, kb * BLOCK)[:N, :K].contiguous()
    return q, (q.t().contiguous() if want_transpose else None), s


def block_gemm(a: QuantRows, b8: torch.Tensor, sb: torch.Tensor, *, sb_strides: tuple[int, int],
               bias: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``C[m, n] = sum_kb a.s_t[kb, m] * sb[(n // 128) * so + kb * sk] * (a.q[m, kb] . b8[n, kb])``."""
    M, K = a.q.shape
    N = b8.shape[0]
    so, sk = sb_strides
    if a.q.is_cuda and _lib.available():
        out = torch.empty(M, N, dtype=out_dtype, device=a.q.device)
        _lib.check(_lib.lib().ccb_fp8_block_gemm(a.q.data_ptr(), a.s_t.data_ptr(), b8.data_ptr(), sb.data_ptr(),
                                                 so, sk, out.data_ptr(), out.stride(0),
                                                 int(out_dtype == torch.float32), _lib.ptr(bias), M, N, K,
                                                 _lib.stream_ptr()), "fp8_block_gemm")
        return out
    kb = K // BLOCK
    nbk = (N + BLOCK - 1) // BLOCK
    idx = (torch.arange(nbk, device=sb.device)[:, None] * so + torch.arange(kb, device=sb.device)[None, :] * sk)
    sbm = sb.reshape(-1)[idx]                                                   # [nb, kb]
    af = a.q.float().view(M, kb, BLOCK)
    bf = F.pad(b8.float(), (0, 0, 0, nbk * BLOCK - N)).view(nbk, BLOCK, kb, BLOCK)
    part = torch.einsum("mkc,jnkc->mjnk", af, bf)                               # per-block partial products
    out = (part * a.s_t.t()[:, None, None, :] * sbm[None, :, None, :]).sum(-1).reshape(M, nbk * BLOCK)[:, :N]
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype)


def block_linear_reference(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 statement of the forward: quantise-dequantise both operands, then an exact matmul."""
    qa, _, _ = quant_rows(x.detach().cpu().to(torch.bfloat16))
    q, _, s = quant_blocks(w.detach().cpu().to(torch.bfloat16), want_transpose=False)
    N, K = w.shape
    wd = (F.pad(q.float(), (0, s.shape[1] * BLOCK - K, 0, s.shape[0] * BLOCK - N))
          .view(s.shape[0], BLOCK, s.shape[1], BLOCK) * s[:, None, :, None]).view(s.shape[0] * BLOCK, -1)[:N, :K]
    out = qa.dequant() @ wd.t()
    return out + bias.detach().cpu().float() if bias is not None else out


# ---------------------------------------------------------------------------
# producer-fused quantisation: RMSNorm that also emits the e4m3 row
# ---------------------------------------------------------------------------
class _RmsNormQuantFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        qr, inv, y = quant_rows(x2, norm_weight=weight, eps=eps, want_normed=True)
        ctx.save_for_backward(x2, weight, inv)
        ctx.shp = shp
        ctx.mark_non_differentiable(qr.q, qr.s_t)
        return y.view(shp), qr.q, qr.s_t

    @staticmethod
    def backward(ctx, go, _gq, _gs):
        x2, weight, inv = ctx.saved_tensors
        R, D = x2.shape
        go2 = go.reshape(R, D)
        if _use_kernels(x2):
            w = weight.to(torch.bfloat16).contiguous()
            go2 = go2.contiguous().to(torch.bfloat16)
            gx = torch.empty_like(x2)
            nb = int(_lib.lib().ccb_rmsnorm_bwd_blocks(R))
            part = torch.empty(nb, D, dtype=torch.float32, device=x2.device)
            gw = torch.empty(D, dtype=torch.float32, device=x2.device)
            _lib.check(_lib.lib().ccb_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), go2.data_ptr(), inv.data_ptr(),
                                                  gx.data_ptr(), part.data_ptr(), gw.data_ptr(), R, D,
                                                  _lib.stream_ptr()), "rmsnorm_bwd")
            return gx.view(ctx.shp), gw.to(weight.dtype), None
        xf, g = x2.float(), go2.float() * weight.to(torch.bfloat16).float()
        xn = xf * inv[:, None]
        gx = inv[:, None] * (g - xn * (g * xn).mean(-1, keepdim=True))
        gw = (go2.float() * xn).sum(0)
        return gx.to(x2.dtype).view(ctx.shp), gw.to(weight.dtype), None


def rmsnorm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm whose result carries its own block-scaled e4m3 copy (attribute
    ``_ccb_quant``), produced in the same pass over the row."""
    y, q, s_t = _RmsNormQuantFn.apply(x, weight, eps)
    y._ccb_quant = QuantRows(q, s_t)
    return y


# ---------------------------------------------------------------------------
# the linear layer
# ---------------------------------------------------------------------------
class _BlockFP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, pre: Optional[QuantRows]):
        shp = x.shape
        K = shp[-1]
        x2 = x.reshape(-1, K)
        wb = weight.to(torch.bfloat16)
        qa = pre if pre is not None else quant_rows(x2.to(torch.bfloat16).contiguous())[0]
        q, qt, s = quant_blocks(wb.contiguous())
        kbw = s.shape[1]
        out = block_gemm(qa, q, s, sb_strides=(kbw, 1), bias=bias.to(torch.bfloat16) if bias is not None else None,
                         out_dtype=torch.bfloat16)
        ctx.save_for_backward(x2, qt, s)
        ctx.meta = (shp, weight.dtype, bias is not None, weight.shape)
        return out.view(*shp[:-1], weight.shape[0]).to(x.dtype if x.dtype != torch.float32 else torch.float32)

    @staticmethod
    def backward(ctx, go):
        x2, qt, s = ctx.saved_tensors
        shp, wdtype, has_bias, (N, K) = ctx.meta
        g2 = go.reshape(-1, N).to(torch.bfloat16).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            if N % BLOCK == 0:
                qg = quant_rows(g2)[0]
                # B = W^T stored [K, N]: output block j is a K block of W, contraction block kb an N block
                gx = block_gemm(qg, qt, s, sb_strides=(1, s.shape[1]), out_dtype=torch.bfloat16)
            else:
                gx = (g2.float() @ _dequant_t(qt, s, N, K).t()).to(torch.bfloat16)
            gx = gx.view(shp).to(x2.dtype)
        if ctx.needs_input_grad[1]:
            xb = x2.to(torch.bfloat16).contiguous()
            if g2.is_cuda and _lib.available():
                S = G.pick_splits(N, K, g2.shape[0])
                part = G.gemm(g2, xb, a_mn=True, b_mn=True, splits=S, out_dtype=torch.float32)
                gw = part.sum(0) if part.dim() == 3 else part
            else:
                gw = g2.float().t() @ xb.float()
            gw = gw.to(wdtype)
        if has_bias and ctx.needs_input_grad[2]:
            gb = g2.float().sum(0).to(wdtype)
        return gx, gw, gb, None


def _dequant_t(qt: torch.Tensor, s: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """fp32 ``W^T`` [K, N] from the transposed e4m3 weight and its block scales."""
    nb, kb = s.shape
    pad = F.pad(qt.float(), (0, nb * BLOCK - N, 0, kb * BLOCK - K)).view(kb, BLOCK, nb, BLOCK)
    return (pad * s.t()[:, None, :, None]).view(kb * BLOCK, nb * BLOCK)[:K, :N]


class BlockFP8Linear(nn.Module):
    """``nn.Linear`` computed in block-scaled e4m3 (bf16 master weight, bf16 output)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None,
                 dtype=torch.bfloat16) -> None:
        super().__init__()
        if in_features % BLOCK:
            raise ValueError(f"BlockFP8Linear: in_features={in_features} must be a multiple of {BLOCK}")
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    @classmethod
    def from_nn_linear(cls, lin: nn.Linear) -> "BlockFP8Linear":
        m = cls(lin.in_features, lin.out_features, bias=lin.bias is not None, device=lin.weight.device,
                dtype=lin.weight.dtype)
        m.weight = lin.weight
        if lin.bias is not None:
            m.bias = lin.bias
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        pre = getattr(x, "_ccb_quant", None)
        if pre is not None and pre.q.shape != (x.numel() // x.shape[-1], x.shape[-1]):
            pre = None
        return _BlockFP8LinearFn.apply(x, self.weight, self.bias, pre)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
