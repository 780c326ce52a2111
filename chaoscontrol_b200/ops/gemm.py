"""Python front-end of the tcgen05 GEMM (``csrc/gemm.cu``).

``gemm(a, b)`` computes ``a @ b.T`` for K-major operands (``a`` is ``[M, K]``,
``b`` is ``[N, K]``: the ``F.linear`` form).  ``a_mn`` / ``b_mn`` say that the
operand is stored transposed (``[K, M]`` / ``[K, N]``), which is how the
backward GEMMs consume activations and weights without any transpose copy:

* forward      ``y  = x @ W.T``        -> ``gemm(x, W)``
* input grad   ``dx = dy @ W``         -> ``gemm(dy, W, b_mn=True)``
* weight grad  ``dW = dy.T @ x``       -> ``gemm(dy, x, a_mn=True, b_mn=True, splits=S)``

A CPU / fp32 reference of every epilogue lives in :func:`gemm_reference` and
is what the GPU tests compare against.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import (EPI_CE_GRAD, EPI_DSILU, EPI_LSE_PART, EPI_RESID_SS, EPI_RMSBWD, EPI_ROWSCALE,
                   EPI_ROWSCALE_SILU, EPI_STORE, GemmArgs)

__all__ = ["gemm", "gemm_fp8", "gemm_lm", "gemm_reference", "pick_splits", "EPI_STORE", "EPI_ROWSCALE",
           "EPI_ROWSCALE_SILU", "EPI_RESID_SS", "EPI_DSILU", "EPI_RMSBWD", "EPI_LSE_PART", "EPI_CE_GRAD"]


def pick_splits(m: int, n: int, k: int, bn: int = 256) -> int:
    """Split-K factor that fills the SMs for a weight-gradient GEMM."""
    tiles = ((m + 127) // 128) * ((n + bn - 1) // bn)
    kblocks = (k + 63) // 64
    sms = _lib.lib().ccb_num_sms() if _lib.available() else 148
    want = max(1, sms // max(tiles, 1))
    want = min(want, kblocks)
    # the kernel needs every split non-empty: shrink until ceil-division is exact
    while want > 1:
        kper = (kblocks + want - 1) // want
        if (kblocks + kper - 1) // kper == want:
            break
        want -= 1
    return want


def _dims(a: torch.Tensor, b: torch.Tensor, a_mn: bool, b_mn: bool):
    batch = a.shape[0] if a.dim() == 3 else 1
    am, ak = (a.shape[-1], a.shape[-2]) if a_mn else (a.shape[-2], a.shape[-1])
    bn, bk = (b.shape[-1], b.shape[-2]) if b_mn else (b.shape[-2], b.shape[-1])
    if ak != bk:
        raise ValueError(f"contraction mismatch: {tuple(a.shape)} vs {tuple(b.shape)}")
    return batch, am, bn, ak


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         splits: int = 1, epi: int = EPI_STORE, alpha: float = 1.0, beta: float = 0.0,
         cin: Optional[torch.Tensor] = None, r1: Optional[torch.Tensor] = None,
         r2: Optional[torch.Tensor] = None, rowss: Optional[torch.Tensor] = None,
         inv_dim: float = 0.0, eps: float = 1e-6, c2: Optional[torch.Tensor] = None,
         ss_out: Optional[torch.Tensor] = None, ss_atomic: bool = False) -> torch.Tensor:
    if not a.is_cuda:
        return _gemm_cpu(a, b, a_mn=a_mn, b_mn=b_mn, out=out, out_dtype=out_dtype, splits=splits,
                         epi=epi, alpha=alpha, beta=beta, cin=cin, r1=r1, r2=r2, rowss=rowss,
                         inv_dim=inv_dim, eps=eps, c2=c2, ss_out=ss_out, ss_atomic=ss_atomic)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm operands must be bf16")
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm operands must have a contiguous last dimension")
    batch, M, N, K = _dims(a, b, a_mn, b_mn)
    if epi == EPI_RESID_SS and ss_out is not None and N > 256 and not ss_atomic:
        # a row spans several N tiles: each tile adds its share into a zeroed buffer
        ss_out.zero_()
        ss_atomic = True
    if out is None:
        shape = (M, N) if a.dim() == 2 else (batch, M, N)
        if splits > 1:
            shape = (splits, *shape)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    args = GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.C2 = _lib.ptr(c2)
    args.Cin = _lib.ptr(cin)
    args.R1, args.R2 = _lib.ptr(r1), _lib.ptr(r2)
    args.rowss, args.ss_out = _lib.ptr(rowss), _lib.ptr(ss_out)
    args.M, args.N, args.K = M, N, K
    args.batch, args.splits = batch, splits
    args.lda, args.ldb = a.stride(-2), b.stride(-2)
    args.ldc = out.stride(-2)
    args.ldcin = cin.stride(-2) if cin is not None else 0
    args.ldr = r1.stride(-2) if r1 is not None else 0
    args.a_batch = a.stride(0) if a.dim() == 3 else 0
    args.b_batch = b.stride(0) if b.dim() == 3 else 0
    if splits > 1:
        args.c_split = out.stride(0)
        args.c_batch = out.stride(1) if a.dim() == 3 else 0
    else:
        args.c_split = 0
        args.c_batch = out.stride(0) if a.dim() == 3 else 0
    args.cin_batch = cin.stride(0) if (cin is not None and cin.dim() == 3) else 0
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.epi = epi
    args.out_fp32 = int(out.dtype == torch.float32)
    args.ss_atomic = int(ss_atomic)
    args.alpha, args.beta, args.inv_dim, args.eps = alpha, beta, inv_dim, eps
    _lib.check(_lib.lib().ccb_gemm(C.byref(args), _lib.stream_ptr()), "gemm")
    return out


def gemm_lm(x: torch.Tensor, w: torch.Tensor, *, epi: int, targets: torch.Tensor,
            rowss: Optional[torch.Tensor], inv_dim: float, eps: float, lse: Optional[torch.Tensor] = None,
            rowweight: Optional[torch.Tensor] = None, alpha: float = 1.0,
            out: Optional[torch.Tensor] = None, zt_out: Optional[torch.Tensor] = None):
    """LM-head epilogues on ``logits = rs * (x @ w.T)`` (``x`` ``[R, D]``, ``w`` ``[V, D]``, bf16, CUDA).

    ``EPI_LSE_PART`` returns ``(partials [2 * ceil(V / 256), R, 2] fp32, zt [R])``: log2-domain
    ``(max, sum)`` per half tile and the target logit; no logits are written.
    ``EPI_CE_GRAD`` returns the bf16 ``[R, V]`` gradient of the summed, ``alpha * rowweight``-weighted
    cross-entropy w.r.t. the un-scaled GEMM output, and fills ``zt_out`` with the per-row CE.
    """
    R, D = x.shape
    V = w.shape[0]
    args = GemmArgs()
    args.A, args.B = x.data_ptr(), w.data_ptr()
    args.M, args.N, args.K = R, V, D
    args.batch, args.splits = 1, 1
    args.lda, args.ldb = x.stride(0), w.stride(0)
    args.epi = epi
    args.alpha, args.beta, args.inv_dim, args.eps = alpha, 0.0, inv_dim, eps
    args.rowss = _lib.ptr(rowss)
    t = targets.reshape(-1)
    if t.dtype != torch.int64:
        t = t.long()
    t = t.contiguous()
    args.targets = t.data_ptr()
    res = None
    if epi == EPI_LSE_PART:
        nparts = 2 * ((V + 255) // 256)
        part = torch.empty(nparts, R, 2, dtype=torch.float32, device=x.device)
        zt = zt_out if zt_out is not None else torch.empty(R, dtype=torch.float32, device=x.device)
        args.part_out, args.zt_out = part.data_ptr(), zt.data_ptr()
        args.ldc = V
        res = (part, zt)
    elif epi == EPI_CE_GRAD:
        if out is None:
            out = torch.empty(R, V, dtype=torch.bfloat16, device=x.device)
        args.C, args.ldc = out.data_ptr(), out.stride(0)
        args.lse, args.rowweight, args.zt_out = lse.data_ptr(), _lib.ptr(rowweight), _lib.ptr(zt_out)
        res = out
    else:
        raise ValueError(f"gemm_lm: epilogue {epi} is not an LM-head epilogue")
    _lib.check(_lib.lib().ccb_gemm(C.byref(args), _lib.stream_ptr()), "gemm_lm")
    return res


_FP8_CODE = {torch.float8_e4m3fn: 1, torch.float8_e5m2: 2}


def gemm_fp8(a: torch.Tensor, b: torch.Tensor, *, scale_a: torch.Tensor, scale_b: torch.Tensor,
             bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
             out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``(scale_a * a) @ (scale_b * b).T (+ bias)`` for 8-bit float operands.

    ``a`` ``[M, K]`` and ``b`` ``[N, K]`` are ``float8_e4m3fn`` / ``float8_e5m2``
    (any mix), K-major, with row strides that are multiples of 16 bytes; the
    scales are one-element fp32 device tensors read by the kernel (no host
    sync).  Runs ``tcgen05.mma kind::f8f6f4`` with fp32 accumulation.  The
    reference's counterpart is its cuBLASLt call
    (src/chaoscontrol/kernels/_cublaslt/src/cublaslt_fp8_matmul.cpp:281-291).
    """
    if a.dtype not in _FP8_CODE or b.dtype not in _FP8_CODE:
        raise TypeError("gemm_fp8 operands must be float8_e4m3fn or float8_e5m2")
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"contraction mismatch: {tuple(a.shape)} vs {tuple(b.shape)}")
    if not a.is_cuda:
        res = (a.float() * scale_a.float()) @ (b.float() * scale_b.float()).T
        if bias is not None:
            res = res + bias.float()
        if out is not None:
            return out.copy_(res.to(out.dtype))
        return res.to(out_dtype)
    if a.stride(-1) != 1 or b.stride(-1) != 1 or a.stride(0) % 16 or b.stride(0) % 16:
        raise ValueError("gemm_fp8 operands need a contiguous last dimension and 16-byte row strides")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    args = GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.M, args.N, args.K = M, N, K
    args.batch, args.splits = 1, 1
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(0)
    args.epi = EPI_STORE
    args.out_fp32 = int(out.dtype == torch.float32)
    args.alpha, args.beta, args.inv_dim, args.eps = 1.0, 0.0, 0.0, 0.0
    args.a_fp8, args.b_fp8 = _FP8_CODE[a.dtype], _FP8_CODE[b.dtype]
    args.dscale_a, args.dscale_b = scale_a.data_ptr(), scale_b.data_ptr()
    args.bias = _lib.ptr(bias)
    _lib.check(_lib.lib().ccb_gemm(C.byref(args), _lib.stream_ptr()), "gemm_fp8")
    return out


def _gemm_cpu(a, b, *, a_mn, b_mn, out, out_dtype, splits, epi, alpha, beta, cin, r1, r2, rowss,
              inv_dim, eps, c2, ss_out, ss_atomic):
    """CPU stand-in with the kernel's exact call contract (any float dtype).

    Used by the CPU tests to check the hand-written backward algebra built on
    these epilogues, and by the CPU training path.  Split-K returns the full
    product in split 0 and zeros elsewhere so reducing over splits is exact.
    """
    res = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, epi=epi, alpha=alpha, beta=beta, cin=cin,
                         r1=r1, r2=r2, rowss=rowss, inv_dim=inv_dim, eps=eps)
    second = None
    if isinstance(res, tuple):
        res, second = res
    dt = out.dtype if out is not None else (a.dtype if out_dtype == torch.bfloat16 and
                                            a.dtype != torch.bfloat16 else out_dtype)
    if splits > 1:
        full = torch.zeros((splits, *res.shape), dtype=dt)
        full[0] = res.to(dt)
        res = full
    if out is not None:
        out.copy_(res.to(out.dtype))
    else:
        out = res.to(dt)
    if epi == EPI_ROWSCALE_SILU and c2 is not None:
        c2.copy_(second.to(c2.dtype))
    if epi == EPI_RESID_SS and ss_out is not None:
        ss = (out.float() ** 2).sum(-1)
        if ss_atomic:
            ss_out.add_(ss)
        else:
            ss_out.copy_(ss)
    return out


def gemm_reference(a, b, *, a_mn=False, b_mn=False, epi=EPI_STORE, alpha=1.0, beta=0.0, cin=None,
                   r1=None, r2=None, rowss=None, inv_dim=0.0, eps=1e-6):
    """fp32 PyTorch statement of what ``gemm`` computes (returns fp32 tensors).

    Returns ``out`` or ``(out, second)`` where ``second`` is the SiLU output
    (``EPI_ROWSCALE_SILU``) or the row sum of squares (``EPI_RESID_SS``).
    """
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float().transpose(-1, -2) if b_mn else b.float()
    acc = A @ B.transpose(-1, -2)
    rs = None
    if rowss is not None:
        rs = torch.rsqrt(rowss.float() * inv_dim + eps).unsqueeze(-1)
    if epi == EPI_STORE:
        out = alpha * acc
        if cin is not None:
            out = out + beta * cin.float()
        return out
    if epi == EPI_ROWSCALE:
        return acc * rs
    lowp = a.dtype == torch.bfloat16
    if epi == EPI_ROWSCALE_SILU:
        u = acc * rs
        if lowp:
            u = u.bfloat16().float()
        return u, torch.nn.functional.silu(u)
    if epi == EPI_RESID_SS:
        out = acc + r1.float()
        if lowp:
            out = out.bfloat16().float()
        return out, (out * out).sum(-1)
    if epi == EPI_DSILU:
        u = r1.float()
        s = torch.sigmoid(u)
        return acc * (s * (1 + u * (1 - s))) * rs
    if epi == EPI_RMSBWD:
        x = r1.float()
        coef = (acc * x).sum(-1, keepdim=True) * rs * rs * inv_dim
        out = acc - x * coef
        if r2 is not None:
            out = out + r2.float()
        return out
    raise ValueError(f"unknown epilogue {epi}")
