"""Fused LM head (``csrc/lmhead.cu``): linear + log-softmax + cross-entropy with
logits recomputed in backward, plus the PyTorch statements used on CPU and as
test oracles.

Inputs are the *un-normalised* final hidden state ``x`` with its row sums of
squares ``rowss`` (the final RMSNorm is applied inside the kernel as a row
scale) and ``W_f = lm_head.weight * final_norm.weight`` (norm weight folded).
Pass ``rowss=None`` for an already-normalised ``x``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from . import gemm as G
from ._lib import f32, i64, vp

_lib.register_sig("ccb_lmhead_lse", [vp, vp, vp, f32, vp, vp, vp, vp, i64, i64, i64, vp])
_lib.register_sig("ccb_lmhead_train", [vp, vp, vp, f32, vp, vp, f32, vp, i64, vp, vp, i64, i64, i64, vp])
_lib.register_sig("ccb_lmhead_dw", [vp, vp, vp, f32, vp, vp, f32, vp, vp, i64, i64, i64, i64, vp])

EPS = 1e-6


def fused_supported(x: torch.Tensor, W: torch.Tensor) -> bool:
    """Shapes / dtypes the tcgen05 LM-head kernels handle."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and W.dtype == torch.bfloat16 and
            x.shape[-1] == 256 and W.shape[0] % 128 == 0 and W.shape[1] == 256)


def general_supported(x: torch.Tensor, W: torch.Tensor) -> bool:
    """Shapes the GEMM-epilogue LM head handles (any model dim that keeps rows 16-byte
    aligned and fits the 512-column RMSNorm-backward tile)."""
    D = x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and W.dtype == torch.bfloat16 and W.shape[1] == D and
            D % 8 == 0 and D <= 512 and W.shape[0] % 8 == 0)


def kernel_supported(x: torch.Tensor, W: torch.Tensor) -> bool:
    """True when one of the two hand-written LM-head paths takes these operands."""
    return fused_supported(x, W) or general_supported(x, W)


def _lse_general(x, rowss, W_f, t, eps):
    """``(loss_rows, lse)`` from one GEMM whose epilogue reduces each half tile to a
    (max, sum) pair, followed by a per-row combine; logits never reach memory."""
    R, D = x.shape
    part, zt = G.gemm_lm(x, W_f, epi=G.EPI_LSE_PART, targets=t, rowss=rowss, inv_dim=1.0 / D, eps=eps)
    lse = torch.empty(R, dtype=torch.float32, device=x.device)
    loss = torch.empty(R, dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().ccb_lse_combine(part.data_ptr(), part.shape[0], R, zt.data_ptr(), lse.data_ptr(),
                                          loss.data_ptr(), _lib.stream_ptr()), "lse_combine")
    return loss, lse


def general_row_chunk(R: int) -> int:
    """Rows per backward chunk: one 128-row block per SM, so the paired-accumulator dX GEMM
    (one CTA per row block) fills the device exactly and the bf16 gradient chunk stays bounded."""
    sms = _lib.lib().ccb_num_sms() if _lib.available() else 148
    return min(R, 128 * sms)


def _train_general(x, rowss, W_f, t, gscale, rowweight, eps, lse, want_dw=True):
    """Chunked LM-head backward from GEMM epilogues.  Per row chunk: ``g = (softmax - onehot) *
    scale`` is produced by the logits GEMM's epilogue as a bf16 ``[rows, V]`` tile (bounded by the
    chunk, never the full ``[R, V]``), then ``dX = RMSNorm-backward(g @ W')`` and
    ``dW' += g^T @ X`` are two more tcgen05 GEMMs."""
    R, D = x.shape
    V = W_f.shape[0]
    if lse is None:
        loss, lse = _lse_general(x, rowss, W_f, t, eps)
    else:
        loss = torch.empty(R, dtype=torch.float32, device=x.device)
    rc = general_row_chunk(R)
    nchunks = (R + rc - 1) // rc
    S = G.pick_splits(V, D, rc)
    dX = torch.empty_like(x)
    part = torch.empty(nchunks * S, V, D, dtype=torch.float32, device=x.device) if want_dw else None
    gbuf = torch.empty(rc, V, dtype=torch.bfloat16, device=x.device)
    for i in range(nchunks):
        r0, r1 = i * rc, min(R, (i + 1) * rc)
        xc = x[r0:r1]
        ssc = rowss[r0:r1] if rowss is not None else None
        g = G.gemm_lm(xc, W_f, epi=G.EPI_CE_GRAD, targets=t[r0:r1], rowss=ssc, inv_dim=1.0 / D, eps=eps,
                      lse=lse[r0:r1], rowweight=rowweight[r0:r1] if rowweight is not None else None,
                      alpha=gscale, out=gbuf[: r1 - r0], zt_out=loss[r0:r1])
        if rowss is not None:
            G.gemm(g, W_f, b_mn=True, epi=G.EPI_RMSBWD, r1=xc, rowss=ssc, inv_dim=1.0 / D, eps=eps,
                   out=dX[r0:r1])
        else:
            G.gemm(g, W_f, b_mn=True, out=dX[r0:r1])
        if not want_dw:
            continue
        Sc = min(S, G.pick_splits(V, D, r1 - r0))
        if Sc != S:
            part[i * S + Sc:(i + 1) * S].zero_()
        G.gemm(g, xc, a_mn=True, b_mn=True, splits=Sc, out=part[i * S: i * S + Sc] if Sc > 1 else part[i * S])
    return loss, lse, dX, part


def lm_head_reference(x, rowss, W_f, targets, *, gscale: float = 1.0, rowweight=None,
                      eps: float = EPS, want_grads: bool = True):
    """fp32 statement.  Returns ``(loss_rows, lse, dX, dW_f)`` (grads None if not wanted)."""
    xf = x.detach().float().requires_grad_(want_grads)
    Wf = W_f.detach().float().requires_grad_(want_grads)
    D = xf.shape[-1]
    with torch.enable_grad():
        if rowss is not None:
            rs = torch.rsqrt((xf * xf).sum(-1) / D + eps)
            xn = xf * rs[:, None]
        else:
            xn = xf
        logits = xn @ Wf.t()
        lse = torch.logsumexp(logits, dim=-1)
        loss_rows = lse - logits.gather(1, targets.view(-1, 1).long()).squeeze(1)
        if not want_grads:
            return loss_rows.detach(), lse.detach(), None, None
        w = rowweight.float() if rowweight is not None else torch.ones_like(loss_rows)
        (loss_rows * w).sum().mul(gscale).backward()
    return loss_rows.detach(), lse.detach(), xf.grad, Wf.grad


def _refuse_unless_allowed(x, W_f, allow_materialized: bool, what: str) -> None:
    """On a CUDA device an operand the kernels do not take is an error, not a quiet drop to a
    logits-materialising PyTorch path (the reference's dispatcher refuses the same way,
    src/chaoscontrol/kernels/_lm_head_loss/__init__.py:1041-1145); a caller that wants that path
    says so with ``allow_materialized=True``.  CPU tensors always take the PyTorch statement."""
    if x.is_cuda and not allow_materialized:
        raise TypeError(f"{what}: no LM-head kernel takes x {tuple(x.shape)} {x.dtype} with W {tuple(W_f.shape)} "
                        f"{W_f.dtype} (bf16, model dim a multiple of 8 and at most 512, vocabulary a multiple of 8); "
                        "pass allow_materialized=True to run the PyTorch statement, which builds the logits")


def _prep(x, rowss, W_f, targets):
    assert x.is_contiguous() and W_f.is_contiguous()
    t = targets.reshape(-1)
    if t.dtype != torch.int64:
        t = t.long()
    return t.contiguous()


SMALL_R_TILES = 32     # below this many 128-row tiles the vocabulary-parallel GEMM-epilogue head is used


def _few_rows(R: int) -> bool:
    """The single-kernel head gives one CTA a 128-row tile and the whole vocabulary: with few
    rows (per-document evaluation, test-time training) that leaves most SMs idle, while the
    GEMM-epilogue head tiles the vocabulary across CTAs."""
    return (R + 127) // 128 < SMALL_R_TILES


def _lse_materialized(x, rowss, W_f, targets, eps, want_entropy, max_logit_bytes: int = 256 << 20):
    """PyTorch statement in row chunks (logits of one chunk at a time, at most ``max_logit_bytes``)."""
    R, D = x.shape
    V = W_f.shape[0]
    rc = max(1, min(R, max_logit_bytes // (4 * V)))
    t = targets.reshape(-1)
    outs = []
    for r0 in range(0, R, rc):
        xs = x[r0:r0 + rc].float()
        if rowss is not None:
            xs = xs * torch.rsqrt((xs * xs).sum(-1, keepdim=True) / D + eps)
        logits = xs @ W_f.float().t()
        lse = torch.logsumexp(logits, -1)
        rows = lse - logits.gather(1, t[r0:r0 + rc].view(-1, 1).long()).squeeze(1)
        ent = lse - (torch.softmax(logits, -1) * logits).sum(-1) if want_entropy else None
        outs.append((rows, lse, ent))
    rows = torch.cat([o[0] for o in outs])
    lse = torch.cat([o[1] for o in outs])
    if want_entropy:
        return rows, lse, torch.cat([o[2] for o in outs])
    return rows, lse


def lm_head_lse(x, rowss, W_f, targets, *, eps: float = EPS, want_entropy: bool = False,
                allow_materialized: bool = False):
    """Forward only: ``(loss_rows, lse)`` fp32 ``[R]`` (plus the softmax entropy
    when asked); no logits in memory.  Operands no kernel takes raise on a CUDA device unless
    ``allow_materialized`` (then the PyTorch statement runs in bounded row chunks)."""
    R, D = x.shape
    if (not fused_supported(x, W_f) or _few_rows(R)) and general_supported(x, W_f) and not want_entropy:
        return _lse_general(x, rowss, W_f, _prep(x, rowss, W_f, targets), eps)
    if not fused_supported(x, W_f):
        _refuse_unless_allowed(x, W_f, allow_materialized, "lm_head_lse" + (" (entropy)" if want_entropy else ""))
        return _lse_materialized(x, rowss, W_f, targets, eps, want_entropy)
    t = _prep(x, rowss, W_f, targets)
    lse = torch.empty(R, dtype=torch.float32, device=x.device)
    loss = torch.empty(R, dtype=torch.float32, device=x.device)
    ent = torch.empty(R, dtype=torch.float32, device=x.device) if want_entropy else None
    _lib.check(_lib.lib().ccb_lmhead_lse(x.data_ptr(), W_f.data_ptr(), _lib.ptr(rowss), eps,
                                         t.data_ptr(), lse.data_ptr(), loss.data_ptr(), _lib.ptr(ent),
                                         R, W_f.shape[0], D, _lib.stream_ptr()), "lmhead_lse")
    return (loss, lse, ent) if want_entropy else (loss, lse)


def default_row_chunks(R: int, V: int) -> int:
    """Row-chunk count for the dW kernel so (V/128 x chunks) work items divide
    evenly over the SMs."""
    sms = _lib.lib().ccb_num_sms() if _lib.available() else 148
    vt = max(V // 128, 1)
    mt = (R + 127) // 128
    best = 1
    for c in range(1, min(mt, 64) + 1):
        per = (mt + c - 1) // c
        if (mt + per - 1) // per != c:
            continue
        items = vt * c
        waves = (items + sms - 1) // sms
        eff = items / (waves * sms)
        if eff > 0.97 and c >= best:
            best = c
            if items >= 8 * sms:
                break
    return best


ONE_SWEEP = True      # module switch: lse + dX in one vocabulary sweep (see lm_head_train)


def lm_head_train(x, rowss, W_f, targets, *, gscale: float, rowweight=None, eps: float = EPS,
                  row_chunks: Optional[int] = None, lse: Optional[torch.Tensor] = None,
                  one_sweep: Optional[bool] = None, allow_materialized: bool = False,
                  want_dw: bool = True):
    """Loss and both gradients.  Returns ``(loss_rows, lse, dX bf16, dW_f_partials fp32 [C,V,D])``.

    ``want_dw=False`` skips the weight-gradient kernel and returns ``None`` in its
    place: test-time training adapts recurrence parameters only and needs ``dX``
    alone.

    ``dX`` is the gradient w.r.t. the un-normalised hidden state (RMSNorm
    backward applied); the partials sum to the gradient w.r.t. ``W_f``.

    ``one_sweep`` (default: the module switch ``ONE_SWEEP``) computes lse and
    ``dX`` in a single pass over the vocabulary: the softmax numerators are
    taken against a fixed per-row reference (the maximum of the row's first 32
    logits plus a 60-bit margin) instead of the true maximum, so no first pass
    is needed and nothing is ever rescaled; the row sum normalises the
    accumulated ``sum p W`` at the end.  Four logits-sized GEMMs per step
    instead of five.  Logits more than ~130 nats above that reference would
    saturate (clamped, never inf); more than ~46 nats below it flush to zero.
    """
    R, D = x.shape
    V = W_f.shape[0]
    if (not fused_supported(x, W_f) or (_few_rows(R) and one_sweep is None)) and general_supported(x, W_f):
        return _train_general(x, rowss, W_f, _prep(x, rowss, W_f, targets), gscale, rowweight, eps, lse, want_dw)
    if not fused_supported(x, W_f):
        _refuse_unless_allowed(x, W_f, allow_materialized, "lm_head_train")
        lr, lse, dX, dW = lm_head_reference(x, rowss, W_f, targets, gscale=gscale,
                                            rowweight=rowweight, eps=eps)
        return lr, lse, dX.to(x.dtype), dW.unsqueeze(0)
    t = _prep(x, rowss, W_f, targets)
    dev = x.device
    lse_given = lse is not None
    if not lse_given:
        lse = torch.empty(R, dtype=torch.float32, device=dev)
    loss = torch.empty(R, dtype=torch.float32, device=dev)
    dX = torch.empty_like(x)
    L = _lib.lib()
    _lib.check(L.ccb_lmhead_train(x.data_ptr(), W_f.data_ptr(), _lib.ptr(rowss), eps, t.data_ptr(),
                                  _lib.ptr(rowweight), gscale, lse.data_ptr(),
                                  1 if lse_given else (2 if (ONE_SWEEP if one_sweep is None else one_sweep) else 0),
                                  loss.data_ptr(), dX.data_ptr(), R, V, D, _lib.stream_ptr()),
               "lmhead_train")
    if not want_dw:
        return loss, lse, dX, None
    C = row_chunks or default_row_chunks(R, V)
    part = torch.empty(C, V, D, dtype=torch.float32, device=dev)
    _lib.check(L.ccb_lmhead_dw(x.data_ptr(), W_f.data_ptr(), _lib.ptr(rowss), eps, t.data_ptr(),
                               _lib.ptr(rowweight), gscale, lse.data_ptr(), part.data_ptr(), C, R, V,
                               D, _lib.stream_ptr()), "lmhead_dw")
    return loss, lse, dX, part
