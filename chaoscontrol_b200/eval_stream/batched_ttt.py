"""Score-then-adapt evaluation of many documents at once.

Per-document test-time training (``run_ttt_eval``: score a chunk, take one SGD
step on it, carry state and adapted weights to the document's next chunk, restore
the weights at the document's end; cf. scripts/run_exp20_eval.py:95-330 and
src/chaoscontrol/eval_stream/legality.py:14-275) is sequential inside a document
but independent across documents.  One document at a time leaves a B200 idle: a
256-token chunk is a few hundred microsecond-sized launches.  Here ``slots``
documents advance in lock step, one chunk each per step, as ONE batch:

* the adapted parameters exist once per slot: ``log_a`` as ``[L, slots, D]`` and
  the delta projection as ``[L, slots, D, D]``; everything else is shared and frozen;
* the three shared content projections are one GEMM over all rows, the delta
  projection is a batched GEMM with a different weight per slot, the scan kernel
  reads one decay vector per batch row;
* one forward serves both purposes: its per-row CE under the pre-update weights is
  the chunk's score, and its backward (input gradients only; no shared-weight
  gradient is ever formed) gives every slot's own ``d log_a`` and ``d delta_proj``;
* a slot whose document ends takes the next document at the next step (its state is
  zeroed and its parameters reset to the base weights by a per-slot flag), so the
  batch stays full until the queue drains;
* the whole pass is planned on the host up front (which document, which chunk, in
  which slot at which step), uploaded once, and each step is one replay of a CUDA
  graph that reads its row of the plan through a device-side step counter.

Supported setting: SGD, one step per chunk, ``reset`` persistence, adapt set
``log_a`` / ``delta_proj`` / ``log_a+delta_proj`` -- the setting of the reference's
headline TTT runs.  Anything else goes through ``run_ttt_eval``.
"""
from __future__ import annotations

import time
from typing import Optional, Sequence

import numpy as np
import torch
import torch.nn as nn

from ..ops import lm_head as LH
from ..ops import trunk as T
from ..ops.gemm import EPI_DSILU, EPI_RESID_SS, EPI_RMSBWD, EPI_ROWSCALE_SILU, gemm
from ..ops.scan import scan_fused_bwd, scan_fused_fwd, scan_fused_reference

SUPPORTED_ADAPT_SETS = ("log_a", "delta_proj", "log_a+delta_proj")
EPS = T.EPS


# ---------------------------------------------------------------------------
# host-side plan
# ---------------------------------------------------------------------------
def plan_slots(doc_lens: Sequence[int], slots: int, chunk: int):
    """Assign every (document, chunk) to a (step, slot).

    Documents are taken longest first; a free slot takes the next document at
    the step after its previous one ended.  Returns ``(start_step [n], slot [n],
    n_steps)`` for the documents with at least two tokens (others get -1)."""
    lens = np.asarray(doc_lens, dtype=np.int64)
    n_chunks = np.where(lens >= 2, (np.maximum(lens - 1, 0) + chunk - 1) // chunk, 0)
    order = np.argsort(-n_chunks, kind="stable")
    free_at = np.zeros(slots, dtype=np.int64)
    start = np.full(lens.size, -1, dtype=np.int64)
    slot = np.full(lens.size, -1, dtype=np.int64)
    for d in order:
        if n_chunks[d] == 0:
            continue
        s = int(np.argmin(free_at))
        start[d], slot[d] = free_at[s], s
        free_at[s] += n_chunks[d]
    return start, slot, int(free_at.max()) if lens.size else 0


def build_plan(docs_tokens: Sequence, slots: int, chunk: int) -> np.ndarray:
    """``int32 [steps, slots, chunk + 4]``: ``chunk + 1`` token ids (zero padded),
    the number of valid targets, a new-document flag, and the document's index
    (``len(docs)`` for an idle slot)."""
    lens = [len(t) for t in docs_tokens]
    start, slot, steps = plan_slots(lens, slots, chunk)
    C = chunk
    plan = np.zeros((max(steps, 1), slots, C + 4), dtype=np.int32)
    plan[:, :, C + 3] = len(docs_tokens)
    for d, toks in enumerate(docs_tokens):
        if start[d] < 0:
            continue
        a = np.asarray(toks, dtype=np.int32)
        n = a.size
        k = (n - 1 + C - 1) // C
        padded = np.zeros(k * C + 1, dtype=np.int32)
        padded[:n] = a
        rows = plan[start[d]: start[d] + k, slot[d]]
        rows[:, :C] = padded[: k * C].reshape(k, C)
        rows[:, C] = padded[C::C][:k]
        valid = np.minimum(C, (n - 1) - C * np.arange(k))
        rows[:, C + 1] = valid
        rows[0, C + 2] = 1
        rows[:, C + 3] = d
    return plan


# ---------------------------------------------------------------------------
# the batched step
# ---------------------------------------------------------------------------
class BatchedTTT:
    def __init__(self, model: nn.Module, *, adapt_set: str = "log_a+delta_proj", chunk_size: int = 256,
                 slots: int = 64, lr: float = 0.064, use_graph: Optional[bool] = None) -> None:
        if adapt_set not in SUPPORTED_ADAPT_SETS:
            raise ValueError(f"BatchedTTT adapts {SUPPORTED_ADAPT_SETS}, not {adapt_set!r}")
        if not self.supported(model):
            raise ValueError("BatchedTTT needs a bare-SSM CareStudentLM with full-rank delta projections")
        self.model, self.C, self.B, self.lr = model, int(chunk_size), int(slots), float(lr)
        self.adapt_log_a = "log_a" in adapt_set
        self.adapt_delta = "delta_proj" in adapt_set
        E = model.embed.weight
        self.device, self.dtype = E.device, E.dtype
        self.cuda = E.is_cuda
        self.use_graph = self.cuda if use_graph is None else bool(use_graph and self.cuda)
        L, D, B = len(model.layers), model.dim, self.B
        self.L, self.D = L, D
        # shared, frozen weights in the form the kernels take them
        self.w = []
        for blk in model.layers:
            c = blk.core
            W3 = torch.cat([c.select_proj.weight, c.in_proj.weight, c.gate_proj.weight], 0).detach().contiguous()
            self.w.append(dict(W3=W3, Wo=c.out_proj.weight.detach().contiguous(),
                               Wfc_f=T.fold_colscale(blk.ff.fc.weight.detach().contiguous(),
                                                     blk.ff_norm.weight.detach()),
                               Wproj=blk.ff.proj.weight.detach().contiguous(),
                               wn1=blk.input_norm.weight.detach().contiguous()))
        self.W_head = T.fold_colscale(model.lm_head.weight.detach().contiguous(), model.final_norm.weight.detach())
        self.head_eps = float(model.final_norm.eps)
        self.base_la = torch.stack([blk.core.log_a.detach() for blk in model.layers])                # [L, D]
        self.base_Wd = torch.stack([blk.core.delta_proj.weight.detach() for blk in model.layers])    # [L, D, D]
        # per-slot adapted parameters, carried state, accumulators
        self.la = self.base_la[:, None, :].repeat(1, B, 1).contiguous()                              # [L, B, D]
        self.Wd = self.base_Wd[:, None].repeat(1, B, 1, 1).contiguous()                              # [L, B, D, D]
        self.g_la = torch.zeros(L, B, D, dtype=torch.float32, device=self.device)
        self.g_Wd = torch.zeros(L, B, D, D, dtype=torch.float32, device=self.device)
        self.h = torch.zeros(L, B, D, dtype=torch.float32, device=self.device)
        self.step_idx = torch.zeros(1, dtype=torch.long, device=self.device)
        self.plan_dev: Optional[torch.Tensor] = None
        self.doc_ce: Optional[torch.Tensor] = None
        self.graph = None
        self.replays = self.captures = 0

    @staticmethod
    def supported(model: nn.Module) -> bool:
        if not hasattr(model, "layers") or not hasattr(model, "lm_head"):
            return False
        if not getattr(model, "_is_bare_ssm", lambda: False)():
            return False
        for blk in model.layers:
            c = blk.core
            if type(getattr(c, "delta_proj", None)) is not nn.Linear or c.delta_proj.weight.shape != (model.dim,
                                                                                                      model.dim):
                return False
        E = model.embed.weight
        if E.is_cuda:
            fn = getattr(model, "kernel_trunk_supported", None)
            return bool(fn and fn() and LH.kernel_supported(E.new_empty(1, model.dim), model.lm_head.weight))
        return True

    # ------------------------------------------------------------------
    def _rms_fwd(self, x, wn):
        """``x * rsqrt(mean x^2 + eps) * wn`` and the per-row ``rsqrt`` factor."""
        if self.cuda:
            from ..ops import _lib
            R, D = x.shape
            y = torch.empty_like(x)
            inv = torch.empty(R, dtype=torch.float32, device=x.device)
            _lib.check(_lib.lib().ccb_rmsnorm_fwd(x.data_ptr(), None, wn.data_ptr(), y.data_ptr(), None,
                                                  inv.data_ptr(), R, D, EPS, _lib.stream_ptr()), "rmsnorm_fwd")
            return y, inv
        xf = x.float()
        inv = torch.rsqrt((xf * xf).mean(-1) + EPS)
        return (xf * inv[:, None] * wn.float()).to(x.dtype), inv

    def _rms_bwd(self, x, wn, go, inv):
        if self.cuda:
            from ..ops import _lib
            R, D = x.shape
            gx = torch.empty_like(x)
            nb = int(_lib.lib().ccb_rmsnorm_bwd_blocks(R))
            part = torch.empty(nb, D, dtype=torch.float32, device=x.device)
            _lib.check(_lib.lib().ccb_rmsnorm_bwd(x.data_ptr(), wn.data_ptr(), go.data_ptr(), inv.data_ptr(),
                                                  gx.data_ptr(), part.data_ptr(), None, R, D, _lib.stream_ptr()),
                       "rmsnorm_bwd")
            return gx
        xf, g = x.float(), go.float() * wn.float()
        coef = (g * xf).sum(-1, keepdim=True) * (inv ** 3)[:, None] / x.shape[1]
        return (g * inv[:, None] - xf * coef).to(x.dtype)

    def _scan_fwd(self, P, la32, h0):
        B, C, D = self.B, self.C, self.D
        if self.cuda:
            return scan_fused_fwd(P, la32, h0, B, C, D, save_h=True)
        y, h, hT = scan_fused_reference(P, la32, h0, B, C, D)
        return y.to(P.dtype), h.to(P.dtype), hT

    def _scan_bwd(self, P, la32, h0, h, dy):
        B, C, D = self.B, self.C, self.D
        if self.cuda:
            dP, dla, _ = scan_fused_bwd(P, la32, h0, h, dy, None, None, 1.0 / D, EPS, B, C, D)
            return dP, dla
        with torch.enable_grad():
            Pr = P.detach().float().requires_grad_(True)
            lar = la32.detach().clone().requires_grad_(True)
            y, _, _ = scan_fused_reference(Pr, lar, h0, B, C, D)
            gP, gla = torch.autograd.grad((y * dy.float()).sum(), [Pr, lar])
        return gP.to(P.dtype), gla

    # ------------------------------------------------------------------
    @torch.no_grad()
    def _body(self) -> None:
        """One step of every slot: score, backward, SGD update, state carry."""
        B, C, D, L = self.B, self.C, self.D, self.L
        R = B * C
        row = self.plan_dev.index_select(0, self.step_idx)[0]              # [B, C + 4]
        tok = row[:, : C + 1]
        n_valid, fresh, doc = row[:, C + 1], row[:, C + 2].bool(), row[:, C + 3].long()
        # a slot that starts a document: zero state, base weights
        torch.where(fresh[None, :, None], self.h.new_zeros(()), self.h, out=self.h)
        torch.where(fresh[None, :, None], self.base_la[:, None, :], self.la, out=self.la)
        torch.where(fresh[None, :, None, None], self.base_Wd[:, None], self.Wd, out=self.Wd)
        la32 = self.la.float()
        inputs = tok[:, :C].contiguous()
        targets = tok[:, 1:].contiguous().long()
        mask = (torch.arange(C, device=self.device)[None, :] < n_valid[:, None]).float().reshape(-1)

        x, ss = T.embed_fwd(inputs, self.model.embed.weight)
        ctxs = []
        for l in range(L):
            w = self.w[l]
            xn, inv = self._rms_fwd(x, w["wn1"])
            P = torch.empty(R, 4 * D, dtype=x.dtype, device=x.device)
            gemm(xn, w["W3"], out=P[:, : 3 * D])
            gemm(xn.view(B, C, D), self.Wd[l], out=P.view(B, C, 4 * D)[:, :, 3 * D:])
            h0 = self.h[l].clone()
            y, hs, hT = self._scan_fwd(P, la32[l], h0)
            self.h[l].copy_(hT)
            ss2 = torch.empty(R, dtype=torch.float32, device=x.device)
            x2 = gemm(y, w["Wo"], epi=EPI_RESID_SS, r1=x, ss_out=ss2)
            f = torch.empty(R, w["Wfc_f"].shape[0], dtype=x.dtype, device=x.device)
            u = gemm(x2, w["Wfc_f"], epi=EPI_ROWSCALE_SILU, rowss=ss2, inv_dim=1.0 / D, eps=EPS, c2=f)
            ss3 = torch.empty(R, dtype=torch.float32, device=x.device)
            x3 = gemm(f, w["Wproj"], epi=EPI_RESID_SS, r1=x2, ss_out=ss3)
            ctxs.append((x, xn, inv, P, hs, h0, x2, ss2, u))
            x, ss = x3, ss3

        rows, _lse, dx, _ = LH.lm_head_train(x, ss, self.W_head, targets.reshape(-1), gscale=1.0, rowweight=mask,
                                             eps=self.head_eps, want_dw=False)
        chunk_ce = (rows.float() * mask).view(B, C).sum(1)
        self.doc_ce.index_add_(0, doc, chunk_ce.double())
        dx = dx.to(x.dtype)

        for l in reversed(range(L)):
            w = self.w[l]
            x0, xn, inv, P, hs, h0, x2, ss2, u = ctxs[l]
            du = gemm(dx, w["Wproj"], b_mn=True, epi=EPI_DSILU, r1=u, rowss=ss2, inv_dim=1.0 / D, eps=EPS)
            dx2 = gemm(du, w["Wfc_f"], b_mn=True, epi=EPI_RMSBWD, r1=x2, r2=dx, rowss=ss2, inv_dim=1.0 / D, eps=EPS)
            dy = gemm(dx2, w["Wo"], b_mn=True)
            dP, dla = self._scan_bwd(P, la32[l], h0, hs, dy)
            self.g_la[l].copy_(dla)
            if self.adapt_delta:
                gemm(dP.view(B, C, 4 * D)[:, :, 3 * D:], xn.view(B, C, D), a_mn=True, b_mn=True,
                     out=self.g_Wd[l], out_dtype=torch.float32)
            if l > 0:
                dxn = gemm(dP[:, : 3 * D], w["W3"], b_mn=True)
                dxn = gemm(dP.view(B, C, 4 * D)[:, :, 3 * D:], self.Wd[l], b_mn=True, cin=dxn.view(B, C, D),
                           beta=1.0).view(R, D)
                dx = self._rms_bwd(x0, w["wn1"], dxn, inv) + dx2
            ctxs[l] = None

        # p -= lr * grad, the gradient first rounded to the parameter dtype as autograd would hand it over
        if self.adapt_log_a:
            self.la.add_(self.g_la.to(self.la.dtype), alpha=-self.lr)
        if self.adapt_delta:
            self.Wd.add_(self.g_Wd.to(self.Wd.dtype), alpha=-self.lr)
        self.step_idx.add_(1)

    # ------------------------------------------------------------------
    def _capture(self) -> None:
        dev = self.device
        keep = (self.step_idx.clone(), self.h.clone(), self.la.clone(), self.Wd.clone(), self.doc_ce.clone())
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.step_idx.zero_()
                self._body()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.step_idx.zero_()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            self._body()
        self.graph = g
        self.captures += 1
        for dst, src in zip((self.step_idx, self.h, self.la, self.Wd, self.doc_ce), keep):
            dst.copy_(src)

    def upload(self, docs_tokens: Sequence) -> dict:
        """Plan the pass on the host and put the plan on the device (one pinned copy)."""
        n = len(docs_tokens)
        plan = torch.from_numpy(build_plan(docs_tokens, self.B, self.C))
        steps = plan.shape[0]
        if self.cuda:
            plan = plan.pin_memory()
        regrow = self.plan_dev is None or self.plan_dev.shape[0] < steps
        if regrow:
            self.plan_dev = torch.zeros(steps, self.B, self.C + 4, dtype=torch.int32, device=self.device)
        self.plan_dev[:steps].copy_(plan, non_blocking=True)
        if self.doc_ce is None or self.doc_ce.numel() < n + 1:
            self.doc_ce = torch.zeros(n + 1, dtype=torch.float64, device=self.device)
            regrow = True
        if self.use_graph and (self.graph is None or regrow):
            self.doc_ce.zero_()
            self._capture()
        self._n, self._steps = n, steps
        return {"steps": steps, "h2d_bytes": int(plan.numel() * 4)}

    def execute(self) -> torch.Tensor:
        """Run the uploaded plan from its first step.  Returns the summed CE per document
        (fp64, on the device); nothing is read back."""
        self.doc_ce.zero_()
        self.step_idx.zero_()
        for _ in range(self._steps):
            if self.use_graph:
                self.graph.replay()
            else:
                self._body()
        self.replays += self._steps
        return self.doc_ce[: self._n].clone()

    def run(self, docs_tokens: Sequence) -> tuple[torch.Tensor, dict]:
        """Score-then-adapt every document once.  ``docs_tokens``: sequences of token
        ids on the host.  Returns ``(summed CE per document, fp64 on the device, info)``."""
        info = self.upload(docs_tokens)
        return self.execute(), info


def pick_slots(doc_lens: Sequence[int], chunk: int, *, lo: int = 8, hi: int = 128) -> int:
    """Slots that keep the batch full: the pass can never be shorter than its longest
    document, so more slots than ``total chunks / longest document's chunks`` only idle."""
    ch = [(max(n - 1, 0) + chunk - 1) // chunk for n in doc_lens if n >= 2]
    if not ch:
        return lo
    want = -(-sum(ch) // max(ch))
    return int(min(hi, max(lo, -(-want // 8) * 8)))


def run_ttt_eval_batched(model: nn.Module, docs, *, adapt_set: str = "log_a+delta_proj", chunk_size: int = 256,
                         eval_lr: float = 0.064, slots: Optional[int] = None, max_docs: Optional[int] = None,
                         runner: Optional[BatchedTTT] = None, use_graph: Optional[bool] = None) -> dict:
    """``run_ttt_eval`` (SGD, one step per chunk, ``reset`` persistence, weights restored
    per document) with ``slots`` documents advancing together (default: :func:`pick_slots`);
    same result keys.  Pass the returned ``runner`` back in to reuse its captured graph."""
    from ..scoring import compute_bpb
    recs = [r for r in docs][: max_docs]
    recs = [r for r in recs if len(r.tokens) >= 2]
    t0 = time.perf_counter()
    was_training = model.training
    model.eval()
    try:
        if runner is None and slots is None:
            slots = pick_slots([len(r.tokens) for r in recs], chunk_size)
        rn = runner or BatchedTTT(model, adapt_set=adapt_set, chunk_size=chunk_size, slots=slots, lr=eval_lr,
                                  use_graph=use_graph)
        ce_dev, info = rn.run([r.tokens for r in recs])
        ce_all = ce_dev.cpu()
    finally:
        model.train(was_training)
    elapsed = time.perf_counter() - t0
    toks = [len(r.tokens) - 1 for r in recs]
    n_chunks = int(sum((t + chunk_size - 1) // chunk_size for t in toks))
    tot_ce, tot_tok, tot_bytes = float(ce_all.sum()), int(sum(toks)), int(sum(r.raw_bytes for r in recs))
    return {"docs_scored": len(recs), "chunks_scored": n_chunks, "tokens_scored": tot_tok, "adapt_steps": n_chunks,
            "elapsed_seconds": elapsed, "chunk_size": chunk_size, "total_ce_nats": tot_ce,
            "total_raw_bytes": tot_bytes, "bpb": compute_bpb(tot_ce, tot_bytes),
            "mean_ce": tot_ce / max(tot_tok, 1), "tokens_per_s": tot_tok / elapsed if elapsed > 0 else 0.0,
            "adapt_set": adapt_set, "persistence_mode": "reset", "slots": rn.B, "batched_steps": info["steps"],
            "graph_replays": info["steps"] if rn.use_graph else 0, "h2d_bytes": info["h2d_bytes"],
            "per_doc_ce": {int(r.doc_id): float(c) for r, c in zip(recs, ce_all.tolist())}, "runner": rn}
