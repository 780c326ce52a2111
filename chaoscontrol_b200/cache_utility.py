"""Memory-utility oracle for cache-reweighted continuation training (behaviour of
src/chaoscontrol/cache_utility.py:55-1286).

For every target token the oracle measures ``utility = NLL(memory off) -
NLL(memory forced on)`` against one stable snapshot of the episodic store and
turns it into

* a probability target + confidence for the read-controller head (optionally
  net of a shadow price kept by a primal-dual budget tracker),
* a positive-only, mean-one weight for the language-model loss,
* per-channel "plasticity" evidence (does a channel move more when memory
  actually helps?), and
* write scores for the tokens appended to the store afterwards, optionally
  vetted by an LM-head-gradient conflict sensor.

On a B200 the per-token NLL comes from the fused tcgen05 LM-head kernel (no
logits tensor, so nothing to chunk); elsewhere a time-chunked PyTorch statement
bounds the logits buffer.  The off / on streams run stacked through the
recurrence in one pass when the model offers ``encode_paired_for_score``.
"""
from __future__ import annotations

import contextlib
import json
import math
import time
from pathlib import Path
from typing import Any, Optional

import torch
import torch.nn.functional as F

from .ops import lm_head as LH
from .ops.trunk import fold_colscale

__all__ = ["alpha_ramp", "assign_memory_credit", "chunked_nll_from_hidden",
           "plasticity_budget_from_hidden_delta", "positive_only_lm_weight", "rank3_score_batch_causal",
           "ScarcityAwareMemoryOptimizer", "CrctGradientConflictMonitor", "LOSS_REWEIGHT_DIAGNOSTIC_NAMES"]

NLL_CHUNK_BUDGET_BYTES = 1 << 30          # logits buffer bound on the training ranks
ORACLE_NLL_CHUNK_BUDGET_BYTES = 2 << 30   # the oracle rank holds no optimizer state

LOSS_REWEIGHT_DIAGNOSTIC_NAMES: tuple[str, ...] = (
    "valid_tokens", "plain_nll_mean", "weighted_nll_mean", "weighted_minus_plain", "weighted_rel_delta",
    "loss_weight_abs_dev_mean", "loss_weight_std", "loss_weight_max")


# ---------------------------------------------------------------- loss weights
def positive_only_lm_weight(utility: torch.Tensor, mask: torch.Tensor, *, tau: float, strength: float,
                            w_max: float) -> torch.Tensor:
    """``clamp(1 + strength * relu(tanh(u / tau)), 1, w_max)`` normalised to mean one
    over valid positions, zero elsewhere.  Tokens that memory hurt are never
    down-weighted below the neutral raw weight."""
    m = mask.bool()
    w = (1.0 + strength * torch.tanh(utility.float() / tau).clamp_min(0.0)).clamp(1.0, w_max)
    mf = m.to(w.dtype)
    n = mf.sum()
    mean = torch.where(n > 0, (w * mf).sum() / n.clamp_min(1.0), torch.ones_like(n)).clamp_min(1e-8)
    return w / mean * mf


def _loss_reweight_diagnostics(*, nll_off: torch.Tensor, loss_weight: torch.Tensor,
                               mask: torch.Tensor) -> torch.Tensor:
    """CPU fp32 vector ordered as ``LOSS_REWEIGHT_DIAGNOSTIC_NAMES`` (one device->host copy)."""
    with torch.no_grad():
        m = mask.bool().float()
        n = m.sum()
        nll, w = nll_off.detach().float(), loss_weight.detach().float()
        nc = n.clamp_min(1.0)
        plain = (nll * m).sum() / nc
        weighted = (nll * w).sum() / w.sum().clamp_min(1e-8)
        wm = (w * m).sum() / nc
        var = (((w - wm) * m) ** 2).sum() / nc
        vals = torch.stack([n, plain, weighted, weighted - plain,
                            (weighted - plain) / plain.abs().clamp_min(1e-8),
                            ((w - 1.0).abs() * m).sum() / nc, var.sqrt(),
                            torch.where(m > 0, w, torch.full_like(w, -math.inf)).max()])
        vals = torch.where(n > 0, vals, torch.zeros_like(vals))
        return vals.float().cpu()


# ---------------------------------------------------------------- per-token NLL
@torch.inference_mode()
def chunked_nll_from_hidden(model: Any, hidden_states: torch.Tensor, targets: torch.Tensor, *,
                            chunk_size: int = 1024, chunk_budget_bytes: Optional[int] = None) -> torch.Tensor:
    """Per-token NLL ``[B, T]`` (fp32) through ``final_norm -> lm_head``.

    ``chunk_size`` is clamped so the fp32 logits of one time chunk
    (``B * chunk * V * 4`` bytes) stay under ``chunk_budget_bytes``.  The fused
    LM-head kernel never materialises logits, so it takes the whole batch in one
    launch and the clamp only governs the PyTorch path."""
    if chunk_size <= 0:
        raise ValueError(f"chunked_nll_from_hidden: chunk_size must be positive, got {chunk_size}")
    budget = NLL_CHUNK_BUDGET_BYTES if chunk_budget_bytes is None else int(chunk_budget_bytes)
    if budget <= 0:
        raise ValueError(f"chunked_nll_from_hidden: chunk_budget_bytes must be positive, got {budget}")
    B, T, D = hidden_states.shape
    head, norm = model.lm_head, model.final_norm
    V = head.out_features
    targets = targets.long()
    nw = getattr(norm, "weight", None)
    if (nw is not None and getattr(head, "bias", None) is None and hidden_states.is_cuda and
            LH.kernel_supported(hidden_states.new_empty(1, D, dtype=head.weight.dtype), head.weight)):
        x = hidden_states.to(head.weight.dtype).reshape(B * T, D).contiguous()
        ss = x.float().square().sum(-1)
        rows, _ = LH.lm_head_lse(x, ss, fold_colscale(head.weight, nw), targets.reshape(-1),
                                 eps=float(getattr(norm, "eps", 1e-6)))
        return rows.view(B, T)
    step = max(1, min(int(chunk_size), budget // max(1, B * V * 4)))
    out = torch.zeros(B, T, dtype=torch.float32, device=hidden_states.device)
    for s in range(0, T, step):
        e = min(T, s + step)
        logits = head(norm(hidden_states[:, s:e].to(head.weight.dtype))).float()
        out[:, s:e] = F.cross_entropy(logits.reshape(-1, V), targets[:, s:e].reshape(-1),
                                      reduction="none").view(B, e - s)
    return out


def alpha_ramp(step: int, total_steps: int, *, alpha_max: float) -> float:
    """``alpha_max * sigmoid(8 * (step / total - 0.3))``; ``total_steps <= 0`` counts as finished."""
    progress = 1.0 if total_steps <= 0 else step / float(total_steps)
    return alpha_max / (1.0 + math.exp(-8.0 * (progress - 0.3)))


# ---------------------------------------------------------------- budgeted targets
def _bid(net: torch.Tensor, tau: float) -> tuple[torch.Tensor, torch.Tensor]:
    net = net.float()
    return torch.sigmoid(net / tau).clamp(0.05, 0.95).detach(), torch.tanh(net.abs() / tau).detach()


class ScarcityAwareMemoryOptimizer:
    """Primal-dual shadow prices for memory reads and writes.  The controller is
    trained toward ``sigmoid((utility - price) / tau)``; each ``dual_step`` moves
    a price by ``dual_lr * (EMA(rate) - target_rate)`` within ``[0, max_price]``."""

    def __init__(self, *, tau: float = 0.10, target_read_rate: float = 0.25, target_write_rate: float = 0.10,
                 dual_lr: float = 0.01, ema_beta: float = 0.95, max_price: float = 0.50) -> None:
        self.tau, self.dual_lr = float(tau), float(dual_lr)
        self.target_read_rate, self.target_write_rate = float(target_read_rate), float(target_write_rate)
        self.ema_beta, self.max_price = float(ema_beta), float(max_price)
        self.read_price = self.write_price = 0.0
        self.read_rate_ema, self.write_rate_ema = self.target_read_rate, self.target_write_rate

    @torch.no_grad()
    def controller_target(self, utility: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``(target, confidence)``: bid probability clamped to [0.05, 0.95] and ``tanh(|net| / tau)``."""
        return _bid(utility.float() - self.read_price, self.tau)

    @torch.no_grad()
    def write_target(self, write_utility: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return _bid(write_utility.float() - self.write_price, self.tau)

    def _dual(self, price: float, ema: float, rate: float, target: float) -> tuple[float, float]:
        ema = self.ema_beta * ema + (1.0 - self.ema_beta) * float(rate)
        return float(min(max(price + self.dual_lr * (ema - target), 0.0), self.max_price)), ema

    @torch.no_grad()
    def dual_step(self, *, actual_read_rate: float, actual_write_rate: Optional[float] = None) -> None:
        self.read_price, self.read_rate_ema = self._dual(self.read_price, self.read_rate_ema, actual_read_rate,
                                                         self.target_read_rate)
        if actual_write_rate is not None:
            self.write_price, self.write_rate_ema = self._dual(self.write_price, self.write_rate_ema,
                                                               actual_write_rate, self.target_write_rate)


# ---------------------------------------------------------------- gradient-conflict sensor
class CrctGradientConflictMonitor:
    """Write-admission sensor.  For the tokens that would be appended to memory it
    forms the unit LM-head-input gradient ``(softmax(logits) - onehot(y)) @ W``,
    takes its cosine with an EMA of previously admitted gradients, scales the
    write score by an optional soft gate and sets it to ``-inf`` below the
    catastrophic threshold.  Utility, controller targets and LM weights are not
    touched."""

    def __init__(self, *, enabled: bool = True, ema_beta: float = 0.95, catastrophic_threshold: float = -0.90,
                 soft_gate_strength: float = 0.0, soft_gate_floor: float = 0.05,
                 trace_path: Optional[str] = None, trace_stride: int = 1, trace_max_rows: int = 0,
                 trace_flush_rows: int = 256, eps: float = 1e-8) -> None:
        self.enabled = bool(enabled)
        self.ema_beta = float(ema_beta)
        self.catastrophic_threshold = float(catastrophic_threshold)
        self.soft_gate_strength = float(soft_gate_strength)
        self.soft_gate_floor = float(soft_gate_floor)
        self.trace_path = Path(str(trace_path)) if trace_path not in (None, "") else None
        self.trace_stride = max(1, int(trace_stride))
        self.trace_max_rows = max(0, int(trace_max_rows))
        self.trace_flush_rows = max(1, int(trace_flush_rows))
        self.eps = float(eps)
        self._ema: Optional[torch.Tensor] = None
        self._trace_buffer: list[str] = []
        self._diag: dict[str, Any] = dict(
            enabled=self.enabled, ema_beta=self.ema_beta, catastrophic_threshold=self.catastrophic_threshold,
            soft_gate_strength=self.soft_gate_strength, soft_gate_floor=self.soft_gate_floor,
            trace_enabled=self.trace_path is not None, trace_path=str(self.trace_path or ""),
            trace_stride=self.trace_stride, trace_max_rows=self.trace_max_rows,
            trace_flush_rows=self.trace_flush_rows, trace_rows_written=0, trace_rows_dropped=0,
            trace_rows_buffered=0, trace_errors=0, last_trace_error="", calls=0, cold_start_calls=0,
            candidates_seen=0, candidates_compared=0, admitted_candidates=0,
            guardrail_suppressed_candidates=0, soft_gated_candidates=0, ema_updates=0, mean_conflict_sum=0.0,
            min_conflict=1.0, max_conflict=-1.0, last_conflict_mean=0.0, last_conflict_min=0.0,
            last_conflict_max=0.0, last_gate_mean=1.0, last_suppressed=0, last_admitted=0,
            last_write_token_limit=None, last_reason="")

    # -- pieces -----------------------------------------------------------
    @staticmethod
    def _candidates(utility: torch.Tensor, mask: torch.Tensor, max_tokens: Optional[int]) -> torch.Tensor:
        valid = mask.reshape(-1).bool().nonzero().reshape(-1)
        k = 0 if max_tokens is None else int(max_tokens)
        if valid.numel() == 0 or k <= 0 or k >= valid.numel():
            return valid
        scores = utility.detach().reshape(-1).float().index_select(0, valid)
        return valid.index_select(0, torch.topk(scores, k=k, sorted=False).indices)

    def _sketches(self, model: Any, hidden: torch.Tensor, targets: torch.Tensor,
                  selected: torch.Tensor) -> torch.Tensor:
        h = hidden.detach().reshape(-1, hidden.shape[-1]).index_select(0, selected)
        y = targets.detach().reshape(-1).index_select(0, selected).long()
        W = model.lm_head.weight.detach()
        err = torch.softmax(model.lm_head(model.final_norm(h.to(W.dtype))).float(), dim=-1)
        err.scatter_add_(1, y.view(-1, 1), torch.full((y.numel(), 1), -1.0, device=err.device))
        return F.normalize(err @ W.float(), dim=-1, eps=self.eps)

    def _fold_into_ema(self, sketches: torch.Tensor) -> None:
        mean = F.normalize(sketches.float().mean(0), dim=0, eps=self.eps)
        if self._ema is not None:
            mean = F.normalize(self.ema_beta * self._ema.to(mean.device) + (1.0 - self.ema_beta) * mean,
                               dim=0, eps=self.eps)
        self._ema = mean.detach().cpu()
        self._diag["ema_updates"] += 1

    # -- main entry -------------------------------------------------------
    @torch.no_grad()
    def apply_to_write_scores(self, *, model: Any, hidden: torch.Tensor, targets: torch.Tensor,
                              utility: torch.Tensor, mask: torch.Tensor, max_tokens: Optional[int],
                              step: Optional[int] = None) -> tuple[torch.Tensor, Optional[int]]:
        """``(write_score, write_token_limit)``; the limit shrinks when the guardrail
        leaves fewer safe candidates than ``max_tokens``."""
        d = self._diag
        if not self.enabled:
            return utility, max_tokens
        d["calls"] += 1
        selected = self._candidates(utility, mask, max_tokens)
        n = int(selected.numel())
        d["candidates_seen"] += n
        if n == 0:
            d["last_reason"] = "no_valid_candidates"
            d["last_write_token_limit"] = None if max_tokens is None else 0
            return utility, (None if max_tokens is None else 0)
        sk = self._sketches(model, hidden, targets, selected)
        if sk.numel() == 0:
            d["last_reason"] = "empty_sketch"
            return utility, max_tokens
        dev = utility.device
        score = utility.detach().clone()
        gate = torch.ones(n, device=dev)
        suppressed = torch.zeros(n, dtype=torch.bool, device=dev)
        had_reference = self._ema is not None
        if not had_reference:
            d["cold_start_calls"] += 1
            conflict = torch.zeros(n, device=dev)
        else:
            ref = F.normalize(self._ema.to(device=sk.device, dtype=torch.float32), dim=0, eps=self.eps)
            conflict = (sk @ ref).clamp(-1.0, 1.0)
            d["candidates_compared"] += n
            suppressed = conflict < self.catastrophic_threshold
            if self.soft_gate_strength > 0.0:
                gate = (1.0 - self.soft_gate_strength * (-conflict).clamp(0.0, 1.0)).clamp(self.soft_gate_floor, 1.0)
                d["soft_gated_candidates"] += int((gate < 1.0).sum())
            flat = score.view(-1)
            vals = flat.index_select(0, selected) * gate.to(flat.dtype)
            flat.index_copy_(0, selected, vals.masked_fill(suppressed, -math.inf))
        keep = ~suppressed
        admitted, n_supp = int(keep.sum()), int(suppressed.sum())
        d["admitted_candidates"] += admitted
        d["guardrail_suppressed_candidates"] += n_supp
        d["last_gate_mean"] = float(gate.mean())
        cm, cmin, cmax = float(conflict.mean()), float(conflict.min()), float(conflict.max())
        d["mean_conflict_sum"] += cm
        d["min_conflict"], d["max_conflict"] = min(d["min_conflict"], cmin), max(d["max_conflict"], cmax)
        d["last_conflict_mean"], d["last_conflict_min"], d["last_conflict_max"] = cm, cmin, cmax
        if admitted > 0:
            self._fold_into_ema(sk[keep])
        elif not had_reference:
            self._fold_into_ema(sk)
        limit = admitted if max_tokens is None else min(int(max_tokens), admitted)
        d["last_write_token_limit"], d["last_suppressed"], d["last_admitted"] = limit, n_supp, admitted
        if n_supp:
            d["last_reason"] = "guardrail_suppressed"
        elif self.soft_gate_strength > 0.0 and bool((gate < 1.0).any()):
            d["last_reason"] = "soft_gated"
        else:
            d["last_reason"] = "observed" if had_reference else "cold_start"
        self._trace(step, selected, targets, utility, conflict, gate, suppressed, max_tokens, had_reference)
        return score, limit

    # -- reporting --------------------------------------------------------
    def diagnostics(self) -> dict[str, Any]:
        self.flush_trace()
        out = dict(self._diag)
        out["trace_rows_buffered"] = len(self._trace_buffer)
        out["mean_conflict_per_call"] = out["mean_conflict_sum"] / out["calls"] if out["calls"] else 0.0
        if not out["candidates_compared"]:
            out["min_conflict"] = out["max_conflict"] = 0.0
        out["has_reference"] = self._ema is not None
        return out

    def flush_trace(self) -> None:
        if self.trace_path is None or not self._trace_buffer:
            return
        try:
            self.trace_path.parent.mkdir(parents=True, exist_ok=True)
            with self.trace_path.open("a", encoding="utf-8") as fh:
                fh.writelines(self._trace_buffer)
            self._trace_buffer.clear()
            self._diag["trace_rows_buffered"] = 0
        except OSError as exc:
            self._diag["trace_errors"] += 1
            self._diag["last_trace_error"] = f"{type(exc).__name__}: {exc}"

    def _trace(self, step, selected, targets, utility, conflict, gate, suppressed, max_tokens, had_reference):
        d = self._diag
        if self.trace_path is None or (d["calls"] - 1) % self.trace_stride:
            return
        T = int(targets.shape[1]) if targets.ndim >= 2 else int(targets.numel())
        T = max(T, 1)
        sel = selected.cpu()
        cols = zip(sel.tolist(), conflict.cpu().tolist(), gate.cpu().tolist(), suppressed.cpu().tolist(),
                   utility.detach().reshape(-1).float().cpu()[sel].tolist(),
                   targets.detach().reshape(-1).long().cpu()[sel].tolist())
        for rank, (idx, cos, g, supp, u, tok) in enumerate(cols):
            if self.trace_max_rows and d["trace_rows_written"] >= self.trace_max_rows:
                d["trace_rows_dropped"] += 1
                continue
            row = {"row_type": "crct_gradient_conflict_candidate", "step": None if step is None else int(step),
                   "call_index": d["calls"], "candidate_rank": rank, "candidate_flat_index": idx,
                   "batch_index": idx // T, "token_pos": idx % T, "token_id": tok, "utility": u,
                   "conflict_cos": cos, "gate": g, "suppressed": bool(supp),
                   "reason": d["last_reason"] if supp else "admitted",
                   "max_tokens": None if max_tokens is None else int(max_tokens),
                   "catastrophic_threshold": self.catastrophic_threshold,
                   "soft_gate_strength": self.soft_gate_strength, "has_reference": bool(had_reference)}
            self._trace_buffer.append(json.dumps(row, separators=(",", ":")) + "\n")
            d["trace_rows_written"] += 1
        d["trace_rows_buffered"] = len(self._trace_buffer)
        if len(self._trace_buffer) >= self.trace_flush_rows:
            self.flush_trace()


# ---------------------------------------------------------------- credit / plasticity
@torch.no_grad()
def assign_memory_credit(entry_credit: torch.Tensor, entry_debit: torch.Tensor, entry_ids: torch.Tensor,
                         weights: torch.Tensor, utility: torch.Tensor) -> None:
    """Scatter ``weights * relu(+-utility)`` of the K entries read per token
    (``entry_ids`` / ``weights`` are ``[B, T, K]``) into the 1-D accumulators in place."""
    ids = entry_ids.reshape(-1).long()
    w = weights.float()
    u = utility.float().unsqueeze(-1)
    entry_credit.scatter_add_(0, ids, (w * u.clamp_min(0.0)).reshape(-1).to(entry_credit.dtype))
    entry_debit.scatter_add_(0, ids, (w * (-u).clamp_min(0.0)).reshape(-1).to(entry_debit.dtype))


def plasticity_budget_from_hidden_delta(*, h_off: torch.Tensor, h_mem: torch.Tensor, utility: torch.Tensor,
                                        mask: torch.Tensor, tau: float, eps: float = 1e-6
                                        ) -> dict[str, torch.Tensor]:
    """Per-channel Pearson correlation, over valid tokens, between
    ``|h_mem - h_off|[..., c]`` and ``relu(utility)`` (``plasticity_coverage`` in
    [-1, 1]); ``plasticity_confidence = |coverage| * tanh(rms(relu(utility)) / tau)``
    and ``plasticity_budget = relu(coverage) * confidence``.

    The first moments are one [2, N] x [N, D] product (ones row and utility row
    against the masked residual); second moments are reduced in row blocks so no
    second [N, D] buffer is alive."""
    if h_off.shape != h_mem.shape:
        raise ValueError(f"h_off and h_mem must have identical shape, got {tuple(h_off.shape)} and "
                         f"{tuple(h_mem.shape)}")
    if h_off.dim() != 3:
        raise ValueError(f"hidden tensors must be (B, T, D), got {tuple(h_off.shape)}")
    if utility.shape != h_off.shape[:2] or mask.shape != h_off.shape[:2]:
        raise ValueError("utility and mask must match hidden batch/time shape; got "
                         f"utility={tuple(utility.shape)} mask={tuple(mask.shape)} hidden={tuple(h_off.shape)}")
    w = mask.detach().float().reshape(-1)
    y = utility.detach().float().reshape(-1).clamp_min(0.0) * w
    n = w.sum().clamp_min(1.0)
    x = (h_mem.detach().float() - h_off.detach().float()).abs_().flatten(0, 1)
    x.mul_(w.unsqueeze(-1))
    first = torch.stack([w, y], 0) @ x                                         # [2, D]: sum x, sum xy
    xx = torch.zeros(x.shape[1], device=x.device, dtype=x.dtype)
    for s in range(0, x.shape[0], 65_536):
        blk = x[s:s + 65_536]
        xx.add_(torch.einsum("nd,nd->d", blk, blk))
    yy = torch.dot(y, y)
    x_mean, y_mean = first[0] / n, y.sum() / n
    cov = first[1] / n - x_mean * y_mean
    x_var = (xx / n - x_mean * x_mean).clamp_min(0.0)
    y_var = (yy / n - y_mean * y_mean).clamp_min(0.0)
    coverage = (cov / (x_var * y_var).clamp_min(float(eps)).sqrt()).clamp(-1.0, 1.0)
    confidence = (coverage.abs() * torch.tanh((yy / n).sqrt() / max(float(tau), float(eps)))).clamp(0.0, 1.0)
    return {"plasticity_coverage": coverage.detach(), "plasticity_confidence": confidence.detach(),
            "plasticity_budget": (coverage.clamp_min(0.0) * confidence).detach()}


# ---------------------------------------------------------------- the oracle
def _compact_residual(residual: torch.Tensor, batch_size: int) -> torch.Tensor:
    """Memory packets travel as ``[B, 1, D]``; ``[B, D]`` is accepted and unsqueezed."""
    ok = (residual.dim() == 2 or (residual.dim() == 3 and residual.shape[1] == 1))
    if not ok:
        raise ValueError("memory_residual packets must be compact with shape (B, D) or (B, 1, D); "
                         f"got {tuple(residual.shape)}")
    if residual.shape[0] != batch_size:
        raise ValueError(f"memory_residual packet batch mismatch: {tuple(residual.shape)} for batch {batch_size}")
    return residual if residual.dim() == 3 else residual.unsqueeze(1)


class _StageClock:
    """Stage timing with CUDA events (one synchronize at the end) or host time."""
    STAGES = ("encode_off", "encode_force_on", "nll_off", "nll_mem", "plasticity", "append_memory")

    def __init__(self, sink: Optional[dict], device: torch.device) -> None:
        self.sink = sink
        self.cuda = sink is not None and device.type == "cuda" and torch.cuda.is_available()
        self.marks: list[Any] = []
        self.mark()

    def mark(self) -> None:
        if self.sink is None:
            return
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append(ev)
        else:
            self.marks.append(time.perf_counter())

    def flush(self) -> None:
        if self.sink is None:
            return
        if self.cuda:
            torch.cuda.synchronize()
        for name, a, b in zip(self.STAGES, self.marks, self.marks[1:]):
            dt = a.elapsed_time(b) * 1e-3 if self.cuda else max(0.0, b - a)
            self.sink[name] = self.sink.get(name, 0.0) + float(dt)


def _autocast(device_type: str):
    return (torch.autocast(device_type, dtype=torch.bfloat16) if device_type in ("cuda", "cpu")
            else contextlib.nullcontext())


@torch.inference_mode()
def rank3_score_batch_causal(*, model: Any, cache: Any, input_ids: torch.Tensor, valid_mask: torch.Tensor,
                             scarcity_optimizer: Optional[ScarcityAwareMemoryOptimizer] = None,
                             tau: float = 0.10, strength: float = 0.10, w_max: float = 1.15,
                             update_model_memory_after: bool = False,
                             memory_write_tokens: Optional[int] = None,
                             gradient_conflict_monitor: Optional[CrctGradientConflictMonitor] = None,
                             step: Optional[int] = None,
                             record_stage_seconds: Optional[dict[str, float]] = None) -> dict[str, Any]:
    """Scores one batch against a stable memory snapshot.

    A cache transaction brackets the whole call: both streams read with the
    transaction's cut-off, and tokens appended afterwards (when
    ``update_model_memory_after``) carry event ids reserved past that cut-off, so
    they become visible only to later batches.  Returns ``utility``,
    ``controller_target``, ``confidence``, ``loss_weight`` (all ``[B, T-1]``, zero
    at invalid positions), ``loss_reweight_diagnostics``, the plasticity vectors,
    and when available ``memory_residual`` / ``memory_gate`` / ``write_score`` /
    ``memory_write_records``.  ``record_stage_seconds`` receives per-stage
    seconds and the problem shape."""
    txn = cache.begin_batch()
    x, y = input_ids[:, :-1], input_ids[:, 1:]
    mask = valid_mask[:, 1:].bool()
    B, T = x.shape
    V = int(getattr(getattr(model, "lm_head", None), "out_features", 0) or 0)
    clock = _StageClock(record_stage_seconds, input_ids.device)
    trace = bool(record_stage_seconds and record_stage_seconds.get("_trace_progress", False))

    def say(stage: str) -> None:
        if trace:
            print(f"[rank3-score-trace] step={-1 if step is None else int(step)} stage={stage} B={B} T={T} "
                  f"V={V} update_memory={bool(update_model_memory_after)}", flush=True)

    say("start")
    meta: Optional[dict] = None
    paired = getattr(model, "encode_paired_for_score", None)
    with _autocast(input_ids.device.type):
        if callable(paired):
            h_off, h_mem, meta = paired(x, cache_read_cutoff=txn.read_cutoff)
            clock.mark()
            clock.mark()
        else:
            h_off = model.encode(x, memory_mode="off", cache_read_cutoff=txn.read_cutoff)
            clock.mark()
            try:
                got = model.encode(x, memory_mode="force_on", cache_read_cutoff=txn.read_cutoff,
                                   return_memory_meta=True)
            except TypeError:
                got = model.encode(x, memory_mode="force_on", cache_read_cutoff=txn.read_cutoff)
            if isinstance(got, dict):
                h_mem = got["hidden"]
                meta = got.get("memory_meta") if isinstance(got.get("memory_meta"), dict) else None
            else:
                h_mem = got
            clock.mark()
    say("encoded")
    if record_stage_seconds is not None:
        chunk = max(1, min(1024, ORACLE_NLL_CHUNK_BUDGET_BYTES // max(1, B * max(V, 1) * 4)))
        record_stage_seconds.update({
            "_batch_size": float(B), "_seq_len": float(T), "_vocab_size": float(V),
            "_hidden_dim": float(h_off.shape[-1]), "_paired_encode": float(callable(paired)),
            "_nll_chunk_budget_bytes": float(ORACLE_NLL_CHUNK_BUDGET_BYTES), "_nll_effective_chunk": float(chunk),
            "_nll_chunks_per_pass": float(math.ceil(T / chunk))})
    nll_off = chunked_nll_from_hidden(model, h_off, y, chunk_budget_bytes=ORACLE_NLL_CHUNK_BUDGET_BYTES)
    clock.mark()
    nll_mem = chunked_nll_from_hidden(model, h_mem, y, chunk_budget_bytes=ORACLE_NLL_CHUNK_BUDGET_BYTES)
    clock.mark()
    say("nll")
    mask_f = mask.float()
    utility = (nll_off - nll_mem) * mask_f
    plasticity = plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem, utility=utility, mask=mask,
                                                     tau=float(tau))
    clock.mark()
    target, confidence = (_bid(utility, tau) if scarcity_optimizer is None
                          else scarcity_optimizer.controller_target(utility))
    target, confidence = target * mask_f, confidence * mask_f
    loss_weight = positive_only_lm_weight(utility, mask, tau=tau, strength=strength, w_max=w_max)
    out: dict[str, Any] = {
        "utility": utility, "controller_target": target, "confidence": confidence, "loss_weight": loss_weight,
        "loss_reweight_diagnostics": _loss_reweight_diagnostics(nll_off=nll_off, loss_weight=loss_weight,
                                                                mask=mask)}
    if meta is not None and isinstance(meta.get("memory_residual"), torch.Tensor):
        out["memory_residual"] = _compact_residual(meta["memory_residual"].detach(), B)
        out["memory_gate"] = target.detach()
    out.update(plasticity)
    if gradient_conflict_monitor is not None:
        out["write_score"] = utility.detach()
    if update_model_memory_after:
        append = getattr(model, "append_memory_from_hidden", None)
        if append is None:
            raise ValueError("rank3_score_batch_causal(update_model_memory_after=True) requires "
                             "model.append_memory_from_hidden(...)")
        score, limit = utility.detach(), memory_write_tokens
        if gradient_conflict_monitor is not None:
            score, limit = gradient_conflict_monitor.apply_to_write_scores(
                model=model, hidden=h_off, targets=y, utility=utility, mask=mask,
                max_tokens=memory_write_tokens, step=step)
            out["write_score"] = score.detach()
        if limit is not None and int(limit) <= 0:
            if gradient_conflict_monitor is not None:
                out["gradient_conflict"] = torch.zeros_like(utility)
            say("skip_append_write_limit")
        else:
            event_ids = None
            reserve = getattr(cache, "reserve_event_ids", None)
            if callable(reserve):
                n_write = B * T if limit is None else min(B * T, max(0, int(limit)))
                event_ids = reserve(n_write, device=h_off.device)
            records = append(h_off.detach(), score=score.detach(), max_tokens=limit, event_ids=event_ids)
            if not isinstance(records, list):
                raise TypeError("append_memory_from_hidden must return generation-stamped records")
            out["memory_write_records"] = records
    clock.mark()
    cache.commit(txn)
    clock.flush()
    say("done")
    return out
