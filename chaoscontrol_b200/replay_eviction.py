"""Adaptive residual-memory maintenance: every episodic slot is scored against the
CURRENT model with counterfactual probes and filed under one of seven actions
(PRESERVE, DECAY, EVICT, REFRESH, QUARANTINE, DISTILL, RELEASE) by a rule policy or a
small learned policy, mutating actions are confirmed under the real memory-injected
dynamics before they are applied (behaviour of src/chaoscontrol/replay_eviction.py:71-4938).

A tick = pick a cached probe frame and a bounded chunk of slots -> ONE trunk encode and
one batched masked NLL over {with memory, without memory, hide slot i ...} -> update the
slots' running evidence -> choose actions -> confirm the mutating ones with the oracle pass
-> apply through the slot table and emit ``SlotCommit`` records for the training ranks.

How the work is shaped for a GPU here: hiding slot ``i`` from a softmax read is closed-form
(``(r - w_i s_i) / (1 - w_i)``), so all hide-one variants are built as one tensor and scored
by the fused LM-head kernel in a single launch; the oracle pass expands the batch by the
variant count and runs the real ``encode(memory_mode="force_on")`` with per-row slot masks
or a per-row slot override, again one forward per chunk of variants.
"""
from __future__ import annotations

import json
import math
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Optional, Sequence

import torch
import torch.nn.functional as F

from .cache_utility import ORACLE_NLL_CHUNK_BUDGET_BYTES, chunked_nll_from_hidden
from .slot_commit import SlotCommit
from .slot_table import SLOT_ACTIVE, SLOT_DECAYING, SLOT_QUARANTINED, SLOT_RETIRED, SLOT_WARMING, SlotRecord, SlotTable

__all__ = ["ReplayEvictionLoop", "TickResult", "counterfactual_probe", "oracle_confirm_slots",
           "oracle_confirm_refresh_candidates", "replay_score_slots", "MaintenancePolicy", "FullAControllerState",
           "LearnedCommitPolicy", "CpuRefreshProposalModel", "ProbeFrame", "SlotCommit", "CommitDecision",
           "CounterfactualResult", "OracleConfirmationResult", "RefreshCandidateOracleResult", "DistillReceipt",
           "MemoryEvent", "SLOT_ACTION_ORDER", "_evict_slots"]

SLOT_PRESERVE, SLOT_DECAY, SLOT_EVICT, SLOT_REFRESH = "PRESERVE", "DECAY", "EVICT", "REFRESH"
SLOT_QUARANTINE, SLOT_DISTILL, SLOT_RELEASE = "QUARANTINE", "DISTILL", "RELEASE"
SLOT_ACTION_ORDER = (SLOT_PRESERVE, SLOT_DECAY, SLOT_EVICT, SLOT_REFRESH, SLOT_QUARANTINE, SLOT_DISTILL, SLOT_RELEASE)
_MUTATING = (SLOT_EVICT, SLOT_REFRESH, SLOT_QUARANTINE, SLOT_DISTILL)


# ---------------------------------------------------------------------------
# records
# ---------------------------------------------------------------------------
@dataclass
class TickResult:
    evicted: list = field(default_factory=list)
    refreshed: list = field(default_factory=list)
    quarantined: list = field(default_factory=list)
    released: list = field(default_factory=list)
    distilled: list = field(default_factory=list)
    decayed: list = field(default_factory=list)
    slot_commits: list = field(default_factory=list)

    @property
    def evicted_indices(self) -> list[int]:
        return list(self.evicted)


@dataclass
class CounterfactualResult:
    marginal_gains: torch.Tensor       # [slots, B, T]  NLL(hide slot) - NLL(all slots): > 0 means the slot helps
    sidecar_value: torch.Tensor        # [B, T]         NLL(no memory) - NLL(all slots)
    nll_baseline: torch.Tensor
    nll_no_sidecar: torch.Tensor
    weights_baseline: torch.Tensor     # [B, slots] retrieval weights of the scored slots
    mask: torch.Tensor
    slot_indices: list
    scoring_mode: str = "proxy"


@dataclass
class OracleConfirmationResult:
    slot_indices: list
    oracle_deltas: torch.Tensor
    nll_baseline: torch.Tensor
    nll_no_sidecar: torch.Tensor
    mask: torch.Tensor


@dataclass
class RefreshCandidateOracleResult:
    slot_index: int
    candidate_names: list
    candidate_scores: torch.Tensor
    candidate_improvements: torch.Tensor
    nll_no_sidecar: torch.Tensor
    nll_candidates: torch.Tensor
    mask: torch.Tensor
    chunk_count: int = 0
    variants_total: int = 0


@dataclass
class DistillReceipt:
    slot_id: int
    step: int
    marginal_gain_before: float
    marginal_gain_peak: float
    marginal_gain_current: float
    target: str
    accepted: bool = False
    prototype_updated: bool = False
    prototype_reason: str = ""


@dataclass
class MemoryEvent:
    step: int
    tick: int
    slot_id: int
    action: str
    marginal_gain: float = 0.0
    sharpness: float = 0.0
    activation_drift: float = 0.0
    representation_drift: float = 0.0
    semantic_drift: float = 0.0
    contradiction: float = 0.0
    retrieval_mass: float = 0.0
    peak_utility: float = 0.0
    peak_sharpness: float = 0.0
    score_count: int = 0
    accepted: bool = True
    reason: str = ""
    refresh_candidate: str = ""


@dataclass
class ProbeFrame:
    frame_id: int
    step: int
    input_ids: torch.Tensor
    valid_mask: torch.Tensor
    cue: Optional[torch.Tensor]
    cache_read_cutoff: Optional[int]
    stream_id: int
    ingested_at: float
    processed_slots: set = field(default_factory=set)


@dataclass
class CommitDecision:
    action: str
    rule_action: str
    confidence: float
    probability: float
    entropy: float
    logits: dict
    probabilities: dict
    rule_values: dict
    vetoed_action: str = ""
    veto_reason: str = ""


# ---------------------------------------------------------------------------
# probes
# ---------------------------------------------------------------------------
def _autocast(dev: torch.device):
    return torch.autocast(dev.type if dev.type in ("cuda", "cpu") else "cpu", dtype=torch.bfloat16)


def _empty_cf(B: int, T: int, dev, mask, n_w: int = 0, idx: Optional[list] = None) -> CounterfactualResult:
    z = torch.zeros(B, T, device=dev)
    return CounterfactualResult(torch.zeros(0, B, T, device=dev), z, z.clone(), z.clone(),
                                torch.zeros(B, n_w, device=dev), mask, list(idx or []))


@torch.inference_mode()
def counterfactual_probe(*, model: Any, outer: Any, probe_input_ids: torch.Tensor, probe_valid_mask: torch.Tensor,
                         probe_cue: Optional[torch.Tensor] = None, cache_read_cutoff: Optional[int] = None,
                         chunk_size: int = 16, score_slot_indices: Optional[list] = None) -> CounterfactualResult:
    """Proxy scoring: one memory-off encode, then the decoded retrieval is ADDED to the hidden state for
    every variant (all slots / none / hide-one) and the variants are scored as one batch.  Variant 0 is
    the full read, variant 1 the empty read, variant ``2 + j`` hides ``score_slot_indices[j]``."""
    x, y = probe_input_ids[:, :-1], probe_input_ids[:, 1:]
    mask = probe_valid_mask[:, 1:].bool()
    B, T = x.shape
    dev = x.device
    table = getattr(outer, "table", None)
    if table is None or len(table) == 0:
        return _empty_cf(B, T, dev, mask)
    vis = table.visible_indices(read_cutoff=cache_read_cutoff)
    if not vis:
        return _empty_cf(B, T, dev, mask)
    if score_slot_indices is None:
        local, phys = list(range(len(vis))), list(vis)
    else:
        pos = {int(p): i for i, p in enumerate(vis)}
        pairs = [(pos[int(p)], int(p)) for p in dict.fromkeys(score_slot_indices) if int(p) in pos]
        if not pairs:
            return _empty_cf(B, T, dev, mask)
        local, phys = [a for a, _ in pairs], [b for _, b in pairs]
    cue_proj, decoder = getattr(outer, "cue_proj", None), getattr(outer, "decoder", None)
    if cue_proj is None or decoder is None:
        return _empty_cf(B, T, dev, mask, n_w=len(phys), idx=phys)
    with _autocast(dev):
        h = model.encode(x, memory_mode="off", cache_read_cutoff=cache_read_cutoff)
        cue = probe_cue.to(dev) if probe_cue is not None else h.detach().mean(dim=1)
        M = table.slot_matrix(vis).to(dev)
        q = cue_proj(cue.to(cue_proj.weight.dtype))
        M = M.to(q.dtype)
        w = F.softmax(q @ M.T, dim=-1)                                   # [B, N]
        r_all = w @ M                                                    # [B, O]
    D = h.shape[-1]
    loc = torch.as_tensor(local, device=dev, dtype=torch.long)
    n_var = len(local) + 2
    nll = torch.empty(n_var, B, T, device=dev, dtype=torch.float32)
    step = n_var if chunk_size <= 0 else int(chunk_size)
    for s in range(0, n_var, step):
        e = min(n_var, s + step)
        with _autocast(dev):
            r = torch.zeros(e - s, B, M.shape[-1], device=dev, dtype=M.dtype)
            if s == 0:
                r[0] = r_all
            hs = max(s, 2)
            if hs < e:
                sel = loc[hs - 2: e - 2]
                wi = w[:, sel].T.unsqueeze(-1)                            # [C, B, 1]
                gone = (r_all.unsqueeze(0) - wi * M[sel].unsqueeze(1)) / (1.0 - wi).clamp_min(1e-7)
                r[hs - s:] = torch.where(1.0 - wi > 1e-7, gone, torch.zeros_like(gone))
            hv = h.unsqueeze(0) + F.linear(r, decoder.weight.to(r.dtype)).unsqueeze(2)
        C = e - s
        nll[s:e] = chunked_nll_from_hidden(model, hv.reshape(C * B, T, D), y.unsqueeze(0).expand(C, -1, -1)
                                           .reshape(C * B, T), chunk_budget_bytes=ORACLE_NLL_CHUNK_BUDGET_BYTES
                                           ).view(C, B, T)
    return CounterfactualResult((nll[2:] - nll[0]).cpu(), (nll[1] - nll[0]).cpu(), nll[0].cpu(), nll[1].cpu(),
                                w[:, loc].float().cpu(), mask.cpu(), phys)


def _n_slots(outer: Any) -> int:
    table = getattr(outer, "table", None)
    return len(table) if table is not None else len(getattr(outer, "_slots", []))


@torch.inference_mode()
def oracle_confirm_slots(*, model: Any, outer: Any, probe_input_ids: torch.Tensor, probe_valid_mask: torch.Tensor,
                         slot_indices: list, cache_read_cutoff: Optional[int] = None,
                         variant_chunk_size: int = 1) -> OracleConfirmationResult:
    """Hide-one deltas measured with the real pre-recurrence memory injection: the batch is expanded by
    the variant count and every row carries its own slot mask."""
    x, y = probe_input_ids[:, :-1], probe_input_ids[:, 1:]
    mask = probe_valid_mask[:, 1:].bool()
    B, T = x.shape
    dev = x.device
    n = _n_slots(outer)
    cands = [int(i) for i in dict.fromkeys(slot_indices) if 0 <= int(i) < n]
    if n <= 0 or not cands:
        z = torch.zeros(B, T, device=dev)
        return OracleConfirmationResult([], torch.zeros(0, B, T, device=dev), z, z.clone(), mask)

    def score(masks: torch.Tensor) -> torch.Tensor:
        V = masks.shape[0]
        with _autocast(dev):
            hid = model.encode(x.repeat(V, 1), memory_mode="force_on", cache_read_cutoff=cache_read_cutoff,
                               memory_slot_mask=masks.repeat_interleave(B, dim=0))
        return chunked_nll_from_hidden(model, hid, y.repeat(V, 1),
                                       chunk_budget_bytes=ORACLE_NLL_CHUNK_BUDGET_BYTES).view(V, B, T)

    base = torch.ones(2, n, device=dev, dtype=torch.bool)
    base[1] = False
    b = score(base)
    deltas = torch.empty(len(cands), B, T, dtype=torch.float32, device=b.device)
    step = max(1, int(variant_chunk_size))
    for s in range(0, len(cands), step):
        chunk = cands[s:s + step]
        m = torch.ones(len(chunk), n, device=dev, dtype=torch.bool)
        m[torch.arange(len(chunk), device=dev), torch.as_tensor(chunk, device=dev)] = False
        deltas[s:s + len(chunk)] = score(m) - b[0]
    return OracleConfirmationResult(cands, deltas.cpu(), b[0].cpu(), b[1].cpu(), mask.cpu())


@torch.inference_mode()
def oracle_confirm_refresh_candidates(*, model: Any, outer: Any, probe_input_ids: torch.Tensor,
                                      probe_valid_mask: torch.Tensor, slot_index: int,
                                      candidate_tensors: list, cache_read_cutoff: Optional[int] = None,
                                      variant_chunk_size: int = 16) -> RefreshCandidateOracleResult:
    """Scores replacement tensors for one slot under the real read path with a per-row slot override (the
    table is never mutated).  ``candidate_scores[k]`` = mean over valid tokens of NLL(no memory) -
    NLL(candidate k); candidate 0 is the current tensor, so ``candidate_improvements[0] == 0``."""
    x, y = probe_input_ids[:, :-1], probe_input_ids[:, 1:]
    mask = probe_valid_mask[:, 1:].bool()
    B, T = x.shape
    dev = x.device
    n, phys = _n_slots(outer), int(slot_index)
    if n <= 0 or not 0 <= phys < n or not candidate_tensors:
        return RefreshCandidateOracleResult(phys, [], torch.zeros(0), torch.zeros(0), torch.zeros(B, T),
                                            torch.zeros(0, B, T), mask)
    names, vals = [], []
    for name, t in candidate_tensors:
        t = t.detach()
        t = t.unsqueeze(0) if t.dim() == 1 else (t.squeeze(1) if t.dim() == 3 and t.shape[1] == 1 else t)
        if t.dim() != 2 or t.shape[0] != 1:
            raise ValueError("refresh candidate tensors must have shape (1, outer_dim)")
        names.append(str(name))
        vals.append(t)
    stack = torch.cat(vals, 0).to(dev)
    K = stack.shape[0]
    with _autocast(dev):
        h_off = model.encode(x, memory_mode="force_on", cache_read_cutoff=cache_read_cutoff,
                             memory_slot_mask=torch.zeros(B, n, device=dev, dtype=torch.bool))
    nll_off = chunked_nll_from_hidden(model, h_off, y, chunk_budget_bytes=ORACLE_NLL_CHUNK_BUDGET_BYTES)
    nll_c = torch.empty(K, B, T, dtype=torch.float32, device=nll_off.device)
    step, chunks = max(1, int(variant_chunk_size)), 0
    for s in range(0, K, step):
        e = min(K, s + step)
        k = e - s
        chunks += 1
        with _autocast(dev):
            hid = model.encode(x.repeat(k, 1), memory_mode="force_on", cache_read_cutoff=cache_read_cutoff,
                               memory_slot_override_index=phys,
                               memory_slot_override_values=stack[s:e].repeat_interleave(B, dim=0))
        nll_c[s:e] = chunked_nll_from_hidden(model, hid, y.repeat(k, 1),
                                             chunk_budget_bytes=ORACLE_NLL_CHUNK_BUDGET_BYTES).view(k, B, T)
    mf = mask.to(nll_c.device).float()
    scores = ((nll_off.unsqueeze(0) - nll_c) * mf).sum((1, 2)) / mf.sum().clamp_min(1.0)
    return RefreshCandidateOracleResult(phys, names, scores.cpu(), (scores - scores[0]).cpu(), nll_off.cpu(),
                                        nll_c.cpu(), mask.cpu(), chunks, K)


@torch.inference_mode()
def replay_score_slots(*, model: Any, probe_input_ids: torch.Tensor, probe_valid_mask: torch.Tensor,
                       cache_read_cutoff: Optional[int] = None) -> dict[str, Any]:
    """Per-slot mean marginal gain over the valid tokens of one probe batch."""
    empty = {"slot_utilities": torch.tensor([]), "slot_indices": [], "mean_utility": 0.0}
    outer = getattr(model, "outer_model", None)
    if outer is None:
        return empty
    r = counterfactual_probe(model=model, outer=outer, probe_input_ids=probe_input_ids,
                             probe_valid_mask=probe_valid_mask, cache_read_cutoff=cache_read_cutoff)
    if not r.slot_indices:
        return empty
    m = r.mask.float()
    per_slot = (r.marginal_gains.float() * m).sum((1, 2)) / m.sum().clamp_min(1.0)
    return {"slot_utilities": per_slot, "slot_indices": list(r.slot_indices),
            "mean_utility": float(r.sidecar_value[r.mask].mean()) if bool(r.mask.any()) else 0.0,
            "n_tokens_scored": int(r.mask.sum()), "retrieval_weights": r.weights_baseline,
            "per_token_utility": r.sidecar_value, "mask": r.mask}


def _per_slot_sharpness(gains: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Variance of the token-level gain per slot: a slot that matters a lot for few tokens is sharp."""
    if gains.shape[0] == 0:
        return torch.zeros(0)
    m = mask.float()
    n = m.sum().clamp_min(1.0)
    mean = (gains * m).sum((1, 2)) / n
    return ((gains * gains * m).sum((1, 2)) / n - mean * mean).clamp_min(0.0)


def _representation_drift(outer: Any, slot: torch.Tensor) -> float:
    """``1 - cos(slot, tanh(encoder(decoder(slot))))``: how badly the slot survives a round trip through
    the CURRENT decoder / encoder."""
    enc, dec = getattr(outer, "encoder", None), getattr(outer, "decoder", None)
    if enc is None or dec is None:
        return 0.0
    with torch.inference_mode():
        back = torch.tanh(enc(dec(slot.to(dec.weight.dtype)).to(enc.weight.dtype)))
    return float(1.0 - F.cosine_similarity(slot.float().flatten(), back.float().flatten(), dim=0))


# ---------------------------------------------------------------------------
# controller state, refresh proposals, policies
# ---------------------------------------------------------------------------
class FullAControllerState:
    """Small full-matrix recurrent state that accumulates maintenance evidence and emits a direction in
    slot space.  Dynamics: rotation pairs + damping + a low-rank perturbation, discretised with a matrix
    exponential and rescaled so the top log singular value is ``target_log_sv`` (a stable, slightly
    contracting map); the state norm is capped."""
    input_dim = 12

    def __init__(self, state_dim: int = 32, rank: int = 8, dt: float = 1.0, gamma: float = 0.08,
                 target_log_sv: float = -0.05, max_state_norm: float = 8.0, perturbation_scale: float = 0.25,
                 feedback_lr: float = 0.05, seed: int = 0) -> None:
        self.state_dim, self.rank = int(state_dim), max(1, min(int(rank), int(state_dim)))
        self.dt, self.gamma, self.target_log_sv = float(dt), max(1e-4, float(gamma)), float(target_log_sv)
        self.max_state_norm, self.feedback_lr, self.seed = max(1e-4, float(max_state_norm)), float(feedback_lr), int(seed)
        g = torch.Generator().manual_seed(self.seed)
        H = self.state_dim
        self.W_in = torch.randn(H, self.input_dim, generator=g) / math.sqrt(self.input_dim)
        cont = -self.gamma * torch.eye(H)
        pairs = H // 2
        if pairs:
            om = torch.linspace(0.05, 0.6, pairs)
            a = torch.arange(pairs) * 2
            cont[a, a + 1] -= om
            cont[a + 1, a] += om
        U = F.normalize(torch.randn(H, self.rank, generator=g), dim=0)
        V = F.normalize(torch.randn(H, self.rank, generator=g), dim=0)
        low = U @ V.T
        cont = cont + low * (float(perturbation_scale) / torch.linalg.matrix_norm(low, ord=2).clamp_min(1e-8))
        A = torch.matrix_exp(cont * self.dt)
        top = float(torch.linalg.svdvals(A).clamp_min(1e-8).log().max())
        if top > self.target_log_sv:
            A = A * math.exp(self.target_log_sv - top)
        self.A = A.contiguous()
        self.top_log_sv = float(torch.linalg.svdvals(self.A).clamp_min(1e-8).log().max())
        self.h = torch.zeros(H)
        self.W_out: Optional[torch.Tensor] = None        # [slot_dim, H], sized on first use
        self.steps = self.clamps = self.feedback_updates = 0
        self._g = g

    def _ensure_slot_dim(self, slot_dim: int) -> None:
        if self.W_out is None or self.W_out.shape[0] != int(slot_dim):
            self.W_out = torch.randn(int(slot_dim), self.state_dim, generator=self._g) * 0.05

    @torch.no_grad()
    def step(self, features: torch.Tensor, *, slot_dim: int) -> torch.Tensor:
        """``h <- A h + tanh(W_in f)``; returns the unit proposal direction ``W_out h`` in slot space."""
        self._ensure_slot_dim(slot_dim)
        f = torch.nan_to_num(features.detach().float().flatten()[: self.input_dim])
        f = F.pad(f, (0, self.input_dim - f.numel()))
        h = self.A @ self.h + torch.tanh(self.W_in @ f)
        n = float(h.norm())
        if n > self.max_state_norm:
            h = h * (self.max_state_norm / n)
            self.clamps += 1
        self.h = h
        self.steps += 1
        return F.normalize(self.W_out @ h, dim=0, eps=1e-8)

    def hidden_state(self) -> torch.Tensor:
        return self.h.clone()

    @torch.no_grad()
    def update_feedback(self, direction: torch.Tensor, reward: float) -> None:
        """Moves the read-out toward (away from) a proposed direction that helped (hurt)."""
        if self.W_out is None or not math.isfinite(float(reward)):
            return
        d = F.normalize(direction.detach().float().flatten(), dim=0, eps=1e-8)
        if d.numel() != self.W_out.shape[0]:
            return
        r = max(-1.0, min(1.0, float(reward)))
        self.W_out += self.feedback_lr * r * torch.outer(d, F.normalize(self.h, dim=0, eps=1e-8))
        self.feedback_updates += 1

    def diagnostics(self) -> dict[str, Any]:
        return {"state_dim": self.state_dim, "rank": self.rank, "top_log_sv": self.top_log_sv,
                "state_norm": float(self.h.norm()), "steps": self.steps, "state_clamp_count": self.clamps,
                "feedback_updates": self.feedback_updates}

    def state_dict(self) -> dict[str, Any]:
        return {"h": self.h.clone(), "W_out": None if self.W_out is None else self.W_out.clone(), "steps": self.steps,
                "clamps": self.clamps, "feedback_updates": self.feedback_updates, "seed": self.seed,
                "state_dim": self.state_dim}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        if int(state.get("state_dim", self.state_dim)) != self.state_dim:
            raise ValueError("FullAControllerState.load_state_dict: state_dim mismatch")
        self.h = state["h"].clone().float()
        self.W_out = None if state.get("W_out") is None else state["W_out"].clone().float()
        self.steps, self.clamps = int(state.get("steps", 0)), int(state.get("clamps", 0))
        self.feedback_updates = int(state.get("feedback_updates", 0))


class CpuRefreshProposalModel:
    """Proposes ``k`` replacement tensors for a drifting slot on the CPU: the current tensor (always
    candidate 0), its round trip through the current decoder / encoder, blends toward the probe cue and
    toward the controller's direction, and perturbations inside a learned low-rank subspace whose basis
    follows (with momentum) the displacements that the oracle accepted."""

    def __init__(self, k: int = 16, rank: int = 8, lr: float = 0.1, noise_scale: float = 0.04, momentum: float = 0.9,
                 seed: int = 1729) -> None:
        self.k, self.rank, self.lr = max(2, int(k)), max(1, int(rank)), float(lr)
        self.noise_scale, self.momentum = float(noise_scale), float(momentum)
        self._g = torch.Generator().manual_seed(int(seed))
        self.basis: Optional[torch.Tensor] = None
        self.accepted = self.proposed = self.updates = 0
        self.weight_version = 0

    def mark_weight_version(self, version: int) -> None:
        self.weight_version = int(version)

    def _ensure_dim(self, dim: int) -> None:
        if self.basis is None or self.basis.shape[1] != dim:
            self.basis = F.normalize(torch.randn(self.rank, dim, generator=self._g), dim=1)

    def _roundtrip(self, outer: Any, slot: torch.Tensor) -> Optional[torch.Tensor]:
        enc, dec = getattr(outer, "encoder", None), getattr(outer, "decoder", None)
        if enc is None or dec is None:
            return None
        with torch.inference_mode():
            w_d, w_e = dec.weight.detach().float().cpu(), enc.weight.detach().float().cpu()
            return torch.tanh(F.linear(F.linear(slot, w_d), w_e))

    @torch.no_grad()
    def sample_k(self, *, outer: Any, slot: torch.Tensor, cue_outer: Optional[torch.Tensor] = None,
                 controller_direction: Optional[torch.Tensor] = None) -> list[tuple[str, torch.Tensor]]:
        s = slot.detach().float().cpu().reshape(1, -1)
        self._ensure_dim(s.shape[1])
        scale = float(s.norm().clamp_min(1e-6))
        out = [("current", s.clone())]
        rt = self._roundtrip(outer, s)
        if rt is not None:
            out.append(("roundtrip", rt))
            out.append(("roundtrip_blend", (1 - self.lr) * s + self.lr * rt))
        if cue_outer is not None:
            c = cue_outer.detach().float().cpu().reshape(1, -1)
            if c.shape == s.shape:
                out.append(("cue_blend", (1 - self.lr) * s + self.lr * c))
        if controller_direction is not None and controller_direction.numel() == s.numel():
            out.append(("controller_dir", s + self.lr * scale * controller_direction.detach().float().cpu().reshape(1, -1)))
        i = 0
        while len(out) < self.k:
            coef = torch.randn(1, self.rank, generator=self._g) * self.noise_scale * scale
            out.append((f"subspace_{i}", s + coef @ self.basis))
            i += 1
        self.proposed += len(out)
        return out[: self.k]

    @torch.no_grad()
    def update(self, *, slot: torch.Tensor, accepted: Optional[torch.Tensor], improvement: float) -> None:
        """Rotates the least-used basis row toward an accepted displacement."""
        self.updates += 1
        if accepted is None or not improvement > 0:
            return
        d = (accepted.detach().float().cpu() - slot.detach().float().cpu()).reshape(-1)
        if float(d.norm()) < 1e-8:
            return
        self._ensure_dim(d.numel())
        d = F.normalize(d, dim=0)
        j = int((self.basis @ d).abs().argmin())
        self.basis[j] = F.normalize(self.momentum * self.basis[j] + (1 - self.momentum) * d, dim=0)
        self.accepted += 1

    def diagnostics(self) -> dict[str, Any]:
        return {"k": self.k, "rank": self.rank, "proposed": self.proposed, "accepted": self.accepted,
                "updates": self.updates, "weight_version": self.weight_version}

    def state_dict(self) -> dict[str, Any]:
        return {"basis": None if self.basis is None else self.basis.clone(), "accepted": self.accepted,
                "proposed": self.proposed, "updates": self.updates, "weight_version": self.weight_version,
                "rng": self._g.get_state()}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.basis = None if state.get("basis") is None else state["basis"].clone().float()
        self.accepted, self.proposed = int(state.get("accepted", 0)), int(state.get("proposed", 0))
        self.updates, self.weight_version = int(state.get("updates", 0)), int(state.get("weight_version", 0))
        if state.get("rng") is not None:
            self._g.set_state(state["rng"])


class MaintenancePolicy:
    """Rule policy: a value per action from a slot's running evidence; the largest wins."""

    def action_values(self, rec: SlotRecord, *, eviction_threshold: float, useful_threshold: float,
                      drift_threshold: float, quarantine_threshold: float, distill_peak_threshold: float,
                      peak_preserve_utility_threshold: float, peak_preserve_sharpness_threshold: float,
                      min_age: int, capacity_pressure: bool = False) -> dict[str, float]:
        scored = rec.score_count > 0
        aged = rec.last_scored_step > 0 and (rec.last_scored_step - rec.created_step) >= min_age
        settled = scored and aged
        protected = (rec.peak_utility >= peak_preserve_utility_threshold or
                     rec.peak_sharpness >= peak_preserve_sharpness_threshold)
        v = dict.fromkeys(SLOT_ACTION_ORDER, 0.0)
        if settled and rec.contradiction_ema > abs(quarantine_threshold):
            v[SLOT_QUARANTINE] = rec.contradiction_ema + 0.5 * rec.negative_streak
        if settled and not protected and rec.peak_utility > distill_peak_threshold:
            absorbed = 1.0 - rec.marginal_gain_ema / max(rec.peak_utility, 1e-6)
            if absorbed > 0.5 and rec.marginal_gain_ema < 2 * eviction_threshold:
                v[SLOT_DISTILL] = absorbed * rec.peak_utility
        if capacity_pressure and settled and not protected and rec.utility_ema < eviction_threshold:
            v[SLOT_EVICT] = eviction_threshold - rec.utility_ema + max(0.0, useful_threshold - rec.marginal_gain_ema)
        drift = max(rec.activation_drift_ema, rec.representation_drift_ema, rec.semantic_drift_ema)
        if drift > drift_threshold and rec.marginal_gain_ema > useful_threshold:
            v[SLOT_REFRESH] = 0.8 * drift + 0.6 * rec.marginal_gain_ema
        if rec.state == SLOT_QUARANTINED and scored:
            v[SLOT_RELEASE] = max(0.0, rec.marginal_gain_ema) + 0.25 * rec.positive_streak
        v[SLOT_PRESERVE] = (rec.marginal_gain_ema + 0.7 * rec.sharpness_ema + 0.25 * rec.peak_utility +
                            0.25 * rec.peak_sharpness)
        if not capacity_pressure and rec.utility_ema < 2 * eviction_threshold:
            v[SLOT_DECAY] = 2 * eviction_threshold - rec.utility_ema
        return v

    def choose(self, rec: SlotRecord, **kw: Any) -> str:
        vals = self.action_values(rec, **kw)
        return max(vals, key=lambda k: vals[k])


class LearnedCommitPolicy:
    """Softmax policy over the maintenance actions: logits = ``W [slot features ; controller state]`` plus a
    prior from the rule values; illegal actions are masked; a chosen action's later physics outcome moves
    its logit with a REINFORCE step (``lr * advantage * (onehot - p)`` on the features)."""
    input_dim = FullAControllerState.input_dim

    def __init__(self, *, state_dim: int = 32, online_lr: float = 0.05, temperature: float = 0.75,
                 rule_prior_weight: float = 4.0, seed: int = 0) -> None:
        self.state_dim, self.lr = int(state_dim), max(0.0, float(online_lr))
        self.temperature, self.rule_prior_weight = max(1e-4, float(temperature)), float(rule_prior_weight)
        self.W = torch.zeros(len(SLOT_ACTION_ORDER), self.input_dim + self.state_dim)
        self.b = torch.zeros(len(SLOT_ACTION_ORDER))
        self._g = torch.Generator().manual_seed(int(seed))
        self.decisions = self.feedbacks = self.vetoes = 0
        self.baseline = 0.0

    @staticmethod
    def features(rec: SlotRecord, *, capacity_pressure: bool) -> torch.Tensor:
        return torch.tensor([rec.utility_ema, rec.marginal_gain_ema, rec.sharpness_ema, rec.activation_drift_ema,
                             rec.representation_drift_ema, rec.semantic_drift_ema, rec.contradiction_ema,
                             rec.retrieval_mass_ema, rec.peak_utility, math.log1p(rec.score_count),
                             float(rec.state == SLOT_QUARANTINED), float(capacity_pressure)], dtype=torch.float32)

    @staticmethod
    def legal_actions(rec: SlotRecord, *, capacity_pressure: bool, min_age: int) -> set:
        legal = {SLOT_PRESERVE, SLOT_DECAY}
        settled = rec.score_count > 0 and (rec.last_scored_step - rec.created_step) >= min_age
        if rec.state == SLOT_QUARANTINED:
            return {SLOT_PRESERVE, SLOT_RELEASE, SLOT_EVICT} if settled else {SLOT_PRESERVE, SLOT_RELEASE}
        if settled:
            legal |= {SLOT_REFRESH, SLOT_QUARANTINE, SLOT_DISTILL}
            if capacity_pressure:
                legal.add(SLOT_EVICT)
        return legal

    @torch.no_grad()
    def choose(self, rec: SlotRecord, *, controller_state: torch.Tensor, rule_values: dict, capacity_pressure: bool,
               min_age: int, sample: bool = False) -> tuple[CommitDecision, torch.Tensor]:
        feat = torch.cat([self.features(rec, capacity_pressure=capacity_pressure),
                          F.pad(controller_state.float().flatten()[: self.state_dim],
                                (0, max(0, self.state_dim - controller_state.numel())))])
        prior = torch.tensor([rule_values.get(a, 0.0) for a in SLOT_ACTION_ORDER])
        logits = (self.W @ feat + self.b + self.rule_prior_weight * prior) / self.temperature
        legal = self.legal_actions(rec, capacity_pressure=capacity_pressure, min_age=min_age)
        rule_action = max(rule_values, key=lambda k: rule_values[k]) if rule_values else SLOT_PRESERVE
        masked = logits.clone()
        for i, a in enumerate(SLOT_ACTION_ORDER):
            if a not in legal:
                masked[i] = -float("inf")
        p = torch.softmax(masked, 0)
        i = int(torch.multinomial(p, 1, generator=self._g)) if sample else int(p.argmax())
        raw_best = SLOT_ACTION_ORDER[int(logits.argmax())]
        veto = raw_best if raw_best not in legal else ""
        if veto:
            self.vetoes += 1
        self.decisions += 1
        ent = float(-(p[p > 0] * p[p > 0].log()).sum())
        dec = CommitDecision(SLOT_ACTION_ORDER[i], rule_action, float(p[i]), float(p[i]), ent,
                             dict(zip(SLOT_ACTION_ORDER, logits.tolist())), dict(zip(SLOT_ACTION_ORDER, p.tolist())),
                             dict(rule_values), vetoed_action=veto, veto_reason="illegal_for_slot_state" if veto else "")
        return dec, feat

    @torch.no_grad()
    def apply_feedback(self, *, decision: CommitDecision, features: torch.Tensor, reward: float) -> None:
        if self.lr <= 0.0 or not math.isfinite(float(reward)):
            return
        adv = max(-1.0, min(1.0, float(reward) - self.baseline))
        self.baseline = 0.9 * self.baseline + 0.1 * float(reward)
        p = torch.tensor([decision.probabilities.get(a, 0.0) for a in SLOT_ACTION_ORDER])
        onehot = torch.zeros_like(p)
        onehot[SLOT_ACTION_ORDER.index(decision.action)] = 1.0
        g = (onehot - p) * adv
        self.W += self.lr * torch.outer(g, features)
        self.b += self.lr * g
        self.feedbacks += 1

    def diagnostics(self) -> dict[str, Any]:
        return {"decisions": self.decisions, "feedbacks": self.feedbacks, "vetoes": self.vetoes,
                "baseline": self.baseline, "weight_norm": float(self.W.norm())}

    def state_dict(self) -> dict[str, Any]:
        return {"W": self.W.clone(), "b": self.b.clone(), "baseline": self.baseline, "decisions": self.decisions,
                "feedbacks": self.feedbacks, "vetoes": self.vetoes}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        if tuple(state["W"].shape) != tuple(self.W.shape):
            raise ValueError("LearnedCommitPolicy.load_state_dict: weight shape mismatch")
        self.W, self.b = state["W"].clone().float(), state["b"].clone().float()
        self.baseline = float(state.get("baseline", 0.0))
        self.decisions, self.feedbacks = int(state.get("decisions", 0)), int(state.get("feedbacks", 0))
        self.vetoes = int(state.get("vetoes", 0))


def _evict_slots(outer: Any, indices: list) -> list:
    """Retires the slots at these PHYSICAL rows; returns their slot ids."""
    table: SlotTable = outer.table
    ids = [sid for sid in (table.physical_to_slot_id(int(i)) for i in indices) if sid is not None]
    return table.retire_many(ids, reason="evicted")


# ---------------------------------------------------------------------------
# the loop
# ---------------------------------------------------------------------------
class ReplayEvictionLoop:
    def __init__(self, *, action_mode: str = "active", memory_streams: int = 8, eviction_threshold: float = 0.01,
                 eviction_ema_beta: float = 0.9, min_slot_age_steps: int = 128, max_seconds_per_tick: float = 0.5,
                 trace_path: Optional[str] = None, trace_max_rows: int = 0, trace_flush_rows: int = 256,
                 probe_chunk_size: int = 16, scoring_mode: str = "proxy", oracle_confirm_top_k: int = 32,
                 oracle_variant_chunk_size: int = 1, drift_threshold: float = 0.3, repr_drift_threshold: float = 0.2,
                 refresh_lr: float = 0.1, refresh_candidate_count: int = 16, refresh_proposal_rank: int = 8,
                 refresh_proposal_noise_scale: float = 0.04, refresh_proposal_momentum: float = 0.9,
                 refresh_candidate_variant_chunk_size: int = 16, refresh_proposal_seed: int = 1729,
                 controller_state_dim: int = 32, controller_rank: int = 8, controller_dt: float = 1.0,
                 controller_gamma: float = 0.08, controller_target_log_sv: float = -0.05,
                 controller_max_state_norm: float = 8.0, controller_perturbation_scale: float = 0.25,
                 controller_feedback_lr: float = 0.05, quarantine_threshold: float = -0.01, max_quarantined: int = 8,
                 distill_peak_threshold: float = 0.04, peak_preserve_utility_threshold: float = 0.20,
                 peak_preserve_sharpness_threshold: float = 0.20, useful_threshold: float = 0.005,
                 probe_buffer_size: int = 32, frame_ttl_steps: int = 256, slot_work_chunk_size: int = 64,
                 action_agreement_count: int = 2, commit_policy: str = "learned", commit_online_lr: float = 0.05,
                 commit_temperature: float = 0.75, max_slots: Optional[int] = None, arm_runtime_enabled: bool = False,
                 arm_runtime_namespace: Optional[str] = None, evidence_engine_enabled: bool = False,
                 evidence_engine_d_model: int = 384, evidence_engine_lanes: int = 8, **unused: Any) -> None:
        if action_mode not in ("active", "shadow"):
            raise ValueError("action_mode must be 'active' or 'shadow'")
        if scoring_mode not in ("proxy", "oracle"):
            raise ValueError("scoring_mode must be 'proxy' or 'oracle'")
        if commit_policy not in ("learned", "rule"):
            raise ValueError("commit_policy must be 'learned' or 'rule'")
        self.action_mode, self.scoring_mode, self.commit_policy = action_mode, scoring_mode, commit_policy
        self.memory_streams = max(1, int(memory_streams))
        self.beta, self.min_age, self.max_seconds = float(eviction_ema_beta), int(min_slot_age_steps), float(max_seconds_per_tick)
        self.probe_chunk_size = int(probe_chunk_size)
        self.oracle_top_k, self.oracle_chunk = max(0, int(oracle_confirm_top_k)), max(1, int(oracle_variant_chunk_size))
        self.refresh_chunk = max(1, int(refresh_candidate_variant_chunk_size))
        self.max_quarantined, self.max_slots = int(max_quarantined), max_slots
        self.frame_ttl, self.slot_chunk = max(0, int(frame_ttl_steps)), max(1, int(slot_work_chunk_size))
        self.agreement = max(1, int(action_agreement_count))
        self._rule_kw = dict(eviction_threshold=float(eviction_threshold), useful_threshold=float(useful_threshold),
                             drift_threshold=float(drift_threshold), quarantine_threshold=float(quarantine_threshold),
                             distill_peak_threshold=float(distill_peak_threshold),
                             peak_preserve_utility_threshold=float(peak_preserve_utility_threshold),
                             peak_preserve_sharpness_threshold=float(peak_preserve_sharpness_threshold),
                             min_age=self.min_age)
        self.repr_drift_threshold = float(repr_drift_threshold)
        self.rule = MaintenancePolicy()
        self.controller = FullAControllerState(controller_state_dim, controller_rank, controller_dt, controller_gamma,
                                               controller_target_log_sv, controller_max_state_norm,
                                               controller_perturbation_scale, controller_feedback_lr)
        self.learned = LearnedCommitPolicy(state_dim=controller_state_dim, online_lr=commit_online_lr,
                                           temperature=commit_temperature)
        self.proposals = CpuRefreshProposalModel(refresh_candidate_count, refresh_proposal_rank, refresh_lr,
                                                 refresh_proposal_noise_scale, refresh_proposal_momentum,
                                                 refresh_proposal_seed)
        # optional native runtime: the C++ scheduler owns frame / slot-chunk selection, the evidence engine
        # scores every frame's 32-token cue on the host cores
        self._sched = self._evidence = None
        if arm_runtime_enabled:
            from .episodic.arm_native import ArmMaintenanceScheduler
            self._sched = ArmMaintenanceScheduler(self.memory_streams, min(self.slot_chunk, 16), self.frame_ttl,
                                                  max(1, int(probe_buffer_size)))
        if evidence_engine_enabled:
            from .episodic.arm_native import CpuEvidenceEngine
            self._evidence = CpuEvidenceEngine(evidence_engine_lanes, evidence_engine_d_model)
        self._frames: deque = deque(maxlen=max(1, int(probe_buffer_size)))
        self._next_frame_id = self._tick = 0
        self._streak: dict[int, tuple[str, int]] = {}
        self._events: list[MemoryEvent] = []
        self._receipts: list[DistillReceipt] = []
        self._trace_path = Path(trace_path) if trace_path else None
        self._trace_max, self._trace_flush = max(0, int(trace_max_rows)), max(1, int(trace_flush_rows))
        self._trace_buf: list[str] = []
        self._trace_rows = 0
        self._counts = dict.fromkeys(SLOT_ACTION_ORDER, 0)
        self._stats = {"frames_ingested": 0, "frames_dropped_overflow": 0, "frames_dropped_stale": 0, "ticks": 0,
                       "slots_scored": 0, "oracle_confirmed": 0, "oracle_rejected": 0, "budget_exhausted": 0,
                       "probe_seconds": 0.0, "oracle_seconds": 0.0}

    # -- frames -----------------------------------------------------------
    def cache_probe(self, *, input_ids: torch.Tensor, valid_mask: torch.Tensor, cue: Optional[torch.Tensor] = None,
                    cache_read_cutoff: Optional[int], step: int, stream_id: int = 0) -> None:
        if len(self._frames) == self._frames.maxlen:
            self._stats["frames_dropped_overflow"] += 1
        self._frames.append(ProbeFrame(self._next_frame_id, int(step), input_ids.detach(), valid_mask.detach(),
                                       None if cue is None else cue.detach(), cache_read_cutoff,
                                       int(stream_id) % self.memory_streams, time.monotonic()))
        frame = self._frames[-1]
        if self._sched is not None:
            self._sched.ingest_frame(frame.frame_id, frame.step, frame.stream_id, cache_read_cutoff)
        if self._evidence is not None:
            self._ingest_evidence(frame)
        self._next_frame_id += 1
        self._stats["frames_ingested"] += 1

    def refresh_evidence_weights(self, model: Any) -> None:
        """Installs the model's current final-norm weight and LM head in the evidence engine."""
        if self._evidence is not None:
            self._evidence.set_lm_head(model.final_norm.weight.detach().float().cpu(),
                                       model.lm_head.weight.detach().cpu())

    def _ingest_evidence(self, frame: ProbeFrame) -> None:
        from .episodic.arm_native import CUE_TOKENS
        d = self._evidence.d_model
        cue = torch.zeros(CUE_TOKENS, d, dtype=torch.bfloat16)
        if frame.cue is not None and frame.cue.shape[-1] == d:
            rows = frame.cue.detach().reshape(-1, d)[:CUE_TOKENS].to("cpu", torch.bfloat16)
            cue[: rows.shape[0]] = rows
        tg = torch.zeros(CUE_TOKENS, dtype=torch.int32)
        ids = frame.input_ids.detach().reshape(-1)[1:CUE_TOKENS + 1].to("cpu", torch.int32)
        tg[: ids.numel()] = ids
        self._evidence.ingest_frame(cue, tg, frame_id=frame.frame_id, step=frame.step, stream_id=frame.stream_id)

    def has_probe(self) -> bool:
        return bool(self._frames)

    def latest_probe_step(self) -> Optional[int]:
        return self._frames[-1].step if self._frames else None

    def _select_work(self, outer: Any, step: int) -> tuple[Optional[ProbeFrame], list]:
        """Newest frame that still has unprocessed visible slots, and the next chunk of those slots
        (least recently scored first)."""
        if self.frame_ttl:
            fresh = deque((f for f in self._frames if step - f.step <= self.frame_ttl), maxlen=self._frames.maxlen)
            self._stats["frames_dropped_stale"] += len(self._frames) - len(fresh)
            self._frames = fresh
        table: SlotTable = outer.table
        for frame in reversed(self._frames):
            vis = table.visible_indices(read_cutoff=frame.cache_read_cutoff)
            todo = [p for p in vis if table.physical_to_slot_id(p) not in frame.processed_slots]
            if todo:
                todo.sort(key=lambda p: table.record(table.physical_to_slot_id(p)).last_scored_step)
                return frame, todo[: self.slot_chunk]
        return None, []

    # -- evidence ---------------------------------------------------------
    def _ema(self, old: float, new: float) -> float:
        return self.beta * old + (1.0 - self.beta) * float(new)

    def _update_record(self, rec: SlotRecord, *, gain: float, sharp: float, mass: float, repr_drift: float,
                       step: int) -> None:
        first = rec.score_count == 0
        prev_mass = rec.retrieval_mass_ema
        rec.marginal_gain_ema = gain if first else self._ema(rec.marginal_gain_ema, gain)
        rec.utility_ema = max(gain, 0.0) if first else self._ema(rec.utility_ema, max(gain, 0.0))
        rec.sharpness_ema = sharp if first else self._ema(rec.sharpness_ema, sharp)
        rec.retrieval_mass_ema = mass if first else self._ema(rec.retrieval_mass_ema, mass)
        rec.activation_drift_ema = 0.0 if first else self._ema(rec.activation_drift_ema, abs(mass - prev_mass) /
                                                               max(prev_mass, 1e-6))
        rec.representation_drift_ema = repr_drift if first else self._ema(rec.representation_drift_ema, repr_drift)
        rec.contradiction_ema = max(-gain, 0.0) if first else self._ema(rec.contradiction_ema, max(-gain, 0.0))
        rec.peak_utility, rec.peak_sharpness = max(rec.peak_utility, gain), max(rec.peak_sharpness, sharp)
        rec.negative_streak = rec.negative_streak + 1 if gain < 0 else 0
        rec.positive_streak = rec.positive_streak + 1 if gain > 0 else 0
        rec.score_count += 1
        rec.last_scored_step = int(step)
        if rec.state == SLOT_WARMING and rec.score_count >= 2:
            rec.state = SLOT_ACTIVE

    def _capacity_pressure(self, outer: Any) -> bool:
        cap = self.max_slots if self.max_slots is not None else getattr(outer, "max_slots", 0)
        return bool(cap) and outer.table.n_active >= int(cap)

    # -- one tick -----------------------------------------------------------
    def tick(self, *, model: Any, step: int) -> TickResult:
        out = TickResult()
        outer = getattr(model, "outer_model", None)
        self._tick += 1
        self._stats["ticks"] += 1
        if outer is None or getattr(outer, "table", None) is None or not self._frames:
            return out
        t0 = time.monotonic()
        job = None
        if self._sched is not None:
            table0: SlotTable = outer.table
            ids = [table0.physical_to_slot_id(p) for p in table0.visible_indices()]
            job = self._sched.next_job(step, [i for i in ids if i is not None])
            frame = next((f for f in self._frames if job is not None and f.frame_id == job["frame_id"]), None)
            work = ([p for p in (table0.slot_id_to_physical(sid) for sid in job["slot_ids"]) if p is not None]
                    if frame is not None else [])
        else:
            frame, work = self._select_work(outer, step)
        if frame is None:
            if job is not None:
                self._sched.record_result({**job, "status": 1})
            return out
        table: SlotTable = outer.table
        if self.scoring_mode == "oracle":
            o = oracle_confirm_slots(model=model, outer=outer, probe_input_ids=frame.input_ids,
                                     probe_valid_mask=frame.valid_mask, slot_indices=work,
                                     cache_read_cutoff=frame.cache_read_cutoff, variant_chunk_size=self.oracle_chunk)
            gains, mask, idx = o.oracle_deltas, o.mask, o.slot_indices
            weights = torch.full((frame.input_ids.shape[0], len(idx)), 1.0 / max(len(idx), 1))
        else:
            r = counterfactual_probe(model=model, outer=outer, probe_input_ids=frame.input_ids,
                                     probe_valid_mask=frame.valid_mask, probe_cue=frame.cue,
                                     cache_read_cutoff=frame.cache_read_cutoff, chunk_size=self.probe_chunk_size,
                                     score_slot_indices=work)
            gains, mask, idx, weights = r.marginal_gains, r.mask, r.slot_indices, r.weights_baseline
        self._stats["probe_seconds"] += time.monotonic() - t0
        if not idx:
            if job is not None:
                self._sched.record_result({**job, "status": 1})
            return out
        m = mask.float()
        mean_gain = (gains.float() * m).sum((1, 2)) / m.sum().clamp_min(1.0)
        sharp = _per_slot_sharpness(gains.float(), mask)
        mass = weights.float().mean(0)
        pressure = self._capacity_pressure(outer)
        decisions: list[tuple[int, int, SlotRecord, CommitDecision, Optional[torch.Tensor]]] = []
        for j, phys in enumerate(idx):
            sid = table.physical_to_slot_id(phys)
            rec = table.record(sid) if sid is not None else None
            if rec is None or rec.state == SLOT_RETIRED:
                continue
            self._update_record(rec, gain=float(mean_gain[j]), sharp=float(sharp[j]), mass=float(mass[j]),
                                repr_drift=_representation_drift(outer, table.get_tensor(sid)), step=step)
            frame.processed_slots.add(sid)
            self._stats["slots_scored"] += 1
            rule_vals = self.rule.action_values(rec, capacity_pressure=pressure, **self._rule_kw)
            feat = None
            if self.commit_policy == "learned":
                direction = self.controller.step(LearnedCommitPolicy.features(rec, capacity_pressure=pressure),
                                                 slot_dim=table.get_tensor(sid).numel())
                dec, feat = self.learned.choose(rec, controller_state=self.controller.hidden_state(),
                                                rule_values=rule_vals, capacity_pressure=pressure, min_age=self.min_age)
                dec.logits["_controller_dir_norm"] = float(direction.norm())
            else:
                a = max(rule_vals, key=lambda k: rule_vals[k])
                dec = CommitDecision(a, a, 1.0, 1.0, 0.0, dict(rule_vals), {a: 1.0}, dict(rule_vals))
            decisions.append((phys, sid, rec, dec, feat))
            if self.max_seconds > 0 and time.monotonic() - t0 > self.max_seconds:
                self._stats["budget_exhausted"] += 1
                break
        before = (self._stats["oracle_confirmed"], self._stats["oracle_rejected"])
        self._act(model, outer, frame, decisions, step, out)
        if job is not None:
            self._sched.record_result({**job, "status": 0, "slots_scored": len(decisions),
                                       "actions_confirmed": self._stats["oracle_confirmed"] - before[0],
                                       "actions_rejected": self._stats["oracle_rejected"] - before[1],
                                       "probe_seconds": time.monotonic() - t0,
                                       "frame_age_seconds": time.monotonic() - frame.ingested_at})
        self._flush_if_needed()
        return out

    # -- acting -------------------------------------------------------------
    def _agreed(self, sid: int, action: str) -> bool:
        """A mutating action must win ``action_agreement_count`` consecutive ticks for the same slot."""
        prev, n = self._streak.get(sid, ("", 0))
        n = n + 1 if prev == action else 1
        self._streak[sid] = (action, n)
        return n >= self.agreement

    def _act(self, model, outer, frame, decisions, step, out: TickResult) -> None:
        table: SlotTable = outer.table
        want = [(phys, sid, rec, dec, feat) for phys, sid, rec, dec, feat in decisions
                if dec.action in _MUTATING and self._agreed(sid, dec.action)]
        for phys, sid, rec, dec, feat in decisions:
            if dec.action not in _MUTATING:
                self._streak.pop(sid, None)
        confirmed: dict[int, float] = {}
        if want and self.oracle_top_k > 0 and self.scoring_mode == "proxy":
            t0 = time.monotonic()
            top = sorted(want, key=lambda w: -w[3].confidence)[: self.oracle_top_k]
            o = oracle_confirm_slots(model=model, outer=outer, probe_input_ids=frame.input_ids,
                                     probe_valid_mask=frame.valid_mask, slot_indices=[w[0] for w in top],
                                     cache_read_cutoff=frame.cache_read_cutoff, variant_chunk_size=self.oracle_chunk)
            mf = o.mask.float()
            means = (o.oracle_deltas.float() * mf).sum((1, 2)) / mf.sum().clamp_min(1.0)
            confirmed = {int(p): float(v) for p, v in zip(o.slot_indices, means)}
            self._stats["oracle_seconds"] += time.monotonic() - t0
        evict_ids: list[int] = []
        for phys, sid, rec, dec, feat in decisions:
            action, accepted, reason = dec.action, True, ""
            if action in _MUTATING:
                if (phys, sid, rec, dec, feat) not in want:
                    accepted, reason = False, "awaiting_agreement"
                elif self.scoring_mode == "proxy" and self.oracle_top_k > 0:
                    real = confirmed.get(int(phys))
                    if real is None:
                        accepted, reason = False, "not_in_oracle_budget"
                    else:
                        # removing / isolating a slot must not be contradicted by the real dynamics
                        ok = real <= self._rule_kw["useful_threshold"] if action in (SLOT_EVICT, SLOT_QUARANTINE, SLOT_DISTILL) \
                            else real > 0.0
                        accepted, reason = ok, "" if ok else "oracle_contradicts"
                        self._stats["oracle_confirmed" if ok else "oracle_rejected"] += 1
                        if feat is not None:
                            self.learned.apply_feedback(decision=dec, features=feat, reward=1.0 if ok else -1.0)
                if accepted and action == SLOT_QUARANTINE:
                    nq = sum(1 for r in table.active_records() if r.state == SLOT_QUARANTINED)
                    if nq >= self.max_quarantined:
                        accepted, reason = False, "quarantine_full"
            cand_name = ""
            gen0 = int(rec.write_generation)
            if accepted and self.action_mode == "active":
                if action == SLOT_EVICT:
                    evict_ids.append(sid)
                    out.evicted.append(int(sid))
                elif action == SLOT_DECAY:
                    table.scale_survival(sid, 0.9)
                    rec.state = SLOT_DECAYING if rec.state != SLOT_QUARANTINED else rec.state
                    out.decayed.append(int(sid))
                elif action == SLOT_QUARANTINE:
                    table.quarantine(sid)
                    out.quarantined.append(int(sid))
                elif action == SLOT_RELEASE:
                    table.release(sid)
                    out.released.append(int(sid))
                elif action == SLOT_REFRESH:
                    ok, cand_name = self._refresh(model, outer, frame, phys, sid, rec)
                    accepted, reason = ok, "" if ok else "no_candidate_beats_current"
                    if ok:
                        out.refreshed.append(int(sid))
                elif action == SLOT_DISTILL:
                    self._distill(model, outer, sid, rec, step)
                    evict_ids.append(sid)
                    out.distilled.append(int(sid))
                if accepted and action != SLOT_PRESERVE:
                    out.slot_commits.append(self._commit(table, sid, action, step, gen0))
            if accepted:
                rec.last_action = action
                self._counts[action] += 1
            self._event(MemoryEvent(step, self._tick, int(sid), action, rec.marginal_gain_ema, rec.sharpness_ema,
                                    rec.activation_drift_ema, rec.representation_drift_ema, rec.semantic_drift_ema,
                                    rec.contradiction_ema, rec.retrieval_mass_ema, rec.peak_utility, rec.peak_sharpness,
                                    rec.score_count, accepted, reason, cand_name), dec)
        if evict_ids and self.action_mode == "active":
            table.retire_many(evict_ids, reason="maintenance")
            for s in evict_ids:
                self._streak.pop(s, None)

    def _commit(self, table: SlotTable, sid: int, action: str, step: int, base_generation: int) -> SlotCommit:
        """The mutation as an ordered record for the ranks that mirror this table: computed against
        ``base_generation``; slots that are retired at the end of the tick get the next generation."""
        rec = table.record(sid)
        new_gen = int(rec.write_generation) if rec is not None else base_generation
        if action in (SLOT_EVICT, SLOT_DISTILL) or new_gen <= base_generation:
            new_gen = base_generation + 1
        tensor = table.get_tensor(sid).detach().clone() if action == SLOT_REFRESH else None
        return SlotCommit(slot_id=int(sid), action=action, step=int(step), base_generation=int(base_generation),
                          new_generation=new_gen, bucket_id=int(rec.bucket_id if rec else -1),
                          event_id=int(rec.event_id if rec else 0), survival_factor=0.9 if action == SLOT_DECAY else 1.0,
                          tensor=tensor, reason="maintenance")

    def _refresh(self, model, outer, frame, phys: int, sid: int, rec: SlotRecord) -> tuple[bool, str]:
        """CPU proposes, the oracle decides: the best candidate replaces the slot only if it beats it."""
        table: SlotTable = outer.table
        cur = table.get_tensor(sid)
        cue_outer = None
        if frame.cue is not None and getattr(outer, "cue_proj", None) is not None:
            with torch.inference_mode():
                cue_outer = outer.cue_proj(frame.cue.to(outer.cue_proj.weight.dtype)).float().mean(0)
        direction = self.controller.step(LearnedCommitPolicy.features(rec, capacity_pressure=False), slot_dim=cur.numel())
        cands = self.proposals.sample_k(outer=outer, slot=cur, cue_outer=cue_outer, controller_direction=direction)
        r = oracle_confirm_refresh_candidates(model=model, outer=outer, probe_input_ids=frame.input_ids,
                                              probe_valid_mask=frame.valid_mask, slot_index=phys,
                                              candidate_tensors=[(n, t.to(cur.device, cur.dtype)) for n, t in cands],
                                              cache_read_cutoff=frame.cache_read_cutoff,
                                              variant_chunk_size=self.refresh_chunk)
        best = int(r.candidate_improvements.argmax())
        gain = float(r.candidate_improvements[best])
        self.controller.update_feedback(direction, gain * 10.0)
        if best == 0 or gain <= 0.0:
            self.proposals.update(slot=cur, accepted=None, improvement=0.0)
            return False, ""
        new = cands[best][1].to(cur.device, cur.dtype)
        self.proposals.update(slot=cur, accepted=new, improvement=gain)
        table.replace_tensor(sid, new)
        rec.refresh_count += 1
        rec.representation_drift_ema = 0.0
        return True, cands[best][0]

    def _distill(self, model, outer, sid: int, rec: SlotRecord, step: int) -> None:
        """Before a slot the model has absorbed is retired, its content is folded into the bucket
        prototype (when the model keeps prototypes)."""
        protos = getattr(model, "bucket_prototypes_module", None)
        rc = DistillReceipt(int(sid), int(step), rec.marginal_gain_ema, rec.peak_utility, rec.marginal_gain_ema,
                            "bucket_prototype" if protos is not None else "none", accepted=True)
        if protos is not None and rec.bucket_id >= 0 and getattr(outer, "decoder", None) is not None:
            try:
                with torch.inference_mode():
                    vec = outer.decoder(outer.table.get_tensor(sid).to(outer.decoder.weight.dtype)).reshape(-1)
                    if vec.numel() == protos.prototypes.shape[-1]:
                        protos.update(int(rec.bucket_id), vec.float())
                        rc.prototype_updated = True
                    else:
                        rc.prototype_reason = "dim_mismatch"
            except Exception as exc:  # noqa: BLE001
                rc.prototype_reason = f"{type(exc).__name__}"
        self._receipts.append(rc)

    # -- tracing / state ----------------------------------------------------
    def _event(self, ev: MemoryEvent, dec: CommitDecision) -> None:
        self._events.append(ev)
        if len(self._events) > 4096:
            del self._events[:2048]
        if self._trace_path is None or (self._trace_max and self._trace_rows >= self._trace_max):
            return
        row = {"row_type": "arm_slot_decision", **asdict(ev), "rule_action": dec.rule_action,
               "probability": dec.probability, "entropy": dec.entropy, "vetoed_action": dec.vetoed_action,
               "commit_policy": self.commit_policy, "action_mode": self.action_mode}
        self._trace_buf.append(json.dumps(row, separators=(",", ":")) + "\n")
        self._trace_rows += 1

    def _flush_if_needed(self) -> None:
        if len(self._trace_buf) >= self._trace_flush:
            self.flush_trace()

    def flush_trace(self) -> None:
        if self._trace_path is None or not self._trace_buf:
            return
        self._trace_path.parent.mkdir(parents=True, exist_ok=True)
        with self._trace_path.open("a", encoding="utf-8") as fh:
            fh.writelines(self._trace_buf)
        self._trace_buf.clear()

    def close(self) -> None:
        self.flush_trace()
        for h in (self._sched, self._evidence):
            if h is not None:
                h.close()
        self._sched = self._evidence = None

    def recent_events(self, n: int = 64) -> list[MemoryEvent]:
        return self._events[-n:]

    def diagnostics(self) -> dict[str, Any]:
        return {**self._stats, "tick": self._tick, "queue_depth": len(self._frames), "action_counts": dict(self._counts),
                "distill_receipts": len(self._receipts), "controller": self.controller.diagnostics(),
                "commit_policy": self.learned.diagnostics(), "refresh_proposals": self.proposals.diagnostics(),
                "action_mode": self.action_mode, "scoring_mode": self.scoring_mode, "trace_rows": self._trace_rows,
                "arm_runtime": self._sched.diagnostics() if self._sched is not None else {"enabled": False},
                "evidence_engine": self._evidence.diagnostics() if self._evidence is not None else {"enabled": False}}

    def state_dict(self) -> dict[str, Any]:
        """Everything learned or counted (probe frames are transient and not saved)."""
        return {"version": 1, "tick": self._tick, "stats": dict(self._stats), "counts": dict(self._counts),
                "streak": {int(k): [v[0], int(v[1])] for k, v in self._streak.items()},
                "controller": self.controller.state_dict(), "learned": self.learned.state_dict(),
                "proposals": self.proposals.state_dict(),
                "receipts": [asdict(r) for r in self._receipts[-256:]]}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        if int(state.get("version", 0)) != 1:
            raise ValueError(f"unsupported ReplayEvictionLoop state version {state.get('version')!r}")
        self._tick = int(state.get("tick", 0))
        self._stats.update(state.get("stats", {}))
        self._counts.update(state.get("counts", {}))
        self._streak = {int(k): (str(v[0]), int(v[1])) for k, v in state.get("streak", {}).items()}
        self.controller.load_state_dict(state["controller"])
        self.learned.load_state_dict(state["learned"])
        self.proposals.load_state_dict(state["proposals"])
        self._receipts = [DistillReceipt(**r) for r in state.get("receipts", [])]
