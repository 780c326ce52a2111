"""Metabolic gate: when surprise is high, spend extra compute on K candidate
futures (cf. src/chaoscontrol/metabolic.py:20-474).

``metabolic_fork``         pick-best: K perturbed rollouts, scored, winner returned.
``metabolic_monte_carlo``  distributional: the ensemble statistics are the signal.
``micro_mcts``             forward-only tree search over the top next tokens using
                           ``model.step`` (the recurrence alone) as world model.
``StructuredProjections``  K learned views of the input instead of Gaussian noise.

The K candidates are independent, so they run as ONE stacked ``[K*B, T, D]``
pass through the layers and the head (one launch sequence instead of K), and
the tree search advances all of its rollouts' batch rows in the same calls.
``model`` is duck-typed: ``embed``, ``outer_model``, ``layers``,
``final_norm``, ``lm_head`` (and ``init_state`` / ``step`` for the search).
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["metabolic_fork", "metabolic_monte_carlo", "micro_mcts", "StructuredProjections"]


class StructuredProjections(nn.Module):
    """K bias-free linear views of ``x``: "choosing the question"."""

    def __init__(self, dim: int, k: int = 4) -> None:
        super().__init__()
        self.projections = nn.ModuleList(nn.Linear(dim, dim, bias=False) for _ in range(k))

    def forward(self, x: torch.Tensor) -> list[torch.Tensor]:
        return [p(x) for p in self.projections]


def _candidates(model, input_ids, k, noise_std, generation_mode, structured_proj):
    """``(logits [K,B,T,V], hidden [K,B,T,D])`` from one stacked pass."""
    from .models.memory import MultiSlotOuterModel
    x = model.embed(input_ids)
    B = x.shape[0]
    if generation_mode == "structured" and structured_proj is not None:
        views = torch.stack(structured_proj(x), 0)
    else:
        views = x.unsqueeze(0) + noise_std * torch.randn(k, *x.shape, device=x.device, dtype=x.dtype)
    K = views.shape[0]
    flat = views.reshape(K * B, *x.shape[1:])
    om = model.outer_model
    if om is not None:
        if isinstance(om, MultiSlotOuterModel):
            read = om.read(K * B, cue=flat.detach().mean(dim=1))
        else:
            read = om.read(K * B)
        flat = flat + read.unsqueeze(1).to(flat.dtype)
    h = flat
    for layer in model.layers:
        h = layer(h)
    logits = model.lm_head(model.final_norm(h))
    return logits.reshape(K, B, *logits.shape[1:]), h.reshape(K, B, *h.shape[1:])


def _agreement_scores(logits: torch.Tensor) -> list[float]:
    mean = logits.mean(dim=0, keepdim=True)
    return (-(logits - mean).pow(2).flatten(1).mean(dim=1)).tolist()


def metabolic_fork(model: Any, input_ids: torch.Tensor, *, k: int = 4, noise_std: float = 0.01,
                   score_mode: str = "memory_consistency", generation_mode: str = "noise",
                   structured_proj: Optional[StructuredProjections] = None,
                   prior_bias: Optional[torch.Tensor] = None) -> dict[str, Any]:
    """Returns the best candidate's ``{"logits", "hidden", "best_idx"}``.

    ``score_mode``: ``ensemble_agreement`` (closest to the ensemble mean),
    ``memory_consistency`` (last hidden state, cue-projected, most similar to
    the stored slots; falls back to agreement without a populated multi-slot
    store) or ``loss_lookahead`` (most confident).  ``prior_bias`` (a regret-
    matching strategy) scales candidate ``i``'s score by ``1 + prior_bias[i]``.
    """
    from .models.memory import MultiSlotOuterModel
    logits, hidden = _candidates(model, input_ids, k, noise_std, generation_mode, structured_proj)
    om = model.outer_model
    if score_mode == "memory_consistency" and isinstance(om, MultiSlotOuterModel) and len(om.table):
        slots = om.table.slot_matrix()
        cue = om.cue_proj(hidden[:, :, -1, :].detach().to(om.cue_proj.weight.dtype))     # [K, B, outer]
        scores = (cue.to(slots.dtype) @ slots.T).flatten(1).mean(dim=1).tolist()
    elif score_mode == "loss_lookahead":
        scores = F.softmax(logits.float(), dim=-1).amax(dim=-1).flatten(1).mean(dim=1).tolist()
    else:
        scores = _agreement_scores(logits.float())
    if prior_bias is not None:
        for i in range(min(len(scores), prior_bias.size(0))):
            scores[i] *= 1.0 + float(prior_bias[i])
    best = max(range(len(scores)), key=scores.__getitem__)
    return {"logits": logits[best], "hidden": hidden[best], "best_idx": best}


def metabolic_monte_carlo(model: Any, input_ids: torch.Tensor, *, k: int = 4, noise_std: float = 0.01,
                          generation_mode: str = "noise",
                          structured_proj: Optional[StructuredProjections] = None) -> dict[str, Any]:
    """Ensemble mean ``logits`` / ``hidden`` plus ``mc_stats``: ``logits_var``
    (per position, across candidates), ``entropy`` of the mean distribution,
    ``agreement`` (1 - normalised variance), ``uncertainty_map`` (normalised
    variance x normalised entropy) and the scalar ``candidate_divergence``
    (mean KL from the ensemble mean to each candidate)."""
    logits, hidden = _candidates(model, input_ids, k, noise_std, generation_mode, structured_proj)
    lf = logits.float()
    mean_logits = lf.mean(dim=0)
    var = lf.var(dim=0).mean(dim=-1)
    mean_probs = F.softmax(mean_logits, dim=-1)
    log_mean = (mean_probs + 1e-10).log()
    entropy = -(mean_probs * log_mean).sum(dim=-1)
    var_n = var / (var.max() + 1e-8)
    cand = F.softmax(lf, dim=-1)
    # KL(candidate || mean), "batchmean" over the batch dimension, averaged over candidates
    kl = (torch.xlogy(cand, cand) - cand * log_mean.unsqueeze(0)).sum(dim=(1, 2, 3)) / lf.shape[1]
    return {
        "logits": mean_logits.to(logits.dtype),
        "hidden": hidden.mean(dim=0),
        "mc_stats": {"logits_var": var, "entropy": entropy, "agreement": 1.0 - var_n,
                     "uncertainty_map": var_n * entropy / math.log(lf.size(-1)),
                     "candidate_divergence": kl.mean()},
    }


def micro_mcts(model: Any, input_ids: torch.Tensor, *, n_rollouts: int = 4, horizon: int = 8, ucb_c: float = 1.41,
               value_proxy: str = "confidence", prior_bias: Optional[torch.Tensor] = None) -> dict[str, Any]:
    """PUCT search over the 8 most likely next tokens (batch-mean logits at the
    last position).  Each rollout forces one root action, then samples
    ``horizon`` tokens through ``model.step`` from the state after the prompt;
    its value is the mean top probability (``confidence``) or its log
    (``neg_ce``) at the last step.  Visited root actions get their last-position
    logit raised by ``visit_fraction * mean_value``.  ``n_rollouts == 0`` is a
    plain forward pass."""
    def _full(x):
        h = x
        for layer in model.layers:
            h = layer(h)
        return model.lm_head(model.final_norm(h)), h

    root_logits, root_hidden = _full(model.embed(input_ids))
    if n_rollouts == 0:
        return {"logits": root_logits, "hidden": root_hidden}
    B, T = input_ids.shape
    k = min(8, root_logits.size(-1))
    mean_last = root_logits[:, -1, :].float().mean(dim=0)
    top_logits, top_actions = torch.topk(mean_last, k)
    prior = F.softmax(top_logits, dim=0).cpu()
    if prior_bias is not None:
        n = min(k, prior_bias.size(0))
        prior[:n] = prior[:n] * prior_bias[:n].cpu()
        prior = prior / prior.sum()
    visits = torch.zeros(k, dtype=torch.long)
    value_sums = torch.zeros(k)
    with torch.no_grad():
        state = model.init_state(B)
        for t in range(T):
            _, _, state = model.step(input_ids[:, t:t + 1], state)
        root_state = [s.clone() for s in state]
        for n_done in range(n_rollouts):
            q = torch.where(visits > 0, value_sums / visits.clamp(min=1), torch.zeros(k))
            ucb = q + ucb_c * prior * math.sqrt(n_done + 1) / (1 + visits.float())
            a = int(ucb.argmax())
            roll_state = [s.clone() for s in root_state]
            tok = top_actions[a].reshape(1, 1).expand(B, 1)
            for _ in range(horizon):
                step_logits, _, roll_state = model.step(tok, roll_state)
                probs = F.softmax(step_logits.float(), dim=-1)
                tok = torch.multinomial(probs, 1)
            conf = probs.amax(dim=-1)
            value = float(conf.mean()) if value_proxy == "confidence" else float(conf.log().mean())
            visits[a] += 1
            value_sums[a] += value
    mean_values = torch.where(visits > 0, value_sums / visits.clamp(min=1), torch.zeros(k))
    total = int(visits.sum())
    root_value = float((mean_values * visits.float()).sum()) / total if total else 0.0
    adjusted = root_logits.clone()
    boost = (visits.float() / max(total, 1) * mean_values).to(device=adjusted.device, dtype=adjusted.dtype)
    seen = (visits > 0).to(adjusted.device)
    adjusted[:, -1, top_actions[seen]] += boost[seen]
    return {"logits": adjusted, "hidden": root_hidden,
            "mcts_stats": {"visit_counts": visits, "mean_values": mean_values, "root_value": root_value}}
