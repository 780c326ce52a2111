"""Structured offline consolidation of the episodic store (N1 / N2 / N3 / REM),
behaviourally equivalent to the reference's ``SleepCycle``
(src/chaoscontrol/sleep.py:22-916):

  N1  mark slots whose survival is still ~0 (written, never tested) as unstable
  N2  leave-one-slot-out utility: CE without the slot minus CE with it, added
      to the slot's survival
  N3  prune slots under the survival floor into latent traces; propose merges of
      near-duplicate slots (similarity x bucket affinity when storage is typed)
  REM greedy dreams seeded from slots, teacher-forced scoring on cached real
      targets, reactivation of latent traces, counterfactual-regret updates,
      validation of the proposed merges (accepted merges raise cross-bucket
      affinity, rejected ones lower it)

How the work is laid out differs.  Leave-one-out and merge validation never
edit the table: they go through the read path's per-sample slot mask and slot
override, so ``G`` hidden-slot variants of a cached batch run as ONE expanded
forward.  Pair similarities are one normalised matmul over the dense slot
matrix.  All dreams advance together as one batch of single-token steps.
"""
from __future__ import annotations

import random as _random
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.nn.functional as F

from .data import maybe_autocast

__all__ = ["SleepConfig", "SleepCycle"]

_REM_STAGES = ("n2_n3_rem_base", "n2_n3_rem_validate", "n2_n3_rem_cfr", "n2_n3_rem_reactivate",
               "n2_n3_rem_all", "full_cycle")


@dataclass
class SleepConfig:
    stages: str = "full_cycle"
    budget: int = 128
    n2_budget: int = 64
    rem_budget: int = 64
    merge_sim_threshold: float = 0.85
    survival_floor: float = 0.1
    n2_batches: int = 8
    rem_dreams: int = 4
    rem_length: int = 128
    rem_validate: bool = True
    rem_cfr: bool = True
    rem_reactivate: bool = True
    loo_group: int = 8          # hidden-slot variants evaluated per expanded forward

    @property
    def use_n1(self) -> bool:
        return self.stages == "full_cycle"

    @property
    def use_n2(self) -> bool:
        return self.stages != "n3_only"

    @property
    def use_n3(self) -> bool:
        return True

    @property
    def use_rem(self) -> bool:
        return self.stages in _REM_STAGES


class SleepCycle:
    """``run(model, cache, device, regret_table=None, partition=None)`` executes the
    configured stages in order and returns per-stage diagnostics plus ``total_ops``."""

    def __init__(self, config: SleepConfig | None = None) -> None:
        self.config = config or SleepConfig()
        self._rng = _random.Random(42)
        self._provisional_merges: list[dict] = []

    # ------------------------------------------------------------------ plumbing
    @staticmethod
    def _autocast_for(model: Any, device):
        dev = device if isinstance(device, torch.device) else torch.device(device)
        return maybe_autocast(dev, next(model.parameters()).dtype)

    @staticmethod
    def _eligible(om: Any, partition: Any | None) -> Optional[set[int]]:
        return None if partition is None else set(om.get_partition_slot_indices(partition))

    def _gather_batches(self, cache: Any, device, partition: Any | None):
        if partition is not None and hasattr(cache, "filter_moments_by_partition"):
            moments = cache.filter_moments_by_partition(partition)
        else:
            moments = cache.moments
        return [(m["inputs"].to(device), m["targets"].to(device))
                for m in moments[: self.config.n2_batches]]

    _gather_n2_batches = _gather_batches

    def _ce_variants(self, model: Any, batches, device, *, masks: Optional[torch.Tensor] = None,
                     override: Optional[tuple[int, torch.Tensor]] = None) -> torch.Tensor:
        """Mean CE over ``batches`` for ``G`` read variants at once.

        ``masks`` ``[G, n_slots]`` (bool, True = visible) gives one variant per row;
        ``None`` is the single unmasked variant.  ``override = (slot, value)``
        makes every variant read ``value`` in place of that slot.  Returns ``[G]``.
        """
        G = 1 if masks is None else masks.shape[0]
        total = torch.zeros(G, dtype=torch.float64)
        with torch.no_grad():
            for inputs, targets in batches:
                b = inputs.shape[0]
                kw: dict[str, Any] = {}
                if masks is not None:
                    kw["memory_slot_mask"] = masks.to(inputs.device).repeat_interleave(b, dim=0)
                if override is not None:
                    kw["memory_slot_override_index"] = override[0]
                    kw["memory_slot_override_values"] = override[1].reshape(1, -1).expand(G * b, -1)
                with self._autocast_for(model, device):
                    hidden = model.encode(inputs.repeat(G, 1), memory_mode="force_on", **kw)
                    logits = model.lm_head(model.final_norm(hidden))
                ce = F.cross_entropy(logits.float().reshape(-1, logits.size(-1)), targets.repeat(G, 1).reshape(-1),
                                     reduction="none").reshape(G, -1).mean(dim=1)
                total += ce.double().cpu()
        return (total / max(len(batches), 1)).float()

    def _compute_mean_ce(self, model: Any, batches, device) -> float:
        return float(self._ce_variants(model, batches, device)[0])

    _score_dream = _compute_mean_ce

    # ------------------------------------------------------------------ entry point
    def run(self, model: Any, cache: Any, device="cpu", regret_table: Any | None = None,
            partition: Any | None = None) -> dict[str, Any]:
        cfg = self.config
        om = model.outer_model
        diag: dict[str, Any] = {"total_ops": 0}
        if om is None or not hasattr(om, "table"):
            diag["skipped"] = "no multislot outer model"
            return diag
        unstable: set[int] = set()
        if cfg.use_n1:
            diag["n1"] = self._n1_transition(om, partition=partition)
            unstable = set(diag["n1"]["unstable_indices"])
        if cfg.use_n2:
            diag["n2"] = self._n2_tag(model, om, cache, device, skip_indices=unstable, partition=partition)
            diag["total_ops"] += diag["n2"].get("ops", 0)
        diag["n3"] = self._n3_rewrite(model, om, partition=partition)
        diag["total_ops"] += diag["n3"].get("ops", 0)
        if cfg.use_rem:
            st = cfg.stages
            diag["rem"] = self._rem_dream(
                model, om, cache, device,
                regret_table=regret_table if st in ("n2_n3_rem_cfr", "n2_n3_rem_all", "full_cycle") else None,
                validate_merges=st in ("n2_n3_rem_validate", "n2_n3_rem_all", "full_cycle"),
                reactivate_on_loss=cfg.rem_reactivate and st in ("n2_n3_rem_reactivate", "n2_n3_rem_all",
                                                                 "full_cycle"),
                partition=partition)
            diag["total_ops"] += diag["rem"].get("ops", 0)
        if model.semantic_tier is not None and len(om.table):
            rows = om.get_partition_slot_indices(partition) if partition is not None else None
            if rows is None or rows:
                slots = om.table.slot_matrix(rows)
                model.semantic_tier.consolidate_from_episodes(om.decoder(slots.to(om.decoder.weight.dtype)))
            diag["semantic_recomputed"] = True
        return diag

    # ------------------------------------------------------------------ N1
    def _n1_transition(self, om: Any, partition: Any | None = None) -> dict[str, Any]:
        ok = self._eligible(om, partition)
        idx = [i for i, s in enumerate(om._survival) if (ok is None or i in ok) and abs(s) < 1e-6]
        return {"unstable_count": len(idx), "unstable_indices": idx}

    # ------------------------------------------------------------------ N2
    def _n2_tag(self, model: Any, om: Any, cache: Any, device, skip_indices: set[int] | None = None,
                partition: Any | None = None) -> dict[str, Any]:
        cfg = self.config
        n = len(om.table)
        if n == 0:
            return {"ops": 0, "slots_scored": 0}
        batches = self._gather_batches(cache, device, partition)
        if not batches:
            return {"ops": 0, "slots_scored": 0, "reason": "no cached batches"}
        baseline = self._compute_mean_ce(model, batches, device)
        skip = skip_indices or set()
        ok = self._eligible(om, partition)
        order = [i for i in range(n) if (ok is None or i in ok) and i not in skip]
        skipped = n - len(order)
        self._rng.shuffle(order)
        order = order[: cfg.n2_budget]
        utilities: list[tuple[int, float]] = []
        for g0 in range(0, len(order), max(1, cfg.loo_group)):
            group = order[g0:g0 + max(1, cfg.loo_group)]
            masks = torch.ones(len(group), n, dtype=torch.bool)
            masks[torch.arange(len(group)), torch.tensor(group)] = False
            ce = self._ce_variants(model, batches, device, masks=masks)
            for slot, c in zip(group, ce.tolist()):
                u = c - baseline
                utilities.append((slot, u))
                om._survival[slot] += u
        return {"ops": len(utilities), "slots_scored": len(utilities), "slots_skipped_unstable": skipped,
                "baseline_ce": baseline, "utilities": utilities}

    # ------------------------------------------------------------------ N3
    def _n3_rewrite(self, model: Any, om: Any, partition: Any | None = None) -> dict[str, Any]:
        cfg = self.config
        t = om.table
        ok = self._eligible(om, partition)
        doomed = [i for i in range(len(t)) if (ok is None or i in ok) and t._survival[i] < cfg.survival_floor]
        for i in doomed:
            om._latent_traces.append({"bucket_id": t._slot_buckets[i], "centroid_contrib": t._store[i:i + 1].clone()})
        if doomed:
            t.retire_many([t.physical_to_slot_id(i) for i in doomed], reason="pruned")
        if om.max_slots > 0:
            del om._latent_traces[: max(0, len(om._latent_traces) - om.max_slots)]
        ops = len(doomed)
        proposals: list[dict[str, Any]] = []
        if len(t) >= 2:
            typed = bool(getattr(model, "typed_storage", False))
            proposals = (self._propose_typed_merges if typed else self._propose_untyped_merges)(
                om, cfg, partition=partition)
        ops += len(proposals)
        committed = 0
        if not cfg.use_rem:
            committed = sum(1 for m in proposals if self._commit_merge(om, m))
            proposals = []
        self._provisional_merges = proposals
        return {"ops": ops, "pruned": len(doomed), "latent_traces_created": len(doomed),
                "merges_proposed": len(proposals) + committed, "merges_committed": committed,
                "slots_remaining": len(t)}

    def _pair_candidates(self, om: Any, rows: list[int], threshold: float):
        """``[(i, j, cosine)]`` for ``i < j`` in ``rows`` with cosine >= threshold,
        from one normalised matmul."""
        if len(rows) < 2:
            return []
        M = F.normalize(om.table.slot_matrix(rows).float(), dim=-1)
        sim = (M @ M.T).cpu()
        iu = torch.triu_indices(len(rows), len(rows), offset=1)
        vals = sim[iu[0], iu[1]]
        keep = torch.where(vals >= threshold)[0]
        return [(rows[int(iu[0, k])], rows[int(iu[1, k])], float(vals[k])) for k in keep.tolist()]

    def _proposal(self, om: Any, a: int, b: int, sim: float) -> dict[str, Any]:
        t = om.table
        return {"idx_a": a, "idx_b": b, "similarity": sim,
                "id_a": t.physical_to_slot_id(a), "id_b": t.physical_to_slot_id(b),
                "slot_a": t._store[a:a + 1].clone(), "slot_b": t._store[b:b + 1].clone(),
                "survival_a": t._survival[a], "survival_b": t._survival[b],
                "bucket_a": t._slot_buckets[a], "bucket_b": t._slot_buckets[b]}

    def _propose_typed_merges(self, om: Any, cfg: SleepConfig, partition: Any | None = None):
        """All pairs, same- and cross-bucket, ranked by ``similarity * max(affinity, 0.01)``;
        each slot joins at most one proposal."""
        ok = self._eligible(om, partition)
        rows = [i for i in range(len(om.table)) if ok is None or i in ok]
        if om._slot_buckets:
            om._ensure_affinity(max(max(om._slot_buckets) + 1, 1))
        b = om._slot_buckets
        scored = sorted(((s * max(om.bucket_affinity(b[i], b[j]), 0.01), i, j, s)
                         for i, j, s in self._pair_candidates(om, rows, cfg.merge_sim_threshold)),
                        key=lambda x: x[0], reverse=True)
        used: set[int] = set()
        out = []
        for _, i, j, s in scored:
            if i in used or j in used:
                continue
            used.update((i, j))
            out.append(self._proposal(om, i, j, s))
        return out

    def _propose_untyped_merges(self, om: Any, cfg: SleepConfig, partition: Any | None = None):
        rows = (om.get_partition_slot_indices(partition) if partition is not None
                else list(range(len(om.table))))
        return self._find_similar_pairs(om, rows, cfg.merge_sim_threshold)

    def _find_similar_pairs(self, om: Any, indices: list[int], threshold: float):
        """First-fit in index order: each slot pairs with its first later partner above threshold."""
        used: set[int] = set()
        out = []
        for i, j, s in sorted(self._pair_candidates(om, indices, threshold)):
            if i in used or j in used:
                continue
            used.update((i, j))
            out.append(self._proposal(om, i, j, s))
        return out

    @staticmethod
    def _merged(m: dict[str, Any]) -> torch.Tensor:
        sa, sb = max(m["survival_a"], 0.01), max(m["survival_b"], 0.01)
        return (sa * m["slot_a"] + sb * m["slot_b"]) / (sa + sb)

    def _commit_merge(self, om: Any, m: dict[str, Any]) -> bool:
        """Slot a becomes the survival-weighted average, slot b retires into a latent
        trace.  Addressed by slot id, so earlier commits cannot misdirect it."""
        t = om.table
        pa, pb = t.slot_id_to_physical(m["id_a"]), t.slot_id_to_physical(m["id_b"])
        if pa is None or pb is None or pa == pb:
            return False
        om._latent_traces.append({"bucket_id": m["bucket_b"], "centroid_contrib": m["slot_b"].clone()})
        t.replace_tensor(m["id_a"], self._merged(m))
        t._survival[pa] = (m["survival_a"] + m["survival_b"]) / 2.0
        t.retire(m["id_b"], reason="merged")
        if om.max_slots > 0:
            del om._latent_traces[: max(0, len(om._latent_traces) - om.max_slots)]
        return True

    def _reject_merge(self, om: Any, m: dict[str, Any]) -> None:
        """Both slots stay exactly as they are: proposals never touched the table."""

    def _validate_merge(self, model: Any, om: Any, m: dict[str, Any], batches, device) -> bool:
        """Accept when CE with (a := merged, b hidden) does not exceed the baseline."""
        if not batches:
            return True
        t = om.table
        pa, pb = t.slot_id_to_physical(m["id_a"]), t.slot_id_to_physical(m["id_b"])
        if pa is None or pb is None:
            return True
        base = self._compute_mean_ce(model, batches, device)
        mask = torch.ones(1, len(t), dtype=torch.bool)
        mask[0, pb] = False
        merged = float(self._ce_variants(model, batches, device, masks=mask, override=(pa, self._merged(m)))[0])
        return merged <= base + 1e-6

    # ------------------------------------------------------------------ REM
    def _rem_dream(self, model: Any, om: Any, cache: Any, device, regret_table: Any | None = None,
                   validate_merges: bool = True, reactivate_on_loss: bool = False,
                   partition: Any | None = None) -> dict[str, Any]:
        cfg = self.config
        t = om.table
        if len(t) == 0:
            return {"ops": 0, "dreams": 0, "reason": "no slots to dream from"}
        pool = om.get_partition_slot_indices(partition) if partition is not None else list(range(len(t)))
        if not pool:
            return {"ops": 0, "dreams": 0, "reason": "no partition slots to dream from"}
        batches = self._gather_batches(cache, device, partition)
        n_dreams = min(cfg.rem_dreams, cfg.rem_budget)
        length = max(0, min(cfg.rem_length, cfg.rem_budget // max(n_dreams, 1)))
        seeds = [pool[d % len(pool)] for d in range(n_dreams)]
        seed_ids = [t.physical_to_slot_id(s) for s in seeds]
        ops = 0
        # all dreams advance together: one batch row per dream, greedy decoding
        with torch.no_grad(), self._autocast_for(model, device):
            seed_h = om.decoder(t.slot_matrix(seeds).to(om.decoder.weight.dtype))
            tok = model.lm_head(model.final_norm(seed_h.unsqueeze(1)).squeeze(1)).argmax(dim=-1, keepdim=True)
            state = model.init_state(len(seeds))
            caches = model.init_kv_caches() if hasattr(model, "init_kv_caches") else None
            tokens = [tok]
            for _ in range(length):
                logits, _h, state = model.dream_step(tok.to(device), state, caches)
                tok = logits.argmax(dim=-1, keepdim=True)
                tokens.append(tok)
        ops += length * len(seeds)
        scores: list[float] = []
        cfr_updates = reactivations = 0
        for d, sid in enumerate(seed_ids):
            if batches:
                score = self._score_dream(model, batches, device)
                scores.append(score)
                pos = t.slot_id_to_physical(sid)
                if pos is not None:
                    t._survival[pos] += (sum(scores) / len(scores) - score) * 0.1
                if reactivate_on_loss and cache.moments:
                    ref = cache.moments[d % len(cache.moments)].get("surprise", 1.0)
                    if ref > 0 and score / ref > 1.0:
                        bucket = t._slot_buckets[pos] if pos is not None else None
                        if om.try_reactivate(bucket_id=bucket, surprise=score / ref):
                            reactivations += 1
                            scores[-1] = min(score, self._score_dream(model, batches, device))
                            ops += 1
            if regret_table is not None and batches and len(tokens) >= 2:
                pos = t.slot_id_to_physical(sid)
                bucket = t._slot_buckets[pos] if pos is not None else 0
                cfr_updates += self._cfr_update(model, device, regret_table, bucket,
                                                [s[d:d + 1] for s in state], tokens[-1][d:d + 1])
                ops += 1
        accepted = rejected = 0
        if validate_merges:
            for m in self._provisional_merges:
                if ops >= cfg.rem_budget:               # out of budget: commit unvalidated
                    accepted += int(self._commit_merge(om, m))
                    continue
                good = self._validate_merge(model, om, m, batches, device)
                ba, bb = m.get("bucket_a", -1), m.get("bucket_b", -1)
                cross = bool(batches) and ba != bb and ba >= 0 and bb >= 0
                if good:
                    if self._commit_merge(om, m):
                        accepted += 1
                        if cross:
                            om.update_affinity(ba, bb, delta=1.0)
                else:
                    self._reject_merge(om, m)
                    rejected += 1
                    if cross:
                        om.update_affinity(ba, bb, delta=-1.0)
                ops += 1
            self._provisional_merges = []
        return {"ops": ops, "dreams": len(scores), "mean_dream_score": sum(scores) / len(scores) if scores else 0.0,
                "cfr_updates": cfr_updates, "reactivations": reactivations, "merges_accepted": accepted,
                "merges_rejected": rejected}

    def _cfr_update(self, model: Any, device, regret_table: Any, bucket_id: int, state, last_token,
                    k: int = 4) -> int:
        """Value of the greedy continuation vs ``k`` alternatives sampled at
        temperature 1.5 (value = top next-token probability); action 0 is the one taken.
        The alternatives run as one batch of ``k`` rows."""
        with torch.no_grad(), self._autocast_for(model, device):
            base_logits, _, _ = model.dream_step(last_token.to(device), state)
            base_value = float(F.softmax(base_logits.float(), dim=-1).amax(dim=-1).mean())
            alt = torch.multinomial(F.softmax(base_logits.float() / 1.5, dim=-1), k, replacement=True).reshape(k, 1)
            cf_logits, _, _ = model.dream_step(alt, [s.expand(k, -1).contiguous() for s in state])
            cf = F.softmax(cf_logits.float(), dim=-1).amax(dim=-1).tolist()
        bucket = max(int(bucket_id), 0) % regret_table.n_buckets
        cf = (cf + [base_value] * regret_table.n_actions)[: regret_table.n_actions]
        regret_table.update(bucket_id=bucket, action_taken=0, counterfactual_values=cf, actual_value=base_value)
        return 1
