"""The all-features research training loop ("legacy trainer"): criticality
regularisation, metabolic gate (fork / Monte-Carlo / tree search) with fixed,
random or adaptive threshold and regret-matched priors, surprise-gated episodic
consolidation with typed storage and polyphasic write gating, latent-trace
reactivation, compression-consequence routing feedback, semantic-tier and
posterior updates, learned-tokenizer and alignment losses, spectral / bucket
snapshots, and the sleep cycle (public surface of
src/chaoscontrol/training.py:28-1143).

Structure: ``train_chaoscontrol_for_budget`` is a thin loop over small helpers
(gate decision, forward, loss assembly, post-step memory updates), each
testable on its own.  Differences from the reference that are deliberate:
gradients of all ranks are reduced with ONE flat collective; the per-token CE
needed by several consumers of a step is computed once; and when
``sleep_enabled`` the loop actually records wake moments and runs the sleep
cycle every ``sleep_interval`` steps (over the sleeping partitions when
polyphasic scheduling is on).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import random
import time
from pathlib import Path
from typing import Any, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .alignment import compute_alignment_loss
from .data import batch_from_starts, maybe_autocast, maybe_sync_cuda
from .metabolic import StructuredProjections, metabolic_fork, metabolic_monte_carlo, micro_mcts
from .models.core import criticality_loss
from .models.posterior import BucketDelta, GlobalDelta, ResidualCache
from .optim import LAMB, Muon
from .sleep import SleepConfig, SleepCycle
from .wake_cache import WakeCache

__all__ = ["chunked_cross_entropy", "chunked_cross_entropy_mean", "train_chaoscontrol_for_budget",
           "build_chaoscontrol_matrix", "run_chaoscontrol_matrix", "parse_chaoscontrol_args"]


def chunked_cross_entropy(logits_flat: torch.Tensor, targets_flat: torch.Tensor, chunk_size: int = 8192,
                          reduction: str = "mean") -> torch.Tensor:
    """``F.cross_entropy`` for ``[N, V]`` logits that only ever upcasts ``chunk_size`` rows
    to fp32 at a time.  Always returns an fp32 scalar."""
    if reduction not in ("mean", "sum"):
        raise ValueError(f"chunked_cross_entropy: reduction must be 'mean' or 'sum', got {reduction!r}")
    n = logits_flat.size(0)
    if n == 0:
        return F.cross_entropy(logits_flat, targets_flat, reduction=reduction)
    total = logits_flat.new_zeros((), dtype=torch.float32)
    for a in range(0, n, chunk_size):
        total = total + F.cross_entropy(logits_flat[a:a + chunk_size].float(), targets_flat[a:a + chunk_size],
                                        reduction="sum")
    return total / n if reduction == "mean" else total


def chunked_cross_entropy_mean(logits_flat, targets_flat, chunk_size: int = 8192) -> torch.Tensor:
    return chunked_cross_entropy(logits_flat, targets_flat, chunk_size=chunk_size, reduction="mean")


def _resolve_ddp_context(rank: Optional[int], world_size: Optional[int]) -> tuple[int, int]:
    from .parallel.distributed import resolve_ddp_context
    return resolve_ddp_context(rank, world_size)


def _allreduce_grads(params: list[torch.Tensor], world_size: int) -> None:
    """One flat averaged all-reduce for every gradient (a post-backward reduction keeps
    collective order identical on all ranks whatever the autograd graph looked like)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch._utils._flatten_dense_tensors(grads)
    dist.all_reduce(flat)
    flat.div_(world_size)
    for g, s in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
        g.copy_(s)


def _build_optimizer(name: str, model, extras: list[tuple[str, Any]], lr: float, wd: float):
    params = list(model.parameters()) + [p for _, m in extras for p in m.parameters()]
    if name == "adamw":
        return torch.optim.AdamW(params, lr=lr, weight_decay=wd), params
    if name == "lamb":
        return LAMB(params, lr=lr, weight_decay=wd), params
    if name == "muon":
        opt = Muon(params, lr=lr, weight_decay=wd, adamw_lr=lr, adamw_weight_decay=wd)
        named = list(model.named_parameters())
        for prefix, m in extras:
            named += [(f"{prefix}.{n}", p) for n, p in m.named_parameters()]
        opt.bind_param_names(named)
        return opt, params
    raise ValueError(f"Unknown optimizer: {name!r}. Expected one of {{'adamw', 'muon', 'lamb'}}.")


def _n_buckets(model, default: int = 16) -> int:
    w = getattr(model, "wernicke", None)
    if w is None:
        return default
    return int(getattr(w, "total_buckets", None) or getattr(w, "k_max", default))


def _dominant(bucket_ids: torch.Tensor) -> int:
    return int(bucket_ids.detach().reshape(-1).mode().values.item())


def _crit_terms(out: dict, alpha: float, beta: float, target: float) -> torch.Tensor | float:
    """Jacobian criticality penalty; per-layer targets fan out +-0.04 around the global one."""
    if "jacobian_stats" not in out:
        return 0.0
    per_layer = out.get("per_layer_jacobian_stats")
    if per_layer:
        n = len(per_layer)
        return sum(criticality_loss(s, alpha=alpha / n, beta=beta / n,
                                    target_log_sv=math.log(target - 0.04 + 0.08 * i / max(n - 1, 1)))
                   for i, s in enumerate(per_layer))
    return criticality_loss(out["jacobian_stats"], alpha=alpha, beta=beta, target_log_sv=math.log(target))


def _alignment_term(model, tokenizer, out: dict, align_type: str) -> Optional[torch.Tensor]:
    w = getattr(model, "wernicke", None)
    if tokenizer is None or align_type == "none" or w is None or not hasattr(w, "codebook"):
        return None
    if align_type == "diversity":
        return compute_alignment_loss(align_type, projected_tok_entries=tokenizer.codebook, wernicke_entries=w.codebook)
    if align_type in ("contrastive", "distillation") and "bucket_ids" in out:
        return compute_alignment_loss(align_type, projected_tok_embeds=out["hidden"], wernicke_entries=w.codebook,
                                      wernicke_assignments=out["bucket_ids"])
    return None


def _counterfactual_values(model, inputs, targets, k_actions: int, last_logits) -> list[float]:
    """Value (negative CE on the last target) of replacing the final input token with each of
    the ``k_actions`` most likely tokens, from the recurrent state just before it.  All
    alternatives advance as one batch."""
    B = inputs.size(0)
    state = model.init_state(B)
    for t in range(inputs.size(1) - 1):
        _, _, state = model.step(inputs[:, t:t + 1], state)
    top = last_logits.mean(dim=0).topk(k_actions).indices
    toks = top.repeat_interleave(B).unsqueeze(-1)                                        # [k*B, 1]
    logits, _, _ = model.step(toks, [s.repeat(k_actions, 1) for s in state])
    ce = F.cross_entropy(logits.float(), targets[:, -1].repeat(k_actions), reduction="none").reshape(k_actions, B)
    return (-ce.mean(dim=1)).tolist()


def train_chaoscontrol_for_budget(
        model: Any, *, train_tokens: torch.Tensor, train_starts: list[int], seq_len: int, batch_size: int,
        device: torch.device, param_dtype: torch.dtype, budget_seconds: float, base_lr: float, weight_decay: float,
        grad_clip_norm: float, seed: int, crit_reg_alpha: float = 0.01, crit_reg_beta: float = 0.001,
        crit_target_coupling: float = 0.88, metabolic_gate: bool = False, metabolic_k: int = 4,
        metabolic_threshold: float = 0.1, metabolic_threshold_mode: str = "fixed",
        metabolic_score: str = "memory_consistency", metabolic_noise_std: float = 0.01, generation_mode: str = "noise",
        metabolic_mode: str = "fork", mcts_horizon: int = 8, mcts_ucb_c: float = 1.41,
        consolidation_write: str = "last", latent_persistence: bool = False, cfr_enabled: bool = False,
        tokenizer: Any = None, align_type: str = "none", align_weight: float = 0.05, sleep_enabled: bool = False,
        sleep_stages: str = "full_cycle", sleep_interval: int = 256, sleep_budget: int = 128, sleep_n2_budget: int = 64,
        sleep_rem_budget: int = 64, sleep_n2_batches: int = 8, sleep_rem_dreams: int = 4, sleep_rem_length: int = 128,
        sleep_merge_sim_threshold: float = 0.85, sleep_survival_floor: float = 0.1, sleep_rem_reactivate: bool = True,
        polyphasic_enabled: bool = False, polyphasic_n_partitions: int = 4, polyphasic_k_awake: int = 3,
        polyphasic_topology: str = "slot_striped", polyphasic_swap_interval: int = 256, buffer_mode: str = "legacy",
        wernicke_enabled: bool = False, rank: Optional[int] = None, world_size: Optional[int] = None,
        optimizer: str = "adamw", max_steps: Optional[int] = None) -> dict[str, Any]:
    """Trains for ``budget_seconds`` (or ``max_steps``).  Under DDP (``world_size > 1``, process
    group initialised by the caller) parameters are broadcast from rank 0, window starts are
    sharded by stride, the RNG is seeded ``seed + rank`` and gradients are averaged after
    backward.  The fork / tree-search gate modes, structured generation and a trainable
    tokenizer are single-process features."""
    rank, world_size = _resolve_ddp_context(rank, world_size)
    ddp = world_size > 1
    if ddp and metabolic_gate and metabolic_mode in ("fork", "mcts"):
        raise NotImplementedError(f"metabolic_gate=True with metabolic_mode={metabolic_mode!r} is incompatible with "
                                  f"DDP (world_size={world_size}): the candidate forwards differ per rank")
    if ddp and (generation_mode == "structured" or tokenizer is not None):
        raise NotImplementedError(f"DDP (world_size={world_size}) with structured generation or a trainable tokenizer "
                                  "is not supported: those auxiliary modules would drift across ranks")
    if ddp and not (dist.is_available() and dist.is_initialized()):
        raise RuntimeError(f"DDP training requested (world_size={world_size}, rank={rank}) but torch.distributed is "
                           "not initialized")
    structured_proj = (StructuredProjections(dim=model.embed.weight.shape[1], k=metabolic_k).to(device)
                       if generation_mode == "structured" else None)
    if ddp:
        from .parallel.distributed import broadcast_params
        broadcast_params(model)
    extras = ([("structured_proj", structured_proj)] if structured_proj is not None else []) + \
             ([("tokenizer", tokenizer)] if tokenizer is not None else [])
    optimizer_name = optimizer
    opt, all_params = _build_optimizer(optimizer_name, model, extras, base_lr, weight_decay)
    if ddp:
        train_starts = [s for i, s in enumerate(train_starts) if i % world_size == rank]
        if not train_starts:
            raise ValueError(f"DDP rank {rank}/{world_size}: sharded train_starts is empty")
    rng = random.Random(seed + rank)
    V = model.vocab_size
    use_crit = crit_reg_alpha > 0 or crit_reg_beta > 0
    om = getattr(model, "outer_model", None)

    regret_table = None
    if cfr_enabled:
        from .regret import RegretTable
        regret_table = RegretTable(n_buckets=_n_buckets(model), n_actions=metabolic_k)
    wake_cache = WakeCache(max_moments=32, max_hidden_buffer=64) if sleep_enabled else None
    sleep_cycle = SleepCycle(SleepConfig(
        stages=sleep_stages, budget=sleep_budget, n2_budget=sleep_n2_budget, rem_budget=sleep_rem_budget,
        merge_sim_threshold=sleep_merge_sim_threshold, survival_floor=sleep_survival_floor,
        n2_batches=sleep_n2_batches, rem_dreams=sleep_rem_dreams, rem_length=sleep_rem_length,
        rem_reactivate=sleep_rem_reactivate)) if sleep_enabled else None
    scheduler = None
    if polyphasic_enabled and sleep_enabled:
        from .partition import PartitionTopology, PolyphasicScheduler
        k_max = int(getattr(model.wernicke, "k_max", 16)) if getattr(model, "wernicke", None) else 16
        make = {"bucket_owned": PartitionTopology.bucket_owned,
                "bucket_striped": PartitionTopology.bucket_striped}.get(polyphasic_topology, PartitionTopology.slot_striped)
        scheduler = PolyphasicScheduler(make(polyphasic_n_partitions, k_max), polyphasic_k_awake, polyphasic_swap_interval)

    history: list[dict[str, Any]] = []
    spectral_snapshots: list[dict[str, Any]] = []
    bucket_snapshots: list[dict[str, Any]] = []
    loss_ema, threshold = 2.0, metabolic_threshold
    fork_count = steps = sleep_cycles_run = wake_steps = 0
    last_forked, pre_fork_loss = False, 0.0
    prev_bucket: Optional[int] = None
    t0 = time.perf_counter()
    model.train()
    while True:
        stop = (time.perf_counter() - t0 >= budget_seconds and steps > 0) or \
               (max_steps is not None and steps >= max_steps)
        if ddp and steps > 0:
            flag = torch.tensor([float(stop)], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            stop = flag.item() > 0.5
        if stop:
            break
        starts = [train_starts[rng.randrange(len(train_starts))] for _ in range(batch_size)]
        inputs, targets = batch_from_starts(train_tokens, starts, seq_len, device)
        tok_out = None
        if tokenizer is not None:
            tok_out = tokenizer(inputs)
            inputs, targets = tok_out["token_ids"][:, :-1], tok_out["token_ids"][:, 1:]

        # ---- gate decision ---------------------------------------------------------------------
        last_loss = history[-1]["loss"] if history else loss_ema
        surprise_ratio = abs(loss_ema - last_loss) / max(loss_ema, 1e-6) if history else 0.0
        would_fire = surprise_ratio > threshold
        use_fork = metabolic_gate and (rng.random() < metabolic_threshold if metabolic_threshold_mode == "random"
                                       else would_fire)
        if metabolic_threshold_mode == "adaptive" and last_forked and history:
            helped = steps > 0 and last_loss < pre_fork_loss
            threshold = max(0.01, threshold * 0.95) if helped else min(1.0, threshold * 1.05)
        prior = None
        if regret_table is not None and prev_bucket is not None and metabolic_threshold_mode != "random":
            prior = regret_table.get_strategy(prev_bucket % regret_table.n_buckets)

        # ---- forward + loss --------------------------------------------------------------------
        opt.zero_grad(set_to_none=True)
        mc_stats = None
        with maybe_autocast(device, param_dtype):
            if use_fork and metabolic_mode in ("fork", "mcts"):
                if metabolic_mode == "fork":
                    out = metabolic_fork(model, inputs, k=metabolic_k, noise_std=metabolic_noise_std,
                                         score_mode=metabolic_score, generation_mode=generation_mode,
                                         structured_proj=structured_proj, prior_bias=prior)
                else:
                    out = micro_mcts(model, inputs, n_rollouts=metabolic_k, horizon=mcts_horizon, ucb_c=mcts_ucb_c,
                                     prior_bias=prior)
                fork_count += 1
                if use_crit:
                    with torch.no_grad():
                        st = model(inputs, return_jacobian_stats=True)
                    if "jacobian_stats" in st:
                        out["jacobian_stats"] = st["jacobian_stats"]
            else:
                out = model(inputs, return_jacobian_stats=use_crit,
                            memory_write_mode="append_only" if buffer_mode == "append_only" else "none")
            if use_fork and metabolic_mode == "monte_carlo":
                fork_count += 1
                with torch.no_grad():
                    mc_stats = metabolic_monte_carlo(model, inputs, k=metabolic_k, noise_std=metabolic_noise_std,
                                                     generation_mode=generation_mode,
                                                     structured_proj=structured_proj)["mc_stats"]
            flat_logits, flat_targets = out["logits"].reshape(-1, V), targets.reshape(-1)
            if mc_stats is not None:
                tok_ce = F.cross_entropy(flat_logits.float(), flat_targets, reduction="none").reshape(inputs.size(0), -1)
                u = mc_stats["uncertainty_map"]
                ce_loss = (tok_ce * (1.0 + u / (u.mean() + 1e-8))).mean()      # uncertain positions weigh more
            else:
                ce_loss = chunked_cross_entropy(flat_logits, flat_targets)
            loss = ce_loss
            if use_crit:
                loss = loss + _crit_terms(out, crit_reg_alpha, crit_reg_beta, crit_target_coupling)
            if "balance_loss" in out and getattr(model, "wernicke", None) is not None:
                loss = loss + model.wernicke_balance_weight * out["balance_loss"]
            if tok_out is not None:
                loss = loss + tok_out["commit_loss"] + tok_out["recon_loss"]
            a_loss = _alignment_term(model, tokenizer, out, align_type)
            if a_loss is not None:
                loss = loss + align_weight * a_loss
        loss.backward()
        if ddp:
            _allreduce_grads(all_params, world_size)
        if grad_clip_norm > 0.0:
            torch.nn.utils.clip_grad_norm_(all_params, grad_clip_norm)
        opt.step()

        # ---- bookkeeping -----------------------------------------------------------------------
        ce_val = float(ce_loss.detach())
        loss_ema = 0.99 * loss_ema + 0.01 * ce_val
        last_forked = use_fork
        if use_fork:
            pre_fork_loss = last_loss
        rec: dict[str, Any] = {"step": float(steps), "loss": ce_val, "forked": use_fork}
        if tok_out is not None:
            rec["commit_loss"] = float(tok_out["commit_loss"].detach())
            rec["recon_loss"] = float(tok_out["recon_loss"].detach())
        if metabolic_gate:
            rec.update(threshold=threshold, surprise_ratio=surprise_ratio, metabolic_mode=metabolic_mode,
                       gate_fired=use_fork, surprise_would_fire=would_fire)
        if mc_stats is not None:
            rec.update(mc_variance=float(mc_stats["logits_var"].mean()), mc_entropy=float(mc_stats["entropy"].mean()),
                       mc_divergence=float(mc_stats["candidate_divergence"]))
        with torch.no_grad():
            logits_d, hidden_d = out["logits"].detach(), out["hidden"].detach()
            tok_ce_d = None                                           # per-token CE, computed at most once per step

            def per_token_ce():
                nonlocal tok_ce_d
                if tok_ce_d is None:
                    tok_ce_d = F.cross_entropy(logits_d.reshape(-1, V).float(), flat_targets,
                                               reduction="none").reshape(inputs.size(0), -1)
                return tok_ce_d

            if steps % 50 == 0 and not use_fork:
                power = torch.fft.rfft(hidden_d.float(), dim=1).abs().pow(2).mean(dim=(0, 2))
                snap: dict[str, Any] = {"step": int(steps), "power_spectrum": power.cpu().tolist(),
                                        "dominant_freq": int(power[1:].argmax()) + 1 if power.numel() > 1 else 0}
                if "jacobian_stats" in out:
                    snap["lambda_max"] = float(out["jacobian_stats"]["lambda_max"])
                    snap["sv_log_var"] = float(out["jacobian_stats"]["sv_log_var"])
                if "per_layer_jacobian_stats" in out:
                    snap["per_layer_lambda_max"] = [float(s["lambda_max"]) for s in out["per_layer_jacobian_stats"]]
                if getattr(model, "semantic_tier", None) is not None and om is not None and hasattr(om, "table") \
                        and len(om.table):
                    snap["semantic_norm"] = float(model.semantic_tier.bases.norm())
                    snap["episodic_norm"] = float(om.table.slot_matrix().norm())
                spectral_snapshots.append(snap)
            if steps % 50 == 0 and "bucket_ids" in out:
                counts = torch.bincount(out["bucket_ids"].detach().reshape(-1), minlength=_n_buckets(model, 1))
                bucket_snapshots.append({"step": int(steps), "bucket_counts": counts.cpu().tolist(),
                                         "active_buckets": int((counts > 0).sum())})

            # ---- episodic consolidation --------------------------------------------------------
            bucket: Optional[int] = None
            if om is not None and buffer_mode != "append_only":
                sample_ce = per_token_ce().mean(dim=1)
                if "bucket_ids" in out and getattr(model, "typed_storage", False):
                    bucket = _dominant(out["bucket_ids"])
                allowed = not (scheduler is not None and bucket is not None
                               and not om.is_write_allowed(bucket, scheduler.topology.partitions))
                avg = om.loss_ema.item()
                if consolidation_write == "full_sequence" and hasattr(om, "write_sequence"):
                    sig = om.compute_consolidation_signal(ce_val, avg)
                    if allowed and avg > 0 and sig / avg > 0.01:
                        om.write_sequence(hidden_d, per_sample_weights=sample_ce, bucket_id=bucket)
                    om.update_survival(ce_val)
                    om.loss_ema = om.ema_decay * om.loss_ema + (1 - om.ema_decay) * ce_val
                elif allowed:
                    sig = om.consolidation_step(hidden_d[:, -1, :], current_loss=ce_val, per_sample_weights=sample_ce,
                                                bucket_id=bucket)
                    avg = om.loss_ema.item()
                else:
                    sig = om.compute_consolidation_signal(ce_val, avg)
                rec["surprise"] = float(sig)
                ratio = float(sig) / max(avg, 1e-6)
                if latent_persistence and hasattr(om, "try_reactivate") and ratio > threshold:
                    if om.try_reactivate(bucket_id=bucket, surprise=ratio):
                        rec["latent_reactivated"] = True
                cc = getattr(om, "_compression_consequences", None)
                if cc is not None:
                    if getattr(model, "compression_consequence", False) and getattr(model, "wernicke", None) is not None:
                        for b, dq in cc:
                            model.wernicke.compression_consequence_update(b, dq)
                    cc.clear()
            elif om is not None and "bucket_ids" in out:
                bucket = _dominant(out["bucket_ids"])

            # ---- regret update -----------------------------------------------------------------
            cfr_bucket = bucket if bucket is not None else prev_bucket
            if regret_table is not None and use_fork and cfr_bucket is not None:
                k_act = min(metabolic_k, V)
                cf = _counterfactual_values(model, inputs, targets, k_act, logits_d[:, -1, :])
                if "best_idx" in out:
                    taken = int(out["best_idx"])
                elif "mcts_stats" in out:
                    taken = int(out["mcts_stats"]["visit_counts"].argmax())
                else:
                    taken = 0
                cf = (cf + [-ce_val] * regret_table.n_actions)[: regret_table.n_actions]
                regret_table.update(bucket_id=cfr_bucket % regret_table.n_buckets, action_taken=min(taken, k_act - 1),
                                    counterfactual_values=cf, actual_value=-ce_val)

            # ---- semantic tier / posterior ------------------------------------------------------
            if getattr(model, "semantic_tier", None) is not None and om is not None and hasattr(om, "table") \
                    and len(om.table):
                rows = list(range(len(om.table)))
                if getattr(model, "typed_consolidation", False) and bucket is not None:
                    rows = [i for i, b in enumerate(om._slot_buckets) if b == bucket] or rows
                recent = om.table.slot_matrix(rows[-5:])
                model.semantic_tier.consolidate_from_episodes(om.decoder(recent.to(om.decoder.weight.dtype)))
            post = getattr(model, "posterior", None)
            if post is not None:
                w = per_token_ce()
                err = ((w / w.sum().clamp_min(1e-8)).unsqueeze(-1) * hidden_d.float()).sum(dim=(0, 1))
                if isinstance(post, GlobalDelta):
                    post.update(err)
                elif isinstance(post, BucketDelta):
                    post.update(_dominant(out["bucket_ids"]) if "bucket_ids" in out else 0, err)
                elif isinstance(post, ResidualCache):
                    post.store(hidden_d.float().mean(dim=(0, 1)), err)

            # ---- wake cache / sleep --------------------------------------------------------------
            if wake_cache is not None:
                wake_cache.record_moment(surprise=rec.get("surprise", ce_val), inputs=inputs, targets=targets,
                                         hidden=hidden_d[:, -1, :], bucket_ids=out.get("bucket_ids"))
                if "bucket_ids" in out:
                    wake_cache.update_bucket_counts(out["bucket_ids"])
        if bucket is not None:
            prev_bucket = bucket
        history.append(rec)
        steps += 1
        wake_steps += 1
        if scheduler is not None:
            scheduler.step()
        if sleep_cycle is not None and wake_steps >= sleep_interval and om is not None and hasattr(om, "table"):
            model.eval()
            parts = scheduler.sleeping() if scheduler is not None else [None]
            for part in parts:
                sleep_cycle.run(model, wake_cache, device, regret_table=regret_table, partition=part)
            model.train()
            sleep_cycles_run += 1
            wake_steps = 0

    maybe_sync_cuda(device)
    if ddp:
        dist.barrier()
    return {"steps": int(steps), "history": history, "elapsed_s": float(time.perf_counter() - t0),
            "fork_count": fork_count,
            "extra_params": sum(p.numel() for p in structured_proj.parameters()) if structured_proj else 0,
            "structured_proj": structured_proj, "spectral_snapshots": spectral_snapshots,
            "bucket_snapshots": bucket_snapshots, "regret_table": regret_table, "sleep_cycles": sleep_cycles_run,
            "peak_vram_mb": torch.cuda.max_memory_allocated(device) / 2 ** 20 if device.type == "cuda" else 0.0,
            "ddp_rank": rank, "ddp_world_size": world_size, "optimizer_type": type(opt).__name__,
            "optimizer_name": optimizer_name}


# ---------------------------------------------------------------------------
# 24-cell matrix and CLI
# ---------------------------------------------------------------------------
def build_chaoscontrol_matrix() -> list[dict[str, Any]]:
    """3 state-matrix modes x 8 (rich-B mode, outer model) rows."""
    rows = [("none", 0, "base"), ("nn", 0, "+nn"), ("hub", 0, "+hub"), ("assembly", 0, "+assembly"),
            ("hybrid", 0, "+hybrid"), ("none", 64, "+outer"), ("nn", 64, "+nn+outer"), ("hub", 64, "+hub+outer")]
    return [{"rich_b_mode": b, "outer_model_dim": o, "label": l, "a_mode": a}
            for a in ("diag", "paired", "full") for b, o, l in rows]


_CELL_TRAIN_KEYS = ("crit_reg_alpha", "crit_reg_beta", "crit_target_coupling", "metabolic_gate", "metabolic_k",
                    "metabolic_threshold", "metabolic_threshold_mode", "metabolic_score", "metabolic_noise_std",
                    "generation_mode", "metabolic_mode", "mcts_horizon", "mcts_ucb_c", "consolidation_write",
                    "latent_persistence", "cfr_enabled")


def run_chaoscontrol_matrix(cfg, *, device: torch.device, param_dtype: torch.dtype, train_tokens: torch.Tensor,
                            train_starts: list[int], eval_tokens: torch.Tensor,
                            eval_starts: list[int]) -> list[dict[str, Any]]:
    """Train + evaluate every matrix cell; results so far are rewritten to ``cfg.output_json`` after
    each cell so a crash loses at most one."""
    from .config import ssm_constructor_kwargs
    from .evaluation import evaluate_chaoscontrol_bpb
    from .models.model import CareStudentLM
    base = {k: v for k, v in vars(cfg).items() if not k.startswith("_")}
    results: list[dict[str, Any]] = []
    cells = build_chaoscontrol_matrix()
    for i, cell in enumerate(cells):
        kw = ssm_constructor_kwargs({**base, **{k: cell[k] for k in ("a_mode", "rich_b_mode", "outer_model_dim")}})
        model = CareStudentLM(**kw).to(device)
        tr = train_chaoscontrol_for_budget(
            model, train_tokens=train_tokens, train_starts=train_starts, seq_len=cfg.seq_len,
            batch_size=cfg.batch_size, device=device, param_dtype=param_dtype, budget_seconds=cfg.budget_seconds,
            base_lr=cfg.base_lr, weight_decay=cfg.weight_decay, grad_clip_norm=cfg.grad_clip_norm, seed=cfg.seed,
            **{k: getattr(cfg, k) for k in _CELL_TRAIN_KEYS})
        ev = evaluate_chaoscontrol_bpb(model, tokens=eval_tokens, eval_starts=eval_starts, batch_size=cfg.batch_size,
                                       seq_len=cfg.seq_len, device=device, warmup=cfg.eval_warmup)
        results.append({**cell, "params": sum(p.numel() for p in model.parameters()),
                        "artifact_bytes": model.artifact_bytes(), "train_steps": tr["steps"],
                        "train_elapsed_s": tr["elapsed_s"], **ev})
        if _resolve_ddp_context(None, None)[0] == 0:
            print(f"[{i + 1}/{len(cells)}] {cell['a_mode']:>6} {cell['label']:<20} bpb={ev['bpb']:.4f}  "
                  f"steps={tr['steps']}  elapsed={tr['elapsed_s']:.1f}s")
            if getattr(cfg, "output_json", None):
                p = Path(cfg.output_json)
                p.parent.mkdir(parents=True, exist_ok=True)
                p.write_text(json.dumps(results, indent=2, default=str))
    return results


def parse_chaoscontrol_args(argv: Optional[list[str]] = None) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="ChaosControl SSM-native experiment")
    p.add_argument("--data-path", required=True)
    p.add_argument("--device", default="auto")
    p.add_argument("--dtype", default="fp16")
    p.add_argument("--seed", type=int, default=1337)
    p.add_argument("--output-json", default=None)
    for name, typ, default in (("model-dim", int, 128), ("num-layers", int, 4), ("ff-mult", int, 2),
                               ("seq-len", int, 128), ("batch-size", int, 4), ("eval-batches", int, 8),
                               ("a-full-rank", int, 8), ("a-full-gamma", float, 0.05), ("outer-model-dim", int, 0),
                               ("budget-seconds", float, 300.0), ("base-lr", float, 2e-3),
                               ("weight-decay", float, 1e-2), ("grad-clip-norm", float, 1.0),
                               ("crit-reg-alpha", float, 0.01), ("crit-reg-beta", float, 0.001),
                               ("crit-target-coupling", float, 0.88), ("stride", int, 64)):
        p.add_argument(f"--{name}", type=typ, default=default)
    p.add_argument("--a-mode", default="diag", choices=["diag", "paired", "full"])
    p.add_argument("--rich-b-mode", default="none", choices=["none", "nn", "hub", "assembly", "hybrid"])
    p.add_argument("--matrix", action="store_true", help="run the 24-cell matrix instead of one configuration")
    return p.parse_args(argv)
