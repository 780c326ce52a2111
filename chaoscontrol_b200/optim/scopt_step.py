"""The training step that feeds the scarcity-aware optimizer.

Reference: experiments/23_fast_path/runner_fast_path.py:908-1145 (coalesced dense
sync, activation hooks, pending record) and :6213-6432 (``_run_scopt_train_step``).

Every step: forward, per-token CE, *scarcity pressure* from the CE (rarity x excess
over a per-frequency-bucket baseline), common gradients (mean CE).  Every
``split_interval``-th step additionally: the pressure-weighted *rare* loss, its
gradients w.r.t. the parameters and w.r.t. the activations named in the optimizer's
scarcity maps (one extra reverse walk over the retained graph), per-channel pressure
= mean |d rare / d activation|, the row-pressure EMA.  Everything that replicas must
agree on is averaged across ranks in ONE flat all-reduce per tensor family (rare
gradients, channel pressures, row pressure) with the same SUM + pre-scale
convention as the gradients, so a topology with a non-training rank that submits
zeros works unchanged.  The rare side is staged in a :class:`ScOptPending` and
committed after the gradient clip: a clipped step keeps its row pressure (derived
from CE) but drops its rare gradients and channel pressures (derived from noisy
gradients).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .scopt import FrequencyBucketBaseline, scarcity_pressure_from_ce, scopt_allreduce_config

FUSED_LM_HEAD_MODES = {"fused", "fused_streaming", "fused_streaming_v2", "fused_streaming_cached",
                       "fused_norm_streaming_v2"}


def sync_dense_tensors_coalesced(tensors: list[torch.Tensor], *, world_size: int, all_group=None) -> None:
    """Average same-dtype tensors across the training ranks in place: flatten, pre-scale by
    ``1 / train ranks``, one SUM all-reduce, copy back."""
    if world_size <= 1 or not tensors:
        return
    import torch.distributed as dist
    cfg = scopt_allreduce_config(world_size=world_size, all_group=all_group)
    flat = torch.cat([t.reshape(-1) for t in tensors])
    if cfg.train_grad_scale != 1.0:
        flat.mul_(cfg.train_grad_scale)
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=all_group)
    off = 0
    for t in tensors:
        n = t.numel()
        t.copy_(flat[off: off + n].view_as(t))
        off += n


def activation_keys(optimizer) -> set[str]:
    """Every activation the optimizer's scarcity maps refer to (``<module>.__in__`` / ``.__out__``)."""
    keys: set[str] = set()
    for out_key, in_key in getattr(optimizer, "_matrix_scarcity_map", {}).values():
        keys.update(str(k) for k in (out_key, in_key) if k is not None)
    keys.update(str(k) for k in getattr(optimizer, "_recurrence_scarcity_map", {}).values())
    return keys


def register_activation_hooks(model: nn.Module, keys: set[str]) -> tuple[dict[str, torch.Tensor], list]:
    """Capture the first input (``__in__``) and the output (``__out__``, or the bare module name) of the
    named modules during the next forward; only tensors that require grad are kept."""
    acts: dict[str, torch.Tensor] = {}
    handles: list = []
    modules = dict(model.named_modules())
    bases = {k[: -len(".__in__")] if k.endswith(".__in__") else k[: -len(".__out__")] if k.endswith(".__out__") else k
             for k in keys}

    def pre(key):
        def hook(_m, args):
            if args and isinstance(args[0], torch.Tensor) and args[0].requires_grad:
                acts[key] = args[0]
        return hook

    def post(key):
        def hook(_m, _args, out):
            t = out[0] if isinstance(out, tuple) else out
            if isinstance(t, torch.Tensor) and t.requires_grad:
                acts[key] = t
        return hook

    for base in sorted(bases):
        mod = modules.get(base)
        if mod is None:
            continue
        if f"{base}.__in__" in keys:
            handles.append(mod.register_forward_pre_hook(pre(f"{base}.__in__")))
        if f"{base}.__out__" in keys or base in keys:
            handles.append(mod.register_forward_hook(post(base if base in keys else f"{base}.__out__")))
    return acts, handles


@dataclass
class ScOptPending:
    rare_map: dict[str, torch.Tensor]
    channel_pressure_items: list[tuple[str, torch.Tensor]]
    row_pressure: Optional[torch.Tensor]
    pressure_stats: dict[str, float] = field(default_factory=dict)


def pressure_summary(pressure: torch.Tensor) -> dict[str, float]:
    p = pressure.detach().float().flatten()
    if p.numel() == 0:
        return {"mean": 0.0, "max": 0.0, "p95": 0.0, "frac_positive": 0.0}
    return {"mean": float(p.mean()), "max": float(p.max()), "p95": float(p.quantile(0.95)) if p.numel() > 1 else float(p.max()),
            "frac_positive": float((p > 0).float().mean())}


def writes_enabled(optimizer) -> bool:
    fn = getattr(optimizer, "_writes_enabled", None)
    return bool(fn()) if callable(fn) else True


def should_run_split_step(optimizer, *, step: int, split_interval: int) -> bool:
    return writes_enabled(optimizer) and int(step) % max(1, int(split_interval)) == 0


def apply_pending(optimizer, pending: Optional[ScOptPending], *, skip: bool) -> None:
    """Commit the staged rare side after the clip decision (``skip`` = the step was clipped)."""
    if pending is None:
        return
    optimizer.record_pressure_stats(pending.pressure_stats)
    if pending.row_pressure is not None:
        optimizer.set_row_pressure_ema(pending.row_pressure)
    if skip:
        return
    optimizer.update_rare_grad_ema(pending.rare_map)
    if pending.channel_pressure_items:
        optimizer.set_channel_pressure(dict(pending.channel_pressure_items))


def _allreduce_grads(model: nn.Module, *, world_size: int, all_group) -> None:
    import torch.distributed as dist
    from ..parallel.distributed import allreduce_grads
    cfg = scopt_allreduce_config(world_size=world_size, all_group=all_group)
    if cfg.train_grad_scale != 1.0:
        for p in model.parameters():
            if p.grad is not None:
                p.grad.mul_(cfg.train_grad_scale)
    allreduce_grads(model, world_size, group=all_group, op=dist.ReduceOp.SUM, materialize_zeros=cfg.materialize_zeros)


def run_scopt_train_step(*, model: nn.Module, optimizer, inputs: torch.Tensor, targets: torch.Tensor, step: int,
                         split_interval: int, token_frequencies: torch.Tensor, ddp_active: bool = False,
                         world_size: int = 1, precision: str = "bf16",
                         baseline: FrequencyBucketBaseline | torch.Tensor | float | None = None,
                         pressure_upper_c: Optional[float] = None, pressure_upper_floor: float = 1.0,
                         lm_head_backward_mode: str = "fused", lm_head_tile_size: int = 1024,
                         all_group=None) -> tuple[torch.Tensor, Optional[ScOptPending]]:
    """Returns ``(detached mean CE, pending)``; ``pending`` is None on steps that are not split steps.
    Gradients are left on ``p.grad`` (averaged across ranks).  Call :func:`apply_pending` after the clip."""
    from ..precision import autocast_context
    from ..train_ssm import (_reject_unsupported, fused_lm_head_backend_for_mode, fused_lm_head_loss_with_ce,
                             fused_lm_head_weighted_loss_with_ce)
    _reject_unsupported(model)
    is_split = should_run_split_step(optimizer, step=step, split_interval=split_interval)
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    params = [p for _, p in named]
    acts: dict[str, torch.Tensor] = {}
    handles: list = []
    if is_split:
        acts, handles = register_activation_hooks(model, activation_keys(optimizer))
    mode = str(lm_head_backward_mode).strip().lower()
    with autocast_context(precision, device_type=inputs.device.type):
        try:
            hidden = model.encode(inputs)
        finally:
            for h in handles:
                h.remove()
        fused = mode in FUSED_LM_HEAD_MODES
        if fused:
            backend = fused_lm_head_backend_for_mode(mode)
            total, per_tok = fused_lm_head_loss_with_ce(hidden=hidden, final_norm=model.final_norm, lm_head=model.lm_head,
                                                        targets=targets, backend=backend, tile_size=int(lm_head_tile_size))
            ce = per_tok.reshape_as(targets)
        else:
            logits = model.lm_head(model.final_norm(hidden))
            ce = F.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), targets.reshape(-1),
                                 reduction="none").reshape_as(targets)
            total = ce.mean()
        if isinstance(baseline, FrequencyBucketBaseline):
            base_val: Any = baseline.baseline(targets)
            baseline.update(ce.detach(), targets)
        else:
            base_val = 0.0 if baseline is None else baseline
        pressure = scarcity_pressure_from_ce(ce.detach(), targets, token_frequencies=token_frequencies, baseline=base_val,
                                             upper_c=pressure_upper_c, upper_floor=pressure_upper_floor)
        rare_loss = None
        if is_split:
            if fused:
                rare_loss, _ = fused_lm_head_weighted_loss_with_ce(
                    hidden=hidden, final_norm=model.final_norm, lm_head=model.lm_head, targets=targets,
                    token_weight=pressure, backend=backend, tile_size=int(lm_head_tile_size))
            else:
                rare_loss = (ce * pressure).sum() / pressure.sum().clamp_min(1.0)

    common = torch.autograd.grad(total, params, retain_graph=is_split, allow_unused=True)
    common_unused = {n for (n, _), g in zip(named, common) if g is None}
    for p, g in zip(params, common):
        p.grad = None if g is None else g.detach().contiguous()
    if ddp_active and world_size > 1:
        _allreduce_grads(model, world_size=world_size, all_group=all_group)
    if not is_split:
        return total.detach(), None

    # rare gradients w.r.t. parameters and named activations in one reverse walk
    items = sorted(acts.items())
    uniq: list[torch.Tensor] = []
    where: dict[int, int] = {}
    idx = []
    for _, a in items:
        if id(a) not in where:
            where[id(a)] = len(uniq)
            uniq.append(a)
        idx.append(where[id(a)])
    outs = torch.autograd.grad(rare_loss, [*params, *uniq], retain_graph=False, allow_unused=True)
    rare, act_grads = outs[: len(params)], outs[len(params):]
    extra = {n for (n, _), g in zip(named, rare) if g is None} - common_unused
    if extra:
        raise RuntimeError("ScOpt: parameters have common-loss gradients but no rare-loss gradients (graph "
                           f"disconnect?): {sorted(extra)}")
    rare_map = {n: g.detach().contiguous() for (n, _), g in zip(named, rare) if g is not None}
    sync = ddp_active and world_size > 1
    if sync and rare_map:
        by_dtype: dict[torch.dtype, list[torch.Tensor]] = {}
        for t in rare_map.values():
            by_dtype.setdefault(t.dtype, []).append(t)
        for group in by_dtype.values():
            sync_dense_tensors_coalesced(group, world_size=world_size, all_group=all_group)
    channel = []
    for (key, _a), i in zip(items, idx):                       # sorted keys: every rank reduces in the same order
        dh = act_grads[i]
        if dh is not None:
            channel.append((key, dh.detach().float().abs().mean(dim=tuple(range(max(0, dh.ndim - 1))))))
    if sync and channel:
        sync_dense_tensors_coalesced([v for _, v in channel], world_size=world_size, all_group=all_group)
    row = optimizer.update_row_pressure_ema(targets, pressure, vocab_size=int(token_frequencies.numel()))
    if row is not None and sync:
        sync_dense_tensors_coalesced([row], world_size=world_size, all_group=all_group)
    return total.detach(), ScOptPending(rare_map, channel, row, pressure_summary(pressure))
