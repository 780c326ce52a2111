"""Production train + eval entry point (one process per GPU, launched by
``torch.distributed.run``):

    python -m torch.distributed.run --nproc-per-node N -m chaoscontrol_b200.runner_fast_path \\
        --config cfg.yaml --data-path DIR --sp-model-path tok.model --output-json out.json

Same contract as the reference's runner (experiments/23_fast_path/
runner_fast_path.py: ``run_condition`` :14201, ``train_fast_for_budget`` :10513,
``_run_train_step`` :9646, ``_build_optimizer`` :600, ``_warmup`` :13975): YAML
config -> model -> optional warm-up with state restore -> wall-clock-budgeted
training -> rank-0 evaluation under the weight EMA / slow weights -> atomic JSON
result and checkpoint.

What the hot loop is made of here: the no-autograd kernel engine for the forward
and backward (``train_ssm_step``), the in-kernel peer-memory all-reduce or the
distributed Muon (``distributed_muon: true``) for gradient exchange, flat-buffer
clip / Muon / AdamW kernels, and the pinned double-buffered prefetcher for input.
The only host synchronisation is the stop-flag reduce every
``stop_check_interval`` steps; losses stay on the device until the loop ends.

Research-only options of the reference's loop that have no implementation here
are listed in ``UNSUPPORTED_OPTIONS`` and rejected up front rather than ignored.
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import math
import os
import random
import signal
import sys
import time
from pathlib import Path
from typing import Any, Callable, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import fast_path as FP
from .config import ssm_constructor_kwargs
from .crct import CrctRuntime, crct_train_step
from .episodic.runtime import EpisodicRuntime
from .data import load_fineweb_tokens, load_fineweb_val_tokens, resolve_param_dtype
from .models.core import verify_diag_recurrence
from .models.model import CareStudentLM
from .optim import LAMB, Muon
from .optim.param_groups import build_optimizer_params
from .optim.schedule import eval_with_ema, wrap_optimizer_step
from .parallel.distributed import (allreduce_grads, broadcast_params, clip_arena_grad_norm, clip_grad_norm_fused,
                                   should_stop_now)
from .train_ssm import _FUSED_LM_HEAD_BACKENDS, _reject_unsupported, train_ssm_step, train_ssm_step_with_ce
from .training_hooks import (CriticalityDistillHook, FastSlowConsolidator, predictive_auxiliary_loss,
                             spectral_regularization_loss, spectral_summary,
                             zero_embedding_grad_until)
from .utils.arena import get_arena

__all__ = ["run_condition", "train_fast_for_budget", "build_model", "main", "UNSUPPORTED_OPTIONS"]

# options that switch on research machinery this runner does not carry
UNSUPPORTED_OPTIONS: tuple[str, ...] = ()      # every research switch of the reference runner is carried
_DREAM_KEYS = ("dreamworld_enabled", "dreamworld_cache_interval", "dreamworld_interval", "dreamworld_weight",
               "dreamworld_prefix_tokens", "dreamworld_replay_tokens", "dreamworld_replay_batch_size",
               "dreamworld_buffer_size", "dreamworld_min_size", "dreamworld_max_age_steps", "event_sleep_enabled",
               "event_sleep_loss_ratio", "event_sleep_pressure_threshold", "event_sleep_ema_decay",
               "event_sleep_warmup_steps", "event_sleep_min_interval", "event_sleep_weight")


# ---------------------------------------------------------------------------
# process set-up
# ---------------------------------------------------------------------------
def _enable_runner_stack_dump_signal() -> None:
    """``kill -USR1 <pid>`` dumps every thread's Python stack to stderr (hang triage)."""
    if hasattr(signal, "SIGUSR1") and not faulthandler.is_enabled():
        try:
            faulthandler.register(signal.SIGUSR1, file=sys.stderr, all_threads=True, chain=False)
        except (ValueError, RuntimeError):        # not the main thread / unsupported platform
            pass


def _init_distributed(world_size_override: Optional[int]) -> tuple[int, int, int]:
    """``(rank, world_size, local_rank)`` from the launcher's environment."""
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    if world_size_override is not None and int(world_size_override) != ws:
        raise ValueError(f"--world-size {world_size_override} does not match the launcher's WORLD_SIZE={ws}")
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if ws > 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo")
    return rank, ws, local


def _pick_device(local_rank: int, name: str) -> torch.device:
    if name == "auto":
        return torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    dev = torch.device(name)
    return torch.device("cuda", local_rank) if dev.type == "cuda" and dev.index is None else dev


def _control_barrier(group, label: str, timeout_s: float = 30.0) -> None:
    """Host-side barrier on the gloo control group with a deadline: a rank that
    never arrives produces an error naming the barrier instead of a silent hang."""
    if group is None:
        return
    import datetime
    try:
        dist.monitored_barrier(group=group, timeout=datetime.timedelta(seconds=timeout_s))
    except RuntimeError as exc:
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        raise RuntimeError(f"control barrier '{label}' timed out after {timeout_s:.0f}s: {exc}") from exc


# ---------------------------------------------------------------------------
# model / optimizer
# ---------------------------------------------------------------------------
def build_model(config: dict[str, Any], device: torch.device, dtype: torch.dtype) -> CareStudentLM:
    return CareStudentLM(**ssm_constructor_kwargs(config)).to(device=device, dtype=dtype)


def _apply_embed_init(model: CareStudentLM, config: dict[str, Any], device: torch.device) -> None:
    """Optional pretrained embedding table (``embed_init_path``: a tensor or ``{"embed": tensor}``)."""
    path = config.get("embed_init_path")
    if not path:
        return
    blob = torch.load(path, map_location="cpu", weights_only=True)
    table = blob["embed"] if isinstance(blob, dict) and "embed" in blob else blob
    if tuple(table.shape) != tuple(model.embed.weight.shape):
        raise ValueError(f"embed_init_path shape {tuple(table.shape)} does not match embed.weight "
                         f"{tuple(model.embed.weight.shape)}")
    with torch.no_grad():
        model.embed.weight.copy_(table.to(device=device, dtype=model.embed.weight.dtype))


def _build_optimizer(config: dict[str, Any], model: torch.nn.Module, *, rank: int = 0) -> torch.optim.Optimizer:
    name = str(config.get("optimizer", "muon")).strip()
    lr, wd = float(config.get("base_lr", 0.128)), float(config.get("weight_decay", 0.01))
    named = list(model.named_parameters())
    params = build_optimizer_params(named, grouping=str(config.get("optimizer_param_grouping", "flat")).strip(),
                                    base_lr=lr, weight_decay=wd,
                                    dynamics_lr_mul=float(config.get("optimizer_dynamics_lr_mul", 0.1)))
    if name == "adamw":
        return torch.optim.AdamW(params, lr=lr, weight_decay=wd)
    if name == "lamb":
        return LAMB(params, lr=lr, weight_decay=wd)
    if name == "muon":
        opt = Muon(params, lr=lr, weight_decay=wd, adamw_lr=lr, adamw_weight_decay=wd,
                   fused=bool(config.get("fused_muon", True)),
                   log_a_beta_coupling=bool(config.get("optimizer_log_a_beta_coupling", False)),
                   log_a_beta_ema=float(config.get("optimizer_log_a_beta_ema", 0.99)),
                   log_a_beta_min=float(config.get("optimizer_log_a_beta_min", 0.5)))
        opt.bind_param_names(named)
        if get_arena(model) is not None:
            opt.bind_arena(get_arena(model))
        wrap_optimizer_step(opt, model=model, target_momentum=float(config.get("muon_momentum", 0.95)),
                            warmup_start=float(config.get("muon_momentum_warmup_start", 0.95)),
                            warmup_steps=int(config.get("muon_momentum_warmup_steps", 0)),
                            weight_ema_decay=float(config.get("weight_ema_decay", 0.0)), is_rank_zero=rank == 0,
                            weight_ema_fake_quant_bits=int(config.get("weight_ema_fake_quant_bits", 0)))
        return opt
    if name == "semantic":
        from .optim.semantic import SemanticOptimizer, semantic_optimizer_config
        opt = SemanticOptimizer(params, lr=lr, weight_decay=wd, adamw_lr=lr, adamw_weight_decay=wd,
                                momentum_min=float(config.get("semantic_momentum_min", 0.5)),
                                **semantic_optimizer_config(model, int(config.get("semantic_layer_index", 0))))
        opt.bind_param_names(named)
        return opt
    if name in {"scopt", "scarcity", "scarcity_aware"}:
        from .optim.scopt import ScarcityAwareOptimizer, scopt_optimizer_config
        opt = ScarcityAwareOptimizer(
            params, lr=lr, weight_decay=wd, adamw_lr=lr, adamw_weight_decay=wd,
            warmup_steps=int(config.get("scopt_warmup_steps", 200)),
            rare_ema_decay=float(config.get("scopt_rare_ema_decay", 0.9)),
            rare_orthogonal_weight=float(config.get("scopt_rare_orthogonal_weight", 1.0)),
            rare_macro_c=float(config.get("scopt_rare_macro_c", 0.5)),
            row_scarcity_power=float(config.get("scopt_row_scarcity_power", 0.5)),
            tau_std_scale=float(config.get("scopt_tau_std_scale", 0.5)),
            **scopt_optimizer_config(model, int(config.get("scopt_layer_index", 0))))
        opt.bind_param_names(named)
        return opt
    raise ValueError(f"unknown optimizer {name!r}")


def _state_dict_clone(model: torch.nn.Module) -> dict[str, torch.Tensor]:
    return {k: v.detach().clone() for k, v in model.state_dict().items() if torch.is_tensor(v)}


def _restore_state_dict(model: torch.nn.Module, saved: dict[str, torch.Tensor]) -> None:
    with torch.no_grad():
        own = model.state_dict()
        for k, v in saved.items():
            own[k].copy_(v)


def _load_checkpoint_into_model_for_runner(model: torch.nn.Module, path: str) -> dict[str, Any]:
    blob = torch.load(path, map_location="cpu", weights_only=False)
    sd = blob.get("model", blob) if isinstance(blob, dict) else blob
    model.load_state_dict(sd, strict=True)
    return {"checkpoint_path": str(path), "online_eval_state": blob.get("online_eval_state") if isinstance(blob, dict) else None}


def _save_output_ckpt(path: str, model: torch.nn.Module, config: dict[str, Any], *, episodic_cache=None,
                      online_eval_state=None) -> None:
    """``{"model": state_dict, "config": config[, "episodic_cache", "online_eval_state"]}``,
    written to a temporary file and renamed."""
    out = Path(path)
    out.parent.mkdir(parents=True, exist_ok=True)
    blob: dict[str, Any] = {"model": {k: (v.detach().cpu() if torch.is_tensor(v) else v)
                                      for k, v in model.state_dict().items()}, "config": dict(config)}
    if episodic_cache is not None:
        blob["episodic_cache"] = episodic_cache
    if online_eval_state:
        blob["online_eval_state"] = online_eval_state
    tmp = out.with_suffix(out.suffix + ".tmp")
    torch.save(blob, tmp)
    tmp.rename(out)


# ---------------------------------------------------------------------------
# training
# ---------------------------------------------------------------------------
def _clip(model: torch.nn.Module, max_norm: float, fused: bool) -> None:
    if max_norm <= 0:
        return
    arena = get_arena(model)
    if arena is not None and arena.grads_fresh:
        clip_arena_grad_norm(arena, max_norm)
        arena.materialize_grads()
    elif fused:
        clip_grad_norm_fused(model.parameters(), max_norm)
    else:
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm)


def _cuda_graph_rejection_reasons(*, device: torch.device, ddp_active: bool, lm_head_backward_mode: str,
                                  optimizer: Optional[torch.optim.Optimizer] = None,
                                  train_sampling_mode: str = "random",
                                  model: Optional[torch.nn.Module] = None) -> list[str]:
    """Why a whole-step capture is not attempted (empty list = capture)
    (runner_fast_path.py:10094-10123).  Data-parallel steps stay eager: the
    peer-memory collectives take a host-incremented epoch as a launch argument,
    which a replay would freeze."""
    reasons: list[str] = []
    if device.type != "cuda" or not torch.cuda.is_available():
        reasons.append("cuda_required")
    if ddp_active:
        reasons.append("ddp_not_supported")
    if str(lm_head_backward_mode).strip().lower() not in _FUSED_LM_HEAD_BACKENDS:
        reasons.append("fused_lm_head_required")
    if optimizer is not None and type(optimizer).__name__ == "ScarcityAwareOptimizer":
        reasons.append("scopt_autograd_grad_not_captured")
    if str(train_sampling_mode).strip().lower() != "random":
        reasons.append("train_sampling_mode_not_supported")
    if model is not None and not reasons:
        from .train_ssm import _engine_for
        if _engine_for(model) is None:             # the autograd fallback is not sync-free
            reasons.append("kernel_engine_required")
    return reasons


def _rejected_cuda_graph_summary(*, mode: str, reasons: list[str], budget_seconds: float, min_total_speedup: float,
                                 max_capture_seconds: float) -> dict[str, Any]:
    summary = FP.summarize_cuda_graph_gate(budget_seconds=budget_seconds, capture_seconds=0.0, warmup_seconds=0.0,
                                           warmup_steps=0, eager_step_seconds=0.0, graph_step_seconds=0.0,
                                           min_total_speedup=min_total_speedup,
                                           max_capture_seconds=max_capture_seconds)
    summary.update({"mode": mode, "accepted": False,
                    "reasons": list(dict.fromkeys([*reasons, *summary["reasons"]]))})
    return summary


def _train_fast_for_budget_cuda_graph(model: torch.nn.Module, *, prefetch: "FP.BatchPrefetcher",
                                      device: torch.device, optimizer: torch.optim.Optimizer, budget_seconds: float,
                                      chunk_size: int, grad_clip_norm: float, fused_grad_clip: bool, rank: int,
                                      seq_len: int, batch_size: int, precision: str, stop_check_interval: int,
                                      stop_margin_seconds: float, max_steps: Optional[int],
                                      lm_head_backward_mode: str, lm_head_tile_size: int, cuda_graph_mode: str,
                                      cuda_graph_min_total_speedup: float, cuda_graph_max_capture_seconds: float,
                                      cuda_graph_warmup_steps: int, embed_freeze_steps: int = 0,
                                      fast_slow: Optional[FastSlowConsolidator] = None,
                                      time_fn: Callable[[], float] = time.perf_counter) -> dict[str, Any]:
    """Single-GPU loop with the forward, backward and gradient clip of a step
    captured once into a CUDA graph and replayed per batch
    (runner_fast_path.py:10221-10510).  Batches land in two static device
    buffers; the optimizer step stays eager so momentum warm-up and the AdamW
    bias corrections (host scalars) keep advancing.  The eager warm-up steps
    and the capture step are real training steps; their wall time is charged to
    the budget and reported through the acceptance gate."""
    model.train()
    losses: list[torch.Tensor] = []
    t0 = time_fn()
    torch.cuda.reset_peak_memory_stats(device)
    static_in, static_tg = (t.contiguous().clone() for t in prefetch.next())

    def fwd_bwd_clip() -> torch.Tensor:
        optimizer.zero_grad(set_to_none=False)
        loss = train_ssm_step(model, static_in, static_tg, chunk_size, ddp_active=False, world_size=1,
                              precision=precision, lm_head_backward_mode=lm_head_backward_mode,
                              lm_head_tile_size=lm_head_tile_size)
        _clip(model, grad_clip_norm, fused_grad_clip)
        return loss

    def load_next() -> None:
        a, b = prefetch.next()
        static_in.copy_(a, non_blocking=True)
        static_tg.copy_(b, non_blocking=True)

    def after_step(n_done: int) -> None:
        if precision == "fp8_fused":
            from .ops.fp8_linear import fused_fp8_flush_all
            fused_fp8_flush_all(model)
        if fast_slow is not None and fast_slow.enabled:
            fast_slow.after_optimizer_step(model, step=n_done)

    warm_n = max(1, int(cuda_graph_warmup_steps))
    eager_times: list[float] = []
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    tw = time_fn()
    done = 0
    with torch.cuda.stream(side):
        for i in range(warm_n):
            if i:                                  # the batch that sized the static buffers trains first
                load_next()
            torch.cuda.synchronize(device)
            ts = time_fn()
            loss = fwd_bwd_clip()
            zero_embedding_grad_until(model, done, embed_freeze_steps)
            optimizer.step()
            torch.cuda.synchronize(device)
            eager_times.append(time_fn() - ts)
            done += 1
            after_step(done)
            losses.append(loss.detach().clone())
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize(device)
    warm_s = time_fn() - tw

    load_next()
    torch.cuda.synchronize(device)
    tc = time_fn()
    graph = torch.cuda.CUDAGraph()
    optimizer.zero_grad(set_to_none=False)
    # thread-local capture mode: the prefetch thread keeps pinning and copying batches meanwhile
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        graph_loss = fwd_bwd_clip()
    torch.cuda.synchronize(device)
    capture_s = time_fn() - tc
    # capture records the launches without running them: replay once so this batch trains too
    graph.replay()
    zero_embedding_grad_until(model, done, embed_freeze_steps)
    optimizer.step()
    done += 1
    after_step(done)
    losses.append(graph_loss.detach().clone())

    steps = 0
    tr = time_fn()
    every = max(1, int(stop_check_interval))
    while True:
        hit_max = max_steps is not None and done >= int(max_steps)
        if steps % every == 0 or hit_max:
            if FP.should_stop_training_loop(steps=done, elapsed_s=time_fn() - t0, budget_seconds=budget_seconds,
                                            stop_margin_seconds=stop_margin_seconds, max_steps=max_steps):
                break
        load_next()
        graph.replay()
        zero_embedding_grad_until(model, done, embed_freeze_steps)
        optimizer.step()
        steps += 1
        done += 1
        after_step(done)
        losses.append(graph_loss.detach().clone())
    torch.cuda.synchronize(device)
    replay_s = time_fn() - tr
    elapsed = time_fn() - t0
    from .ops import _lib as _ops_lib
    _ops_lib.assert_ok()

    hist = torch.stack([l.float() for l in losses]).cpu().tolist()
    eager_step = FP.steady_state_step_seconds(eager_times) if eager_times else warm_s / warm_n
    graph_step = replay_s / max(steps, 1)
    summary = FP.summarize_cuda_graph_gate(budget_seconds=budget_seconds, capture_seconds=capture_s,
                                           warmup_seconds=warm_s, warmup_steps=warm_n,
                                           eager_step_seconds=eager_step, graph_step_seconds=graph_step,
                                           min_total_speedup=cuda_graph_min_total_speedup,
                                           max_capture_seconds=cuda_graph_max_capture_seconds)
    summary.update({"mode": cuda_graph_mode, "replay_steps": steps, "replay_seconds": replay_s,
                    "capture_counted_as_training_step": True, "optimizer_step_captured": False,
                    "eager_step_times": [float(t) for t in eager_times],
                    "eager_warmup_mean_seconds": warm_s / warm_n})
    result: dict[str, Any] = {
        "steps": done, "elapsed_s": elapsed, "rank": rank, "world_size": 1,
        "initial_loss": hist[0], "final_loss": hist[-1], "loss_history": hist,
        "loss_delta": hist[-1] - hist[0] if len(hist) >= 2 else float("nan"),
        "peak_vram_mb": torch.cuda.max_memory_allocated(device) / 2 ** 20,
        "steady_state_step_seconds": graph_step, "train_sampling_mode": "random",
        "lm_head_backward_mode": lm_head_backward_mode, "cuda_graph_mode": cuda_graph_mode,
        "distributed_muon": False, "spectral": spectral_summary(model), "cuda_graph": summary,
    }
    result.update(FP.summarize_train_timing(steps=done, elapsed_s=elapsed, batch_size=batch_size, seq_len=seq_len,
                                            world_size=1))
    if fast_slow is not None:
        result["fast_slow"] = fast_slow.diagnostics(model)
    return result


def train_fast_for_budget(model: torch.nn.Module, *, train_tokens: torch.Tensor, train_num_tokens: int, stride: int,
                          seq_len: int, batch_size: int, device: torch.device, optimizer: torch.optim.Optimizer,
                          budget_seconds: float, chunk_size: int = 64, grad_clip_norm: float = 1.0,
                          fused_grad_clip: bool = True, rank: int = 0, world_size: int = 1, seed: int = 0,
                          precision: str = "bf16", stop_check_interval: int = 4, stop_margin_seconds: float = 2.0,
                          vocab_size: Optional[int] = None, max_steps: Optional[int] = None,
                          compile_full_path: bool = False, prefetch_batches: bool = True,
                          lm_head_backward_mode: str = "fused_streaming_cached", lm_head_tile_size: int = 8192,
                          cuda_graph_mode: str = "none", train_sampling_mode: str = "random",
                          fast_slow: Optional[FastSlowConsolidator] = None, embed_freeze_steps: int = 0,
                          distributed_muon: bool = False, cuda_graph_min_total_speedup: float = 0.05,
                          cuda_graph_max_capture_seconds: float = 30.0, cuda_graph_warmup_steps: int = 3,
                          crct_enabled: bool = False, crct: Optional["CrctRuntime"] = None,
                          replay_eviction_enabled: bool = False, dreamworld_enabled: bool = False,
                          dreamworld_cache_interval: int = 0, dreamworld_interval: int = 0,
                          dreamworld_weight: float = 0.0, dreamworld_prefix_tokens: int = 128,
                          dreamworld_replay_tokens: int = 64, dreamworld_replay_batch_size: int = 0,
                          dreamworld_buffer_size: int = 16, dreamworld_min_size: int = 2,
                          dreamworld_max_age_steps: int = 256, event_sleep_enabled: bool = False,
                          event_sleep_loss_ratio: float = 1.10, event_sleep_pressure_threshold: float = 0.05,
                          event_sleep_ema_decay: float = 0.99, event_sleep_warmup_steps: int = 32,
                          event_sleep_min_interval: int = 8, event_sleep_weight: float = 0.0,
                          criticality: Optional[CriticalityDistillHook] = None,
                          episodic: Optional["EpisodicRuntime"] = None,
                          spectral_reg_lambda_dead: float = 0.0, spectral_reg_lambda_sticky: float = 0.0,
                          spectral_reg_min_a: float = 0.05, spectral_reg_max_a: float = 0.98,
                          predictive_aux_weight: float = 0.0, predictive_aux_horizon: int = 0,
                          predictive_aux_dim: int = 0, scopt_split_interval: int = 4,
                          scopt_baseline_buckets: int = 16, scopt_baseline_decay: float = 0.99,
                          scopt_pressure_upper_c: Optional[float] = None, scopt_pressure_upper_floor: float = 1.0,
                          grad_allreduce_mode: str = "bulk", emit_topology_snapshot: bool = False,
                          scopt_trace_interval_steps: int = 0,
                          time_fn: Callable[[], float] = time.perf_counter, **unused: Any) -> dict[str, Any]:
    """Budgeted hot loop.  Returns the train-result dict (``steps``, ``elapsed_s``,
    ``initial_loss``, ``final_loss``, ``loss_history``, throughput keys,
    ``peak_vram_mb`` ...)."""
    crct_enabled = bool(crct_enabled) or crct is not None
    _reject_unsupported(model, crct_enabled=crct_enabled)
    bad = [k for k in UNSUPPORTED_OPTIONS if unused.get(k)]
    if bad:
        raise NotImplementedError(f"options {bad} are not supported by this runner")
    ar_mode = str(grad_allreduce_mode).strip().lower()
    if ar_mode not in {"bulk", "async_param"}:
        raise ValueError(f"grad_allreduce_mode must be 'bulk' or 'async_param', got {grad_allreduce_mode!r}")
    if ar_mode == "async_param":
        # per-parameter reductions start inside backward: every gradient of the step must come from that
        # one backward pass, reduced symmetrically over all ranks
        clash = [name for name, on in (("crct_enabled", crct_enabled), ("episodic_enabled", episodic is not None),
                                       ("dreamworld_enabled", dreamworld_enabled),
                                       ("distributed_muon", distributed_muon),
                                       ("predictive_aux_weight", float(predictive_aux_weight) > 0.0 and
                                        int(predictive_aux_horizon) > 0),
                                       ("criticality_distill_enabled", criticality is not None)) if on]
        if clash:
            raise ValueError(f"grad_allreduce_mode='async_param' cannot be combined with {clash}")
    if replay_eviction_enabled and not crct_enabled:
        raise ValueError("replay_eviction_enabled needs crct_enabled: slot maintenance runs beside the teacher")
    if event_sleep_enabled and not dreamworld_enabled:
        raise ValueError("event_sleep_enabled requires dreamworld_enabled=True")
    # the scarcity-aware optimizer is fed by its own step (pressure from CE, rare gradients on split steps)
    from .optim.scopt import FrequencyBucketBaseline, ScarcityAwareOptimizer
    scopt_on = isinstance(optimizer, ScarcityAwareOptimizer)
    scopt_freq = scopt_baseline = None
    if scopt_on:
        if crct_enabled or episodic is not None or dreamworld_enabled or distributed_muon:
            raise ValueError("optimizer 'scopt' runs its own training step: not combinable with crct / episodic / "
                             "dreamworld / distributed_muon")
        if ar_mode != "bulk":
            raise ValueError("optimizer 'scopt' requires grad_allreduce_mode='bulk'")
        V = int(vocab_size or model.lm_head.weight.shape[0])
        scopt_freq = torch.bincount(train_tokens[: int(train_num_tokens)].to(torch.int64).clamp_(0, V - 1),
                                    minlength=V).to(device=device, dtype=torch.float32)
        scopt_baseline = FrequencyBucketBaseline(scopt_freq, num_buckets=int(scopt_baseline_buckets),
                                                 decay=float(scopt_baseline_decay), device=device)
    scopt_stats = {"split_steps": 0, "clipped": 0}
    scopt_traces: list[dict[str, Any]] = []
    topo_snapshot = None
    if emit_topology_snapshot:
        from .utils.profiling import topology_snapshot
        topo_snapshot = topology_snapshot()                      # host / GPU wiring of this run, read-only queries
    if dreamworld_enabled and crct_enabled:
        raise ValueError("dreamworld_enabled and crct_enabled cannot be combined in this runner")
    if episodic is not None and (crct_enabled or dreamworld_enabled or criticality is not None):
        raise ValueError("episodic_enabled cannot be combined with crct, dreamworld or criticality distillation")
    if criticality is not None and world_size > 1:
        raise ValueError("criticality_distill_enabled=True is single-rank only: seat masks, the score "
                         "accumulators and the log_a loss are rank-local")
    spectral_on = float(spectral_reg_lambda_dead) > 0.0 or float(spectral_reg_lambda_sticky) > 0.0
    predictive_on = float(predictive_aux_weight) > 0.0 and int(predictive_aux_horizon) > 0
    if predictive_on and (episodic is not None or crct_enabled):
        # the auxiliary gradient is rank-local and is reduced with the main one; the memory-rank
        # topologies reduce with a SUM over a mixed group (runner_fast_path.py:10942-10951)
        raise ValueError("predictive_aux_weight > 0 cannot be combined with episodic_enabled or crct_enabled")
    ddp = world_size > 1
    if ddp:
        broadcast_params(model)
    # CRCT: the memory rank leaves for its service loop; train ranks shrink to the gradient group
    grad_group = None
    if crct is not None and ddp:
        if crct.is_memory_rank:
            B_T = (int(batch_size), int(seq_len))
            out = crct.run_memory_rank(budget_seconds=budget_seconds, stop_margin_seconds=stop_margin_seconds,
                                       max_steps=max_steps, batch_shape=B_T, time_fn=time_fn)
            crct.close()
            out.update({"initial_loss": 0.0, "final_loss": 0.0, "loss_history": [], "crct": crct.diagnostics()})
            return out
        grad_group = crct.train_group
        rank, world_size = crct.topology["train_ranks"].index(rank), crct.grad_world_size
        ddp = world_size > 1
        distributed_muon = False
    epi_idle = episodic is not None and episodic.is_episodic_rank     # this rank only replays
    data_rank, data_world = rank, world_size
    if episodic is not None and ddp:
        data_rank, data_world = (0 if epi_idle else rank), episodic.n_train
        distributed_muon = False
    model.train()
    mode = str(train_sampling_mode).strip().lower()
    # Epoch samplers shard over the ranks that train (data_world): with an episodic or memory rank in
    # the job no shard of the epoch is lost, so the reference's random-sampling-only restriction
    # (experiments/23_fast_path/runner_fast_path.py:10755-10782) is not needed here.
    sampler = {"random": None, "sequential_epoch": FP.SequentialShardedStartSampler(),
               "shuffled_epoch": FP.ShuffledEpochShardedStartSampler(seed=seed)}.get(mode, "bad")
    if sampler == "bad":
        raise ValueError(f"train_sampling_mode must be random, sequential_epoch or shuffled_epoch; got {mode!r}")
    gen = torch.Generator().manual_seed(int(seed) + int(rank))
    prefetch = FP.BatchPrefetcher(tokens=train_tokens[:train_num_tokens], seq_len=seq_len, stride=stride,
                                  batch_size=batch_size, rank=data_rank, world_size=data_world, device=device,
                                  generator=gen, vocab_size=vocab_size, batch_sampler=sampler)
    if prefetch_batches:
        prefetch.prime()
    graph_mode = str(cuda_graph_mode).strip().lower()
    if graph_mode not in {"none", "probe"}:
        prefetch.close()
        raise ValueError(f"cuda_graph_mode must be 'none' or 'probe', got {cuda_graph_mode!r}")
    graph_summary: Optional[dict[str, Any]] = None
    if graph_mode != "none":
        gate = dict(budget_seconds=budget_seconds, min_total_speedup=float(cuda_graph_min_total_speedup),
                    max_capture_seconds=float(cuda_graph_max_capture_seconds))
        why_not = _cuda_graph_rejection_reasons(device=device, ddp_active=ddp,
                                                lm_head_backward_mode=lm_head_backward_mode, optimizer=optimizer,
                                                train_sampling_mode=mode, model=model)
        if crct_enabled:
            why_not.append("crct_not_supported")
        if dreamworld_enabled:
            why_not.append("dreamworld_not_supported")
        if criticality is not None:
            why_not.append("criticality_distill_not_supported")
        if episodic is not None:
            why_not.append("episodic_not_supported")
        if spectral_on or predictive_on:
            why_not.append("auxiliary_loss_not_supported")
        if why_not:
            graph_summary = _rejected_cuda_graph_summary(mode=graph_mode, reasons=why_not, **gate)
        else:
            try:
                return _train_fast_for_budget_cuda_graph(
                    model, prefetch=prefetch, device=device, optimizer=optimizer, budget_seconds=budget_seconds,
                    chunk_size=chunk_size, grad_clip_norm=grad_clip_norm, fused_grad_clip=fused_grad_clip,
                    rank=rank, seq_len=seq_len, batch_size=batch_size, precision=precision,
                    stop_check_interval=stop_check_interval, stop_margin_seconds=stop_margin_seconds,
                    max_steps=max_steps, lm_head_backward_mode=lm_head_backward_mode,
                    lm_head_tile_size=lm_head_tile_size, cuda_graph_mode=graph_mode,
                    cuda_graph_min_total_speedup=float(cuda_graph_min_total_speedup),
                    cuda_graph_max_capture_seconds=float(cuda_graph_max_capture_seconds),
                    cuda_graph_warmup_steps=int(cuda_graph_warmup_steps), embed_freeze_steps=embed_freeze_steps,
                    fast_slow=fast_slow, time_fn=time_fn)
            except RuntimeError as exc:           # capture refused: carry on eagerly with the same prefetcher
                graph_summary = _rejected_cuda_graph_summary(mode=graph_mode, reasons=["capture_failed"], **gate)
                graph_summary["error"] = str(exc)[:500]
            finally:
                if graph_summary is None:
                    prefetch.close()
    dist_opt = None
    if distributed_muon and ddp and isinstance(optimizer, Muon):
        from .parallel import symm
        from .parallel.dist_muon import DistributedMuon
        arena = get_arena(model)
        if arena is not None:
            dist_opt = DistributedMuon(optimizer, arena, comm=symm.active_comm(None), grad_clip_norm=grad_clip_norm)
    # overlapped exchange on the autograd path: hooks launch one all-reduce per parameter during backward
    # (the kernel engine has its own bucketed exchange for the same mode and takes no hooks)
    async_reducer = None
    if ar_mode == "async_param" and ddp and get_arena(model) is None:
        from .parallel.distributed import AsyncGradAllReducer
        async_reducer = AsyncGradAllReducer(model, world_size)
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    losses: list[torch.Tensor] = []
    step_times: list[float] = []
    steps = 0
    epoch_steps = (FP.sequential_epoch_steps(num_tokens=train_num_tokens, seq_len=seq_len, stride=stride,
                                             batch_size=batch_size, world_size=world_size)
                   if mode != "random" else None)
    dream_buffer = dream_gate = None
    dream = {"replays": 0, "event_triggers": 0, "event_replays": 0, "event_decisions": 0, "pressure_sum": 0.0,
             "last_decision": None}
    if dreamworld_enabled:
        from .dreamworld import (DreamReplayBuffer, LossTriggeredReplayEMA, capture_dream_entry,
                                 dreamworld_replay_backward)
        dream_buffer = DreamReplayBuffer(max_entries=int(dreamworld_buffer_size),
                                         max_age_steps=int(dreamworld_max_age_steps))
        if event_sleep_enabled:
            dream_gate = LossTriggeredReplayEMA(decay=float(event_sleep_ema_decay),
                                                warmup_steps=int(event_sleep_warmup_steps))
    event_pending, event_last_replay, queued = False, -10 ** 9, None
    # predictive auxiliary head: a bias-free dim x dim projection with its own AdamW at the trunk's
    # learning rate (runner_fast_path.py:11333-11350); it is a training aid and is not saved
    aux_proj = aux_opt = None
    aux_stats = {"steps": 0, "last_loss": float("nan"), "spectral_steps": 0}
    if predictive_on:
        dim = int(getattr(model, "dim", 0) or model.lm_head.in_features)
        if int(predictive_aux_dim) not in (0, dim):
            raise ValueError("predictive_aux_dim must be 0 or equal to the model dim")
        aux_proj = torch.nn.Linear(dim, dim, bias=False).to(device=device, dtype=next(model.parameters()).dtype)
        aux_opt = torch.optim.AdamW(aux_proj.parameters(), lr=float(optimizer.param_groups[0]["lr"]),
                                    weight_decay=0.0)
        if ddp:
            broadcast_params(aux_proj)

    def aux_backward(inputs: torch.Tensor) -> None:
        """Adds the auxiliary gradients to ``p.grad`` after the main backward: the predictive loss
        through a second (autograd) encoder pass, the spectral hinge straight on ``log_a``."""
        added = False
        if aux_proj is not None:
            aux_opt.zero_grad(set_to_none=True)
            aux = predictive_auxiliary_loss(model.encode(inputs), projection=aux_proj,
                                            horizon=int(predictive_aux_horizon))
            if aux is not None:
                (float(predictive_aux_weight) * aux).backward()
                aux_stats["steps"] += 1
                if steps % 64 == 0:                 # sampled: reading the value waits for the device
                    aux_stats["last_loss"] = float(aux.detach())
                added = True
        if spectral_on:
            reg = spectral_regularization_loss(model, float(spectral_reg_lambda_dead),
                                               float(spectral_reg_lambda_sticky), float(spectral_reg_min_a),
                                               float(spectral_reg_max_a))
            if reg is not None and reg.requires_grad:
                reg.backward()
                aux_stats["spectral_steps"] += 1
                added = True
        arena_now = get_arena(model)
        if added and arena_now is not None and arena_now.grads_fresh:
            arena_now.pull_grads()                  # fold what autograd added into the flat gradient buffer

    sync_teacher = crct is not None and crct.mode == "sync" and crct.world_size > 1
    if sync_teacher:
        stop_check_interval = 1                    # the memory rank mirrors every step: it needs every flag
    t0 = time_fn()
    try:
        while True:
            if steps % max(1, int(stop_check_interval)) == 0:
                local = FP.should_stop_training_loop(steps=steps, elapsed_s=time_fn() - t0,
                                                     budget_seconds=budget_seconds,
                                                     stop_margin_seconds=stop_margin_seconds, max_steps=max_steps)
                if epoch_steps is not None and steps >= epoch_steps:
                    local = True
                if sync_teacher:
                    if crct.signal_stop_sync(local):
                        break
                elif should_stop_now(local, device, ddp, group=grad_group):
                    break
            elif max_steps is not None and steps >= max_steps:
                break
            ts = time_fn()
            inputs, targets = prefetch.next()
            optimizer.zero_grad(set_to_none=True)
            # dream replay: last step's gate decision first, then what this step replays and caches
            dream_entry, dream_w = None, float(dreamworld_weight)
            if dream_buffer is not None:
                if queued is not None:
                    dec, dec_step = queued
                    queued = None
                    dream["event_decisions"] += 1
                    dream["pressure_sum"] += dec.global_pressure
                    dream["last_decision"] = {"step": dec_step, "local_loss": dec.local_loss,
                                              "ema_loss": dec.ema_loss, "global_pressure": dec.global_pressure,
                                              "fire_count": dec.fire_count, "triggered": dec.triggered}
                    if (dec.triggered and dec_step - event_last_replay >= int(event_sleep_min_interval)
                            and len(dream_buffer) >= int(dreamworld_min_size)):
                        dream["event_triggers"] += 1
                        event_pending = True
                have = len(dream_buffer) >= int(dreamworld_min_size)
                scheduled = (have and dreamworld_interval > 0 and dreamworld_weight > 0.0
                             and steps % int(dreamworld_interval) == 0)
                if scheduled or (event_pending and have):
                    dream_entry = dream_buffer.sample(generator=gen, current_step=steps)
                    if event_pending and have:
                        dream["event_replays"] += 1
                        event_pending, event_last_replay = False, steps
                        if float(event_sleep_weight) > 0.0:
                            dream_w = float(event_sleep_weight)
                if dreamworld_cache_interval > 0 and steps % int(dreamworld_cache_interval) == 0:
                    e = capture_dream_entry(model, inputs, step=steps, prefix_tokens=int(dreamworld_prefix_tokens),
                                            replay_tokens=int(dreamworld_replay_tokens))
                    dream_buffer.add(step=e.step, states=e.states, replay_tokens=e.replay_tokens)
            if episodic is not None:
                if epi_idle:
                    loss = torch.zeros((), device=device)
                else:
                    loss, ce_bt, hid = train_ssm_step_with_ce(model, inputs, targets, precision=precision,
                                                              lm_head_backward_mode=lm_head_backward_mode,
                                                              lm_head_tile_size=lm_head_tile_size)
                    episodic.emit(inputs=inputs, targets=targets, per_token_ce=ce_bt, hidden=hid, step=steps)
                replayed = episodic.consume(model, step=steps, lm_head_backward_mode=lm_head_backward_mode,
                                            lm_head_tile_size=lm_head_tile_size)
                arena_now = get_arena(model)
                if replayed and not epi_idle and arena_now is not None and arena_now.grads_fresh:
                    arena_now.pull_grads()          # one rank plays both parts: fold replay into the flat buffer
                episodic.join_gradients(model)
            elif dream_entry is not None and dream_w > 0.0:
                # replay gradients ADD to this step's: reduce once, after both backward passes
                loss = train_ssm_step(model, inputs, targets, chunk_size, ddp_active=False, world_size=world_size,
                                      precision=precision, lm_head_backward_mode=lm_head_backward_mode,
                                      lm_head_tile_size=lm_head_tile_size)
                dreamworld_replay_backward(model, dream_entry, dream_w, lm_head_backward_mode=lm_head_backward_mode,
                                           lm_head_tile_size=lm_head_tile_size,
                                           replay_batch_size=int(dreamworld_replay_batch_size), generator=gen)
                dream["replays"] += 1
                arena_now = get_arena(model)
                if arena_now is not None and arena_now.grads_fresh:
                    arena_now.pull_grads()
                if predictive_on:
                    aux_backward(inputs)
                if ddp and dist_opt is None:
                    allreduce_grads(model, world_size)
                    if aux_proj is not None:
                        allreduce_grads(aux_proj, world_size)
            elif scopt_on:
                from .optim.scopt_step import run_scopt_train_step
                loss, scopt_pending = run_scopt_train_step(
                    model=model, optimizer=optimizer, inputs=inputs, targets=targets, step=steps,
                    split_interval=int(scopt_split_interval), token_frequencies=scopt_freq, ddp_active=ddp,
                    world_size=world_size, precision=precision, baseline=scopt_baseline,
                    pressure_upper_c=scopt_pressure_upper_c, pressure_upper_floor=float(scopt_pressure_upper_floor),
                    lm_head_backward_mode=lm_head_backward_mode, lm_head_tile_size=lm_head_tile_size)
            elif crct_enabled:
                payload = crct_payload = None
                if crct is not None:
                    payload, inputs, targets = crct.begin_step(inputs, targets, steps)
                    crct_payload = payload
                loss = crct_train_step(model, inputs, targets, payload, precision=precision,
                                       lm_head_backward_mode=lm_head_backward_mode,
                                       lm_head_tile_size=lm_head_tile_size)
                if ddp:
                    allreduce_grads(model, world_size, group=grad_group)
            else:
                # a rank-local auxiliary gradient joins before the one reduction of the step
                loss = train_ssm_step(model, inputs, targets, chunk_size,
                                      ddp_active=ddp and dist_opt is None and not predictive_on,
                                      world_size=world_size, precision=precision,
                                      compile_full_path=compile_full_path,
                                      lm_head_backward_mode=lm_head_backward_mode,
                                      lm_head_tile_size=lm_head_tile_size,
                                      grad_allreduce_mode=ar_mode if (async_reducer is not None or
                                                                      get_arena(model) is not None) else "bulk",
                                      async_grad_reducer=async_reducer)
                if predictive_on:
                    aux_backward(inputs)
                    if ddp and dist_opt is None:
                        allreduce_grads(model, world_size)
                        allreduce_grads(aux_proj, world_size)
            if spectral_on and not predictive_on and not epi_idle:
                aux_backward(inputs)               # a function of the weights alone: identical on every rank
            if criticality is not None:
                if criticality.after_backward(model, inputs, targets, step=steps,
                                              lm_head_tile_size=lm_head_tile_size) is not None:
                    arena_now = get_arena(model)
                    if arena_now is not None and arena_now.grads_fresh:
                        arena_now.pull_grads()       # the log_a loss added to p.grad: fold it into the flat buffer
            zero_embedding_grad_until(model, steps, embed_freeze_steps)
            if dist_opt is not None:
                dist_opt.step()                     # reduce (sharded) + clip + owned update + gather
            elif scopt_on:
                # the rare side is committed only when the step was not clipped
                from .optim.scopt_step import apply_pending
                clipped = False
                if grad_clip_norm > 0:
                    total = torch.nn.utils.clip_grad_norm_(model.parameters(), grad_clip_norm)
                    clipped = bool(total > grad_clip_norm)
                    optimizer.record_clip_event(triggered=clipped)
                apply_pending(optimizer, scopt_pending, skip=clipped)
                if scopt_pending is not None:
                    scopt_stats["split_steps"] += 1
                    scopt_stats["clipped"] += int(clipped)
                optimizer.step()
                if int(scopt_trace_interval_steps) > 0 and (steps + 1) % int(scopt_trace_interval_steps) == 0:
                    scopt_traces.append({"step": steps + 1, **optimizer.scarcity_trace()})
            else:
                _clip(model, grad_clip_norm, fused_grad_clip)
                if crct is not None and crct_enabled:
                    crct.apply_plasticity_budget(optimizer, crct_payload)
                optimizer.step()
            if aux_opt is not None:
                if dist_opt is not None and ddp:
                    allreduce_grads(aux_proj, world_size)
                aux_opt.step()
            if precision == "fp8_fused":
                from .ops.fp8_linear import fused_fp8_flush_all
                fused_fp8_flush_all(model)
            if crct is not None:
                crct.after_optimizer_step(steps)
            steps += 1
            if fast_slow is not None and fast_slow.enabled:
                fast_slow.after_optimizer_step(model, step=steps)
            losses.append(loss.detach())
            if dream_gate is not None:
                d = dream_gate.update(loss, threshold=float(event_sleep_loss_ratio),
                                      pressure_threshold=float(event_sleep_pressure_threshold), ddp_active=ddp,
                                      world_size=world_size)
                if d is not None:
                    queued = (d, steps - 1)
            step_times.append(time_fn() - ts)
    finally:
        prefetch.close()
        if async_reducer is not None:
            async_reducer.close()
        if crct is not None:
            crct.close()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    elapsed = time_fn() - t0
    hist = torch.stack([l.float() for l in losses]).cpu().tolist() if losses else []
    result: dict[str, Any] = {
        "steps": steps, "elapsed_s": elapsed, "rank": rank, "world_size": world_size,
        "initial_loss": hist[0] if hist else float("nan"), "final_loss": hist[-1] if hist else float("nan"),
        "loss_history": hist, "peak_vram_mb": (torch.cuda.max_memory_allocated(device) / 2 ** 20
                                               if device.type == "cuda" else 0.0),
        "steady_state_step_seconds": FP.steady_state_step_seconds(step_times) if step_times else float("nan"),
        "train_sampling_mode": mode, "lm_head_backward_mode": lm_head_backward_mode,
        "cuda_graph_mode": str(cuda_graph_mode), "distributed_muon": dist_opt is not None,
        "grad_allreduce_mode": ar_mode,
        "spectral": spectral_summary(model),
    }
    result.update(FP.summarize_train_timing(steps=steps, elapsed_s=elapsed, batch_size=batch_size, seq_len=seq_len,
                                            world_size=world_size))
    if topo_snapshot is not None:
        result["topology_snapshot"] = topo_snapshot
    if fast_slow is not None:
        result["fast_slow"] = fast_slow.diagnostics(model)
    if graph_summary is not None:
        result["cuda_graph"] = graph_summary
    if crct is not None:
        result["crct"] = crct.diagnostics()
    if episodic is not None:
        result["episodic"] = episodic.diagnostics()
        result.update(FP.summarize_train_timing(steps=steps, elapsed_s=elapsed, batch_size=batch_size,
                                                seq_len=seq_len, world_size=world_size, episodic_enabled=ddp))
    if predictive_on:
        result["predictive_aux"] = {"weight": float(predictive_aux_weight), "horizon": int(predictive_aux_horizon),
                                    "steps": aux_stats["steps"], "last_loss": aux_stats["last_loss"],
                                    "projection_norm": float(aux_proj.weight.detach().float().norm())}
    if spectral_on:
        result["spectral"]["regularized_steps"] = aux_stats["spectral_steps"]
    if scopt_on:
        result["scopt"] = {"split_interval": int(scopt_split_interval), "split_steps": scopt_stats["split_steps"],
                           "clipped_split_steps": scopt_stats["clipped"], "trace": optimizer.scarcity_trace()}
        if scopt_traces:
            result["scopt"]["interval_traces"] = scopt_traces
    if criticality is not None:
        result["criticality_distillation"] = criticality.diagnostics()
    if dream_buffer is not None:
        n = max(dream["event_decisions"], 1)
        result["dreamworld"] = {
            "enabled": True, "weight": float(dreamworld_weight), "cache_interval": int(dreamworld_cache_interval),
            "dream_interval": int(dreamworld_interval), "prefix_tokens": int(dreamworld_prefix_tokens),
            "replay_tokens": int(dreamworld_replay_tokens), "replay_batch_size": int(dreamworld_replay_batch_size),
            "replays": dream["replays"], "buffer": dream_buffer.diagnostics(steps),
            "event_sleep": {"enabled": dream_gate is not None, "loss_ratio": float(event_sleep_loss_ratio),
                            "pressure_threshold": float(event_sleep_pressure_threshold),
                            "ema_decay": float(event_sleep_ema_decay),
                            "warmup_steps": int(event_sleep_warmup_steps),
                            "min_interval": int(event_sleep_min_interval), "weight": float(event_sleep_weight),
                            "trigger_count": dream["event_triggers"], "replay_count": dream["event_replays"],
                            "decision_count": dream["event_decisions"],
                            "mean_global_pressure": dream["pressure_sum"] / n,
                            "last_decision": dream["last_decision"]}}
    return result


_LOOP_KEYS = ("chunk_size", "grad_clip_norm", "fused_grad_clip", "precision", "stop_check_interval",
              "stop_margin_seconds", "compile_full_path", "prefetch_batches", "lm_head_backward_mode",
              "lm_head_tile_size", "cuda_graph_mode", "cuda_graph_min_total_speedup",
              "cuda_graph_max_capture_seconds", "cuda_graph_warmup_steps", "train_sampling_mode",
              "embed_freeze_steps", "distributed_muon", "grad_allreduce_mode", "emit_topology_snapshot",
              "scopt_trace_interval_steps", "crct_enabled",
              "replay_eviction_enabled", "spectral_reg_lambda_dead", "spectral_reg_lambda_sticky",
              "spectral_reg_min_a", "spectral_reg_max_a", "predictive_aux_weight", "predictive_aux_horizon",
              "predictive_aux_dim", "scopt_split_interval", "scopt_baseline_buckets", "scopt_baseline_decay",
              "scopt_pressure_upper_c", "scopt_pressure_upper_floor") + _DREAM_KEYS


def _loop_kwargs(config: dict[str, Any]) -> dict[str, Any]:
    return {k: config[k] for k in _LOOP_KEYS if k in config}


def _warmup(*, model, train_tokens, train_num_tokens, stride, seq_len, batch_size, device, optimizer, config, rank,
            world_size, seed, vocab_size) -> None:
    """``warmup_steps`` untimed steps (kernel selection, allocator growth, peer buffers)."""
    steps = int(config.get("warmup_steps", 0))
    if steps <= 0:
        return
    kw = _loop_kwargs(config)
    kw.update(stop_check_interval=1, stop_margin_seconds=0.0, cuda_graph_mode="none")
    train_fast_for_budget(model, train_tokens=train_tokens, train_num_tokens=train_num_tokens, stride=stride,
                          seq_len=seq_len, batch_size=batch_size, device=device, optimizer=optimizer,
                          budget_seconds=300.0, rank=rank, world_size=world_size, seed=seed, vocab_size=vocab_size,
                          max_steps=steps, **kw)


# ---------------------------------------------------------------------------
# run_condition
# ---------------------------------------------------------------------------
_CONTROL: dict[int, Any] = {}


def _control_group(world_size: int):
    """Gloo side group for object / flag collectives, created once per process group."""
    if world_size not in _CONTROL:
        _CONTROL[world_size] = dist.new_group(list(range(world_size)), backend="gloo")
    return _CONTROL[world_size]


def run_condition(config: dict[str, Any], *, data_path: str, sp_model_path: Optional[str], budget_seconds: float,
                  output_json: Optional[str], output_ckpt: Optional[str], world_size_override: Optional[int],
                  val_cache_dir: Optional[str] = None, keep_process_group: bool = False) -> dict[str, Any]:
    """``keep_process_group`` leaves the process group (and the cached control group) alive on return,
    for a warm worker that runs many conditions back to back."""
    _enable_runner_stack_dump_signal()
    rank, world_size, local_rank = _init_distributed(world_size_override)
    ddp = world_size > 1
    control = _control_group(world_size) if ddp else None
    device = _pick_device(local_rank, str(config.get("device", "auto")))
    dtype = resolve_param_dtype(str(config.get("dtype", "bf16")), device)
    seed = int(config.get("seed", 1337))
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    verify_diag_recurrence(device)
    vocab = int(config["vocab_size"])
    eval_only = bool(config.get("eval_only", False))
    calc_types = list(config.get("calc_types") or [])
    if eval_only:
        train_tokens = torch.empty(0, dtype=torch.int16)
        val_tokens = torch.empty(0, dtype=torch.int16) if calc_types else load_fineweb_val_tokens(data_path)
    else:
        train_tokens, val_tokens = load_fineweb_tokens(data_path)
    luts = (None, None, None)
    if sp_model_path:
        import sentencepiece as spm

        from .sp_eval import build_sentencepiece_luts
        sp = spm.SentencePieceProcessor()
        sp.Load(sp_model_path)
        luts = build_sentencepiece_luts(sp, vocab, device)
    seq_len = int(config["seq_len"])
    stride = int(config.get("stride", seq_len // 2))
    batch = int(config["batch_size"])
    eval_batches = int(config.get("eval_batches", 0))
    eval_starts = FP.choose_lm_starts_lazy(num_tokens=int(val_tokens.numel()), seq_len=seq_len, stride=stride,
                                           batch_size=batch, eval_batches=max(0, eval_batches), seed=seed)
    model = build_model(config, device, dtype)
    _apply_embed_init(model, config, device)
    _reject_unsupported(model, crct_enabled=bool(config.get("crct_enabled", False)))
    n_params = sum(p.numel() for p in model.parameters())
    ckpt_meta = None
    if str(config.get("checkpoint_path", "") or "").strip():
        ckpt_meta = _load_checkpoint_into_model_for_runner(model, str(config["checkpoint_path"]).strip())
    elif eval_only:
        raise ValueError("eval_only=True requires config.checkpoint_path")
    if rank == 0:
        print(f"[rank 0/{world_size}] {config.get('name', '<unnamed>')} vocab={vocab} batch={batch} "
              f"params={n_params:,}", flush=True)
    # flat parameter / gradient arena: required by the kernel engine, the flat-buffer optimizer
    # kernels, the peer-memory collectives and the distributed optimizer
    from .engine import TrainEngine
    from .utils.arena import ParamArena
    arena = None
    if TrainEngine.supported(model):
        arena = ParamArena.install(model)
    elif bool(config.get("distributed_muon", False)):
        # sharded Muon without the kernel engine: the arena's shape checks (8-aligned rows / columns,
        # 128-element matrices) decide; a model they reject keeps the replicated optimizer
        try:
            arena = ParamArena.install(model)
        except ValueError as exc:
            if rank == 0:
                print(f"[rank 0/{world_size}] distributed_muon disabled: {exc}", flush=True)
            config = dict(config, distributed_muon=False)
    if ddp and device.type == "cuda" and arena is not None:
        from .parallel import symm_comm
        if not symm_comm.try_enable(arena.flat_grad.numel()) and rank == 0:
            # same answer on every rank (the communicator votes): collectives stay on the library
            print(f"[rank 0/{world_size}] peer-memory collectives unavailable ({symm_comm.last_reason()}); "
                  "using the torch.distributed backend", flush=True)

    train_result: dict[str, Any]
    optimizer = None
    fast_slow = None
    episodic = None
    episodic_cache_blob = None
    if eval_only:
        train_result = {"steps": 0, "elapsed_s": 0.0, "initial_loss": 0.0, "final_loss": 0.0,
                        "aggregate_tokens_per_sec": 0.0, "peak_vram_mb": 0.0, "eval_only": True}
    else:
        common = dict(model=model, train_tokens=train_tokens, train_num_tokens=int(train_tokens.numel()),
                      stride=stride, seq_len=seq_len, batch_size=batch, device=device, rank=rank,
                      world_size=world_size, seed=seed, vocab_size=vocab)
        restore = bool(config.get("restore_after_warmup", False)) and int(config.get("warmup_steps", 0)) > 0
        saved = _state_dict_clone(model) if restore else None
        optimizer = _build_optimizer(config, model, rank=rank)
        _warmup(optimizer=optimizer, config=config, **common)
        if saved is not None:
            _restore_state_dict(model, saved)
            optimizer = _build_optimizer(config, model, rank=rank)
            if ddp:
                dist.barrier()
        fast_slow = FastSlowConsolidator.from_config(model, config)
        common.pop("model")
        max_steps = None if config.get("max_steps") is None else int(config["max_steps"])
        crct = None
        if bool(config.get("crct_enabled", False)):
            crct = CrctRuntime(model=model, config=config, rank=rank, world_size=world_size, device=device,
                               batch_size=batch, seq_len=seq_len, total_steps=max_steps)
        if bool(config.get("episodic_enabled", False)):
            episodic = EpisodicRuntime(model=model, config=config, rank=rank, world_size=world_size, device=device)
        try:
            train_result = train_fast_for_budget(
                model, optimizer=optimizer, budget_seconds=budget_seconds, fast_slow=fast_slow, max_steps=max_steps,
                crct=crct, criticality=CriticalityDistillHook.from_config(model, config), episodic=episodic,
                **common, **_loop_kwargs(config))
            if episodic is not None:
                episodic_cache_blob = episodic.cache_state()
                if ddp:                                   # the cache lives on the episodic rank; rank 0 saves
                    blobs = [None] * world_size if rank == 0 else None
                    dist.gather_object(episodic_cache_blob, blobs, dst=0, group=control)
                    if rank == 0:
                        episodic_cache_blob = next((b for b in blobs if b is not None), None)
        finally:
            if episodic is not None:
                episodic.close()
        if bool(config.get("rare_bucket_ce_enabled", False)):
            freq = torch.bincount(train_tokens.to(torch.int64).clamp_(0, vocab - 1), minlength=vocab)
            is_mem = crct is not None and crct.is_memory_rank
            ev_rank, ev_world = (rank, world_size) if crct is None or not ddp else (
                (0, 1) if is_mem else (crct.topology["train_ranks"].index(rank), crct.grad_world_size))
            if not is_mem and ev_world == world_size:
                train_result.update(FP.compute_per_bucket_val_ce(
                    model=model, device=device, tokens=val_tokens, num_tokens=int(val_tokens.numel()),
                    seq_len=seq_len, stride=stride, batch_size=batch, vocab_size=vocab, token_frequencies=freq,
                    num_buckets=int(config.get("rare_bucket_ce_num_buckets", 4)), rank=ev_rank,
                    world_size=ev_world, precision=str(config.get("precision", "bf16")),
                    max_batches=config.get("rare_bucket_ce_max_batches")))
    if ddp:
        _control_barrier(control, "post_train")

    eval_result: dict[str, Any] = {}
    if rank == 0 and (eval_batches > 0 or calc_types):
        if luts[0] is None:
            raise ValueError("evaluation reports bits per byte and needs the SentencePiece model: pass "
                             "--sp-model-path, or set eval_batches: 0 (and no calc_types) to train only")
        from .eval import dispatch_eval_for_config
        from .sp_eval import evaluate_bpb_sp
        val_cache = None
        if calc_types:
            if not val_cache_dir:
                raise ValueError("config sets calc_types but --val-cache-dir was not provided to the runner")
            from .eval_stream import load_val_cache
            val_cache = load_val_cache(Path(val_cache_dir))
        slow_backup = None
        if fast_slow is not None and fast_slow.should_copy_slow_to_model_for_eval():
            slow_backup = _state_dict_clone(model)
            fast_slow.copy_slow_to_model(model)

        def _do_eval():
            return dispatch_eval_for_config(
                config, model=model, val_cache=val_cache, val_tokens=val_tokens, eval_starts=eval_starts,
                batch_size=batch, seq_len=seq_len, device=device, base_bytes_lut=luts[0],
                has_leading_space_lut=luts[1], is_boundary_token_lut=luts[2], legacy_evaluate_fn=evaluate_bpb_sp)
        eval_result = eval_with_ema(model, getattr(optimizer, "_weight_ema", None), _do_eval)
        if slow_backup is not None:
            _restore_state_dict(model, slow_backup)
    if ddp:
        _control_barrier(control, "post_eval", timeout_s=float(config.get("eval_barrier_timeout_s", 3600.0)))

    result = {
        "config": config, "params": n_params, "train": train_result, "eval": eval_result,
        "artifact": {"artifact_impact": str(config.get("artifact_impact", "artifact_changes_weights_only")),
                     "submit_valid": bool(config.get("submit_valid", True)),
                     "artifact_bytes_estimate": int(model.artifact_bytes()),
                     "compressed_artifact_bytes": config.get("compressed_artifact_bytes")},
        "exp24": {"phase": config.get("exp24_phase"), "mechanism": config.get("exp24_mechanism")},
    }
    if ckpt_meta is not None:
        result["checkpoint"] = {"checkpoint_path": ckpt_meta["checkpoint_path"]}
    if rank == 0:
        bad = [f"train.{k} is not finite" for k in ("initial_loss", "final_loss")
               if not math.isfinite(float(train_result.get(k, float("nan"))))]
        bad += [f"eval.{k} is not finite" for k in ("bpb", "loss")
                if k in eval_result and not math.isfinite(float(eval_result[k]))]
        if bad:
            raise RuntimeError("; ".join(bad))
        if output_json:
            out = Path(output_json)
            out.parent.mkdir(parents=True, exist_ok=True)
            tmp = out.with_suffix(out.suffix + ".tmp")
            tmp.write_text(json.dumps(result, indent=2, default=str))
            tmp.rename(out)
        if output_ckpt:
            _save_output_ckpt(output_ckpt, model, config, episodic_cache=episodic_cache_blob)
        print(f"[rank 0/{world_size}] done steps={train_result['steps']} "
              f"tok/s={train_result.get('aggregate_tokens_per_sec', 0.0):.0f} "
              f"loss={train_result['final_loss']:.4f} vram={train_result.get('peak_vram_mb', 0.0):.1f}MB", flush=True)
    if ddp and dist.is_initialized():
        # collective teardown of the peer-memory communicator (drain, barrier, unmap the peers,
        # barrier, free): must precede the process group's destruction and happens on every rank
        from .parallel import symm_comm
        symm_comm.disable()
    if ddp and dist.is_initialized() and not keep_process_group:
        _CONTROL.clear()
        dist.destroy_process_group()
    return result


def main(argv: Optional[list[str]] = None) -> int:
    import yaml
    ap = argparse.ArgumentParser(description="throughput runner (train + eval)")
    ap.add_argument("--config", required=True)
    ap.add_argument("--data-path", required=True)
    ap.add_argument("--sp-model-path", default=None)
    ap.add_argument("--budget", type=float, default=None)
    ap.add_argument("--output-json", default=None)
    ap.add_argument("--output-ckpt", default=None)
    ap.add_argument("--world-size", type=int, default=None)
    ap.add_argument("--val-cache-dir", default=None,
                    help="ValCache directory (tokens.npy / docs.npy / manifest.json); required with calc_types")
    a = ap.parse_args(argv)
    config = yaml.safe_load(Path(a.config).read_text())
    run_condition(config, data_path=a.data_path, sp_model_path=a.sp_model_path,
                  budget_seconds=float(a.budget) if a.budget is not None else float(config.get("budget_seconds", 90.0)),
                  output_json=a.output_json, output_ckpt=a.output_ckpt, world_size_override=a.world_size,
                  val_cache_dir=a.val_cache_dir)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
