"""Lean training entry points: ``train_ssm_step`` and ``train_ssm_for_budget``
plus the LM-head backward helpers, with the reference's signatures and result
contract (src/chaoscontrol/train_ssm.py:50-774).

Execution paths of ``train_ssm_step``:

* **engine** -- bare-SSM model whose parameters live in a ``ParamArena`` on a
  CUDA device, bf16, with a fused LM-head mode: the whole step (forward,
  fused LM head with recompute, backward) is the hand-scheduled kernel
  sequence of :class:`chaoscontrol_b200.engine.TrainEngine`; gradients land in
  the arena's flat fp32 buffer and are also exposed as ``p.grad``.
* **autograd** -- everything else (CPU, fp32, hooks, ``chunked`` / ``single``
  head modes): ``model.encode`` under autocast, then the requested LM-head
  backward.

In both cases gradients are averaged across ranks before returning when DDP is
active, and the caller owns ``zero_grad`` / ``optimizer.step``.
"""
from __future__ import annotations

import random
import time
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .data import batch_from_starts
from .engine import TrainEngine
from .kernels.lm_head_loss import (fused_linear_cross_entropy, fused_linear_cross_entropy_with_ce,
                                   fused_rms_linear_cross_entropy, fused_rms_norm)
from .parallel.distributed import (allreduce_grads, broadcast_params, clip_arena_grad_norm,
                                   clip_grad_norm_fused, resolve_ddp_context, should_stop_now)
from .precision import autocast_context
from .utils.arena import get_arena

_FUSED_LM_HEAD_BACKENDS: dict[str, str] = {
    "fused": "auto",
    "fused_streaming": "streaming",
    "fused_streaming_v2": "streaming_v2",
    "fused_streaming_cached": "streaming_cached",
    "fused_norm_streaming_v2": "norm_streaming_v2",
}

_UNSUPPORTED_ATTRS = (
    ("wernicke", "wernicke layer"),
    ("outer_model", "outer_model / typed buffer"),
    ("semantic_tier", "semantic_tier bias"),
    ("posterior", "posterior correction module"),
    ("bucket_prototypes_module", "bucket_prototypes"),
)


def fused_lm_head_backend_for_mode(lm_head_backward_mode: str) -> str:
    try:
        return _FUSED_LM_HEAD_BACKENDS[str(lm_head_backward_mode).strip().lower()]
    except KeyError as exc:
        raise ValueError(
            "lm_head_backward_mode must be 'fused', 'fused_streaming', 'fused_streaming_v2', "
            f"'fused_streaming_cached', or 'fused_norm_streaming_v2', got {lm_head_backward_mode!r}"
        ) from exc


def _reject_unsupported(model: nn.Module, *, crct_enabled: bool = False) -> None:
    """With ``crct_enabled`` the episodic store and the bucket prototypes may be
    present: train ranks only ever run ``encode(memory_mode="packet")``, which
    reads neither (runner_fast_path.py:1223-1244)."""
    for attr, label in _UNSUPPORTED_ATTRS:
        if crct_enabled and attr in ("outer_model", "bucket_prototypes_module"):
            continue
        if getattr(model, attr, None) is not None:
            raise ValueError(f"train_ssm does not support the {label} path (model.{attr} is not "
                             "None). Use chaoscontrol_b200.training.train_chaoscontrol_for_budget "
                             "for configs that enable this feature.")


# ---------------------------------------------------------------------------
# LM-head backward helpers
# ---------------------------------------------------------------------------
def chunked_lm_head_backward(hidden: torch.Tensor, final_norm: nn.Module, lm_head: nn.Linear,
                             targets: torch.Tensor, chunk_size: int) -> torch.Tensor:
    """final_norm -> lm_head -> CE -> backward in time chunks; the full
    ``(B, T, V)`` logits tensor never exists.  ``hidden`` must be a detached leaf
    with ``requires_grad=True``; its ``.grad`` and the head / norm weight grads
    are populated.  Each chunk's loss is ``CE(sum) / (B*T)`` so the accumulated
    gradient is that of one mean-reduced loss.  Returns the detached loss."""
    if chunk_size <= 0:
        raise ValueError(f"chunked_lm_head_backward: chunk_size must be positive, got {chunk_size}. "
                         "A non-positive value would wedge the time-chunk loop indefinitely "
                         "rather than failing cleanly.")
    if not hidden.requires_grad:
        raise ValueError("chunked_lm_head_backward: ``hidden`` must have requires_grad=True so "
                         "per-chunk backward can accumulate into hidden.grad. Call "
                         "hidden.detach().requires_grad_(True) before passing it here.")
    batch, seq, _ = hidden.shape
    vocab = lm_head.out_features
    total = batch * seq
    loss_accum = hidden.new_zeros((), dtype=torch.float32)
    start = 0
    while start < seq:
        end = min(start + chunk_size, seq)
        logits = lm_head(final_norm(hidden[:, start:end, :]))
        chunk_loss = F.cross_entropy(logits.reshape(-1, vocab).float(),
                                     targets[:, start:end].reshape(-1), reduction="sum") / total
        chunk_loss.backward()
        loss_accum = loss_accum + chunk_loss.detach()
        start = end
    return loss_accum


def full_lm_head_backward(hidden, final_norm, lm_head, targets, *, loss_weight: float = 1.0):
    """Materialise full logits, one ``backward()``."""
    logits = lm_head(final_norm(hidden))
    loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1))
    (loss * float(loss_weight)).backward()
    return loss.detach()


def fused_lm_head_loss_with_ce(*, hidden, final_norm, lm_head, targets, backend: str = "auto",
                               tile_size: int = 1024):
    """``(mean loss, per-token CE)`` through the fused head; differentiable."""
    weight = getattr(final_norm, "weight", None)
    eps = float(getattr(final_norm, "eps", 1e-6))
    normed = fused_rms_norm(hidden, weight, eps=eps) if weight is not None else final_norm(hidden)
    b = "streaming_v2" if str(backend).strip().lower() == "norm_streaming_v2" else backend
    loss, ce = fused_linear_cross_entropy_with_ce(normed, lm_head.weight, targets, reduction="mean",
                                                  backend=b, tile_size=int(tile_size))
    return loss, ce.view(targets.shape)


def fused_lm_head_weighted_loss_with_ce(*, hidden, final_norm, lm_head, targets, token_weight,
                                        backend: str = "auto", tile_size: int = 1024):
    """``(sum(ce * w) / max(sum w, 1), detached per-token CE)``, differentiable in ``hidden`` and the
    head / norm weights; ``token_weight`` is treated as a constant (train_ssm.py:210-270)."""
    from .kernels.lm_head_loss import fused_linear_cross_entropy_weighted
    if token_weight.device != hidden.device:
        raise ValueError("fused_lm_head_weighted_loss_with_ce: token_weight must be on the same device as hidden, "
                         f"got {token_weight.device} and {hidden.device}")
    weight = getattr(final_norm, "weight", None)
    eps = float(getattr(final_norm, "eps", 1e-6))
    w = token_weight.reshape(-1).detach().float()
    if weight is None:
        logits = lm_head(final_norm(hidden))
        ce = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1), reduction="none")
        return (ce * w).sum() / w.sum().clamp_min(1.0), ce.detach()
    b = "streaming_v2" if str(backend).strip().lower() == "norm_streaming_v2" else backend
    loss, ce = fused_linear_cross_entropy_weighted(fused_rms_norm(hidden, weight, eps=eps), lm_head.weight,
                                                   targets.reshape(-1), w, backend=b, tile_size=int(tile_size))
    return loss, ce.detach()


def fused_lm_head_backward(hidden, final_norm, lm_head, targets, *, backend: str = "auto",
                           tile_size: int = 1024, loss_weight: float = 1.0) -> torch.Tensor:
    """Fused RMSNorm + tiled linear+CE, one backward.  Returns the detached loss."""
    weight = getattr(final_norm, "weight", None)
    eps = float(getattr(final_norm, "eps", 1e-6))
    if weight is None:
        return full_lm_head_backward(hidden, final_norm, lm_head, targets, loss_weight=loss_weight)
    if str(backend).strip().lower() == "norm_streaming_v2":
        loss = fused_rms_linear_cross_entropy(hidden, weight, lm_head.weight, targets, eps=eps,
                                              reduction="mean", backend="streaming_v2",
                                              tile_size=int(tile_size))
    else:
        loss = fused_linear_cross_entropy(fused_rms_norm(hidden, weight, eps=eps), lm_head.weight,
                                          targets, reduction="mean", backend=backend,
                                          tile_size=int(tile_size))
    (loss * float(loss_weight)).backward()
    return loss.detach()


def fused_lm_head_backward_with_ce(hidden, final_norm, lm_head, targets, *, backend: str = "auto",
                                   tile_size: int = 1024, loss_weight: float = 1.0):
    loss, ce = fused_lm_head_loss_with_ce(hidden=hidden, final_norm=final_norm, lm_head=lm_head,
                                          targets=targets, backend=backend, tile_size=tile_size)
    (loss * float(loss_weight)).backward()
    return loss.detach(), ce.detach()


# ---------------------------------------------------------------------------
# one step
# ---------------------------------------------------------------------------
def _engine_for(model: nn.Module) -> Optional[TrainEngine]:
    eng = getattr(model, "_ccb_engine", None)
    if eng is not None and eng.arena.still_valid():
        return eng
    arena = get_arena(model)
    if arena is None or not TrainEngine.supported(model):
        return None
    eng = TrainEngine(model, arena)
    model._ccb_engine = eng          # type: ignore[attr-defined]
    return eng


def train_ssm_step(model: nn.Module, inputs: torch.Tensor, targets: torch.Tensor, chunk_size: int, *,
                   ddp_active: bool = False, world_size: int = 1, precision: str = "bf16",
                   compile_full_path: bool = False, lm_head_backward_mode: str = "chunked",
                   lm_head_tile_size: int = 1024, grad_allreduce_mode: str = "bulk",
                   async_grad_reducer=None) -> torch.Tensor:
    """One forward + backward.  Gradients are left on the parameters (averaged
    across ranks when ``ddp_active``); returns the detached mean CE.

    ``grad_allreduce_mode``: ``"bulk"`` reduces once after backward; ``"async_param"`` overlaps the
    exchange with backward (train_ssm.py:1186-1260 of the reference).  On the autograd path that is
    an :class:`~chaoscontrol_b200.parallel.distributed.AsyncGradAllReducer` whose per-parameter hooks
    launched the all-reduces during backward (pass it as ``async_grad_reducer``; this function waits
    for it); on the kernel engine it is the bucketed peer-memory exchange on a side stream.

    ``compile_full_path`` is accepted for signature compatibility and ignored:
    there is no tracing compiler in this stack, the encoder is already one
    hand-scheduled kernel sequence on the GPU.
    """
    _reject_unsupported(model)
    mode = str(lm_head_backward_mode).strip().lower()
    fused_mode = mode in _FUSED_LM_HEAD_BACKENDS
    if mode not in ("single", "chunked") and not fused_mode:
        raise ValueError("lm_head_backward_mode must be 'chunked', 'single', 'fused', "
                         "'fused_streaming', 'fused_streaming_v2', or 'fused_streaming_cached', or "
                         f"'fused_norm_streaming_v2', got {lm_head_backward_mode!r}")

    ar_mode = str(grad_allreduce_mode).strip().lower()
    if ar_mode not in ("bulk", "async_param"):
        raise ValueError(f"grad_allreduce_mode must be 'bulk' or 'async_param', got {grad_allreduce_mode!r}")
    if ar_mode == "async_param" and mode == "chunked":
        # the chunked head runs one backward per chunk, so the head's gradients accumulate over several
        # passes and a per-parameter hook would reduce partial sums
        raise ValueError("grad_allreduce_mode='async_param' needs a single backward pass: use "
                         "lm_head_backward_mode 'single' or one of the fused modes, not 'chunked'")
    engine = _engine_for(model) if (fused_mode and precision in ("bf16", "fp8_fused") and
                                    model.training) else None
    if engine is not None:
        reducer = None
        if ddp_active and world_size > 1:
            from .parallel.grad_overlap import reducer_for
            reducer = reducer_for(engine, world_size, force=ar_mode == "async_param")
        loss = engine.step(inputs, targets, reducer=reducer)
        if ddp_active and world_size > 1:
            allreduce_grads(model, world_size)       # no-op when the reducer already did the exchange
        engine.arena.materialize_grads()
        return loss

    with autocast_context(precision, device_type=inputs.device.type):
        hidden = model.encode(inputs)
        if mode == "single":
            loss = full_lm_head_backward(hidden, model.final_norm, model.lm_head, targets)
        elif fused_mode:
            loss = fused_lm_head_backward(hidden, model.final_norm, model.lm_head, targets,
                                          backend=fused_lm_head_backend_for_mode(mode),
                                          tile_size=int(lm_head_tile_size))
        else:
            hidden_for_ce = hidden.detach().requires_grad_(True)
            loss = chunked_lm_head_backward(hidden_for_ce, model.final_norm, model.lm_head, targets,
                                            chunk_size)
            hidden.backward(gradient=hidden_for_ce.grad)
    if ddp_active and world_size > 1:
        if ar_mode == "async_param":
            if async_grad_reducer is None:
                raise ValueError("grad_allreduce_mode='async_param' requires an AsyncGradAllReducer instance")
            async_grad_reducer.wait()
        else:
            allreduce_grads(model, world_size)
    return loss


class GraphedTrainStep:
    """A fixed-shape training step -- forward, backward, the data-parallel gradient exchange and the
    gradient clip -- captured once in a CUDA graph and replayed per batch.

    ``step(inputs, targets)`` copies the batch into two static device buffers (the copy may come
    straight from pinned host memory), replays the graph and returns the loss as a device scalar
    that the next replay overwrites.  The first ``eager_steps`` calls run :func:`train_ssm_step`
    eagerly (they are real training steps and also finish every lazy set-up a capture must not
    contain), the next call captures.  The optimizer step stays outside: its AdamW bias corrections
    are host scalars that change every step.

    Data-parallel steps can be captured because the peer-memory collectives keep their epoch in
    device memory (no launch argument changes between steps); with the library fallback
    (NCCL / gloo) the step is not capturable here and ``step`` stays eager.

    The reference rejected whole-step graphs at this model size (2.34 M vs 2.55 M tokens/s eager,
    experiments/23_fast_path/RESULTS_GRAPH_PROBE.md:15-16); here the step is about 220 launches of
    10-700 us, and the graph removes the gaps between them.
    """

    def __init__(self, model: nn.Module, *, chunk_size: int = 64, ddp_active: bool = False, world_size: int = 1,
                 precision: str = "bf16", lm_head_backward_mode: str = "fused_streaming_cached",
                 lm_head_tile_size: int = 8192, grad_clip_norm: float = 0.0, eager_steps: int = 2) -> None:
        self.model = model
        self.kw = dict(ddp_active=ddp_active, world_size=world_size, precision=precision,
                       lm_head_backward_mode=lm_head_backward_mode, lm_head_tile_size=lm_head_tile_size)
        self.chunk_size = int(chunk_size)
        self.grad_clip_norm = float(grad_clip_norm)
        self.eager_left = max(1, int(eager_steps))
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._in: Optional[torch.Tensor] = None
        self._tg: Optional[torch.Tensor] = None
        self._loss: Optional[torch.Tensor] = None
        self.capturable = True
        self.replays = 0
        self.launches_per_replay = 0

    def _eager(self, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        loss = train_ssm_step(self.model, inputs, targets, self.chunk_size, **self.kw)
        if self.grad_clip_norm > 0.0:
            arena = get_arena(self.model)
            if arena is not None and arena.grads_fresh:
                clip_arena_grad_norm(arena, self.grad_clip_norm)
            else:
                clip_grad_norm_fused(self.model.parameters(), self.grad_clip_norm)
        return loss

    def _can_capture(self) -> bool:
        if not (torch.cuda.is_available() and next(self.model.parameters()).is_cuda):
            return False
        if _engine_for(self.model) is None:
            return False
        if self.kw["ddp_active"] and self.kw["world_size"] > 1:
            from .parallel import symm
            comm = symm.active_comm(None)
            return comm is not None and comm.ws == self.kw["world_size"]
        return True

    def step(self, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        if self.graph is None:
            if self.eager_left > 0 or not self.capturable:
                self.eager_left -= 1
                return self._eager(inputs.to(next(self.model.parameters()).device, non_blocking=True),
                                   targets.to(next(self.model.parameters()).device, non_blocking=True))
            if not self._can_capture():
                self.capturable = False
                return self.step(inputs, targets)
            dev = next(self.model.parameters()).device
            self._in = torch.empty(inputs.shape, dtype=inputs.dtype, device=dev)
            self._tg = torch.empty(targets.shape, dtype=targets.dtype, device=dev)
            self._in.copy_(inputs, non_blocking=True)
            self._tg.copy_(targets, non_blocking=True)
            torch.cuda.synchronize(dev)
            g = torch.cuda.CUDAGraph()
            from .ops import _lib
            n0 = _lib.launch_count()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self._loss = self._eager(self._in, self._tg)
            self.launches_per_replay = _lib.launch_count() - n0     # this library's kernels inside the graph
            self.graph = g
        else:
            if inputs.shape != self._in.shape or targets.shape != self._tg.shape:
                raise ValueError(f"GraphedTrainStep was captured for batches of {tuple(self._in.shape)}; got "
                                 f"{tuple(inputs.shape)}")
            self._in.copy_(inputs, non_blocking=True)
            self._tg.copy_(targets, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        arena = get_arena(self.model)
        if arena is not None:
            arena.grads_fresh = True          # host flags a replay does not set
            arena.grads_reduced = False
        return self._loss

    __call__ = step


def train_ssm_step_with_ce(model: nn.Module, inputs: torch.Tensor, targets: torch.Tensor, *,
                           precision: str = "bf16", lm_head_backward_mode: str = "fused",
                           lm_head_tile_size: int = 1024) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Forward + backward that also hands back what an event producer needs:
    ``(loss, per-token CE [B, T], trunk output [B, T, D])``.  No gradient
    reduction happens here.  The kernel engine already keeps both by-products
    of its fused head; the autograd path uses the CE-returning fused head."""
    _reject_unsupported(model)
    B, Tn = inputs.shape
    mode = str(lm_head_backward_mode).strip().lower()
    fused_mode = mode in _FUSED_LM_HEAD_BACKENDS
    engine = _engine_for(model) if (fused_mode and precision in ("bf16", "fp8_fused") and model.training) else None
    if engine is not None:
        loss = engine.step(inputs, targets)
        engine.arena.materialize_grads()
        return loss, engine.last_loss_rows.reshape(B, Tn), engine.last_hidden.reshape(B, Tn, -1)
    with autocast_context(precision, device_type=inputs.device.type):
        hidden = model.encode(inputs)
        if fused_mode:
            loss, ce = fused_lm_head_backward_with_ce(hidden, model.final_norm, model.lm_head, targets,
                                                      backend=fused_lm_head_backend_for_mode(mode),
                                                      tile_size=int(lm_head_tile_size))
        else:
            logits = model.lm_head(model.final_norm(hidden))
            ce = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1),
                                 reduction="none").reshape(B, Tn)
            loss = ce.mean()
            loss.backward()
            loss, ce = loss.detach(), ce.detach()
    return loss, ce.reshape(B, Tn), hidden.detach()


# ---------------------------------------------------------------------------
# budgeted loop
# ---------------------------------------------------------------------------
def train_ssm_for_budget(model: nn.Module, *, train_tokens: torch.Tensor, train_starts: list[int],
                         seq_len: int, batch_size: int, device: torch.device,
                         optimizer: torch.optim.Optimizer, budget_seconds: float, chunk_size: int,
                         grad_clip_norm: float = 0.0, fused_grad_clip: bool = False,
                         rank: Optional[int] = None, world_size: Optional[int] = None, seed: int = 0,
                         time_fn: Callable[[], float] = time.perf_counter, precision: str = "bf16",
                         compile_full_path: bool = False, max_steps: Optional[int] = None,
                         lm_head_backward_mode: str = "chunked",
                         lm_head_tile_size: int = 1024) -> dict[str, Any]:
    """Wall-clock-budgeted training loop.  Returns ``{"history", "steps",
    "elapsed_s", "rank", "world_size", "peak_vram_mb"}``; losses stay on the
    device until the loop ends (one transfer)."""
    _reject_unsupported(model)
    rank_, world_size_ = resolve_ddp_context(rank, world_size)
    ddp_active = world_size_ > 1
    if ddp_active:
        broadcast_params(model)
    rng = random.Random(seed + rank_)
    model.train()
    loss_tensors: list[torch.Tensor] = []
    steps = 0
    start_time = time_fn()
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)

    while True:
        elapsed = time_fn() - start_time
        local_stop = (elapsed >= budget_seconds and steps > 0) or (
            max_steps is not None and steps >= max_steps)
        if should_stop_now(local_stop, device, ddp_active):
            break
        starts = [train_starts[rng.randrange(len(train_starts))] for _ in range(batch_size)]
        inputs, targets = batch_from_starts(train_tokens, starts, seq_len, device)
        optimizer.zero_grad(set_to_none=True)
        loss = train_ssm_step(model=model, inputs=inputs, targets=targets, chunk_size=chunk_size,
                              ddp_active=ddp_active, world_size=world_size_, precision=precision,
                              compile_full_path=compile_full_path,
                              lm_head_backward_mode=lm_head_backward_mode,
                              lm_head_tile_size=int(lm_head_tile_size))
        if grad_clip_norm > 0.0:
            arena = get_arena(model)
            if arena is not None and arena.grads_fresh:
                clip_arena_grad_norm(arena, grad_clip_norm)
                arena.materialize_grads()
            elif fused_grad_clip:
                clip_grad_norm_fused(model.parameters(), grad_clip_norm)
            else:
                torch.nn.utils.clip_grad_norm_(model.parameters(), grad_clip_norm)
        optimizer.step()
        if precision == "fp8_fused":
            from .ops.fp8_linear import fused_fp8_flush_all
            fused_fp8_flush_all(model)
        loss_tensors.append(loss.detach())
        steps += 1

    if ddp_active:
        dist.barrier()
    if loss_tensors:
        stacked = torch.stack([t.float() for t in loss_tensors]).cpu()
        history = [{"step": float(i), "loss": float(stacked[i])} for i in range(len(loss_tensors))]
    else:
        history = []
    peak = torch.cuda.max_memory_allocated(device) / (1024 * 1024) if device.type == "cuda" else 0.0
    return {"history": history, "steps": steps, "elapsed_s": time_fn() - start_time, "rank": rank_,
            "world_size": world_size_, "peak_vram_mb": peak}
