"""Dream replay for training: a bounded, age-limited buffer of (recurrent state,
token window) seeds, teacher-forced replay backward passes from them, and replay
from curated episodic-cache spans (behaviour of
experiments/23_fast_path/dreamworld.py:37-463).

Differences that matter on a GPU: the buffer is a deque (O(1) eviction), the
replay-gradient norm is one fused reduction with a single host read (over the
flat gradient arena when the model has one), and
``dreamworld_replay_from_cache_slots`` replays any number of tagged cache slots
as ONE batched forward / backward instead of one tiny pass per slot.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass
from typing import Any, Optional, Sequence

import torch

from .train_ssm import full_lm_head_backward, fused_lm_head_backend_for_mode, fused_lm_head_backward
from .utils.arena import get_arena

__all__ = ["LossTriggeredReplayDecision", "LossTriggeredReplayEMA", "DreamReplayEntry", "DreamReplayBuffer",
           "build_dream_replay_tokens", "capture_dream_entry",
           "dreamworld_replay_backward", "compute_utility_signal", "dreamworld_replay_from_cache_entry",
           "dreamworld_replay_from_cache_slots", "replay_grad_norm"]


@dataclass
class DreamReplayEntry:
    step: int
    states: list
    replay_tokens: torch.Tensor


class DreamReplayBuffer:
    """FIFO of replay seeds: at most ``max_entries``, none older than ``max_age_steps``."""

    def __init__(self, max_entries: int, max_age_steps: int) -> None:
        if max_entries <= 0:
            raise ValueError("max_entries must be greater than 0")
        if max_age_steps <= 0:
            raise ValueError("max_age_steps must be greater than 0")
        self.max_entries, self.max_age_steps = int(max_entries), int(max_age_steps)
        self._entries: deque = deque()
        self.add_count = self.sample_count = self.drop_count = 0

    def __len__(self) -> int:
        return len(self._entries)

    def _enforce(self, current_step: int) -> None:
        before = len(self._entries)
        if any(current_step - e.step > self.max_age_steps for e in self._entries):
            self._entries = deque(e for e in self._entries if current_step - e.step <= self.max_age_steps)
        while len(self._entries) > self.max_entries:
            self._entries.popleft()
        self.drop_count += before - len(self._entries)

    def add(self, *, step: int, states: list, replay_tokens: torch.Tensor) -> None:
        """Stores detached copies, then applies the age and capacity bounds."""
        self._entries.append(DreamReplayEntry(int(step), [s.detach().clone() for s in states],
                                              replay_tokens.detach().clone()))
        self.add_count += 1
        self._enforce(int(step))

    def sample(self, generator: torch.Generator, current_step: int) -> Optional[DreamReplayEntry]:
        self._enforce(current_step)
        self.sample_count += 1
        if not self._entries:
            return None
        return self._entries[int(torch.randint(0, len(self._entries), (1,), generator=generator))]

    def diagnostics(self, current_step: int) -> dict[str, Any]:
        self._enforce(current_step)
        ages = [current_step - e.step for e in self._entries]
        return {"size": len(ages), "max_entries": self.max_entries, "max_age_steps": self.max_age_steps,
                "add_count": self.add_count, "sample_count": self.sample_count, "drop_count": self.drop_count,
                "age_min": int(min(ages)) if ages else 0, "age_max": int(max(ages)) if ages else 0,
                "age_mean": float(sum(ages) / len(ages)) if ages else 0.0}


def build_dream_replay_tokens(inputs: torch.Tensor, prefix_tokens: int, replay_tokens: int) -> torch.Tensor:
    """``inputs[:, prefix - 1 : prefix + replay]``: the seed token plus ``replay_tokens`` targets."""
    if prefix_tokens <= 0:
        raise ValueError(f"prefix_tokens must be > 0, got {prefix_tokens}")
    if replay_tokens <= 0:
        raise ValueError(f"replay_tokens must be > 0, got {replay_tokens}")
    if inputs.dim() != 2:
        raise ValueError(f"inputs must be 2D (batch, seq), got shape {tuple(inputs.shape)}")
    start, end = prefix_tokens - 1, prefix_tokens + replay_tokens
    if end > inputs.shape[1]:
        raise ValueError(f"replay span [{start}, {end}) does not fit into seq length {inputs.shape[1]}")
    return inputs[:, start:end].detach()


def capture_dream_entry(model: Any, inputs: torch.Tensor, *, step: int, prefix_tokens: int,
                        replay_tokens: int) -> DreamReplayEntry:
    """Recurrent state after ``prefix_tokens - 1`` tokens and the window that follows it."""
    if prefix_tokens < 2:
        raise ValueError(f"prefix_tokens must be at least 2, got {prefix_tokens}")
    with torch.no_grad():
        _, states = model.encode(inputs[:, : prefix_tokens - 1], return_final_states=True)
    return DreamReplayEntry(step, states, build_dream_replay_tokens(inputs, prefix_tokens, replay_tokens))


def _head_backward(model, hidden, targets, weight, mode, tile):
    if str(mode).strip().lower() == "single":
        return full_lm_head_backward(hidden, model.final_norm, model.lm_head, targets, loss_weight=float(weight))
    return fused_lm_head_backward(hidden, model.final_norm, model.lm_head, targets,
                                  backend=fused_lm_head_backend_for_mode(str(mode).strip().lower()),
                                  tile_size=int(tile), loss_weight=float(weight))


def dreamworld_replay_backward(model: Any, entry: DreamReplayEntry, weight: float, *,
                               lm_head_backward_mode: str = "single", lm_head_tile_size: int = 1024,
                               replay_batch_size: int = 0, generator: Optional[torch.Generator] = None
                               ) -> torch.Tensor:
    """Teacher-forced pass over the entry's window from its stored state; gradients (scaled by
    ``weight``) accumulate into the parameters; returns the un-weighted loss.  A positive
    ``replay_batch_size`` replays a random subset of the entry's rows."""
    dev = next(model.parameters()).device
    tokens, states = entry.replay_tokens, entry.states
    rows = tokens.shape[0]
    if 0 < int(replay_batch_size) < rows:
        pick = torch.randperm(rows, generator=generator)[: int(replay_batch_size)]
        tokens = tokens.index_select(0, pick.to(tokens.device))
        states = [s.index_select(0, pick.to(s.device)) for s in states]
    tokens = tokens.to(dev)
    hidden = model.encode(tokens[:, :-1].to(torch.int32), initial_states=[s.to(dev) for s in states],
                          return_final_states=False)
    return _head_backward(model, hidden, tokens[:, 1:].long(), weight, lm_head_backward_mode, lm_head_tile_size)


def replay_grad_norm(model: Any) -> float:
    """L2 norm of all parameter gradients at this moment.  Replay passes ADD into the gradients, so
    the value after the k-th replay of a step is the norm of the sum of the first k replay gradients."""
    arena = get_arena(model)
    if arena is not None and getattr(arena, "grads_fresh", False):
        return float(arena.flat_grad.norm())
    grads = [p.grad.detach() for p in model.parameters() if p.grad is not None]
    if not grads:
        return 0.0
    return float(torch.linalg.vector_norm(torch.stack(torch._foreach_norm(grads))))


_replay_grad_norm_flat = replay_grad_norm


def compute_utility_signal(replay_grad_cos_rare: float) -> tuple[float, float]:
    """``(raw, transformed)``: the cosine as given (NaN preserved) and what the cache's utility average
    consumes, ``max(0, raw)`` with NaN mapped to 0 (a negative utility would invert the retrieval order)."""
    raw = float(replay_grad_cos_rare)
    return raw, (0.0 if math.isnan(raw) else max(0.0, raw))


def dreamworld_replay_from_cache_slots(*, model: Any, cache: Any, slots: Sequence[int], weight: float = 1.0,
                                       lm_head_backward_mode: str = "single", lm_head_tile_size: int = 1024
                                       ) -> Optional[dict[str, Any]]:
    """Replays the value spans of all occupied ``slots`` as one batch (one row per slot, mean CE over all
    targets).  Returns ``None`` when no slot is replayable, else the loss, the replayed slots and the
    cumulative gradient norm."""
    span = int(cache.span_length)
    for s in slots:
        if not 0 <= int(s) < int(cache.capacity):
            raise IndexError(f"slot {s} out of range for cache capacity {cache.capacity}")
    idx = torch.as_tensor([int(s) for s in slots], dtype=torch.long)
    if idx.numel() == 0 or span < 2:
        return None
    idx = idx[cache.occupied[idx].cpu()]
    if idx.numel() == 0:
        return None
    dev = next(model.parameters()).device
    rows = cache.value_tok_ids[idx].detach().to(dev)
    if rows.shape != (idx.numel(), span):
        raise ValueError(f"cache value_tok_ids rows have shape {tuple(rows.shape)}; expected (*, {span})")
    hidden = model.encode(rows[:, :-1].to(torch.int32))
    loss = _head_backward(model, hidden, rows[:, 1:].long(), weight, lm_head_backward_mode, lm_head_tile_size)
    return {"replay_loss": float(loss.detach()), "slots": idx.tolist(), "replay_grad_norm": replay_grad_norm(model)}


def dreamworld_replay_from_cache_entry(*, model: Any, cache: Any, slot: int, current_step: int, weight: float = 1.0,
                                       lm_head_backward_mode: str = "single", lm_head_tile_size: int = 1024
                                       ) -> Optional[dict[str, Any]]:
    """One cache slot's span as a single-row replay.  ``None`` for an unoccupied slot or a span shorter
    than 2.  The returned dict has every replay-log column this pass can fill; the three gradient
    cosines are NaN because no live rare-gradient direction exists on the replaying rank, so the
    transformed utility signal is 0."""
    out = dreamworld_replay_from_cache_slots(model=model, cache=cache, slots=[int(slot)], weight=weight,
                                             lm_head_backward_mode=lm_head_backward_mode,
                                             lm_head_tile_size=lm_head_tile_size)
    if out is None:
        return None
    raw, transformed = compute_utility_signal(float("nan"))
    return {"replay_loss": out["replay_loss"], "replay_grad_norm": out["replay_grad_norm"],
            "replay_grad_cos_common": float("nan"), "replay_grad_cos_rare": raw,
            "replay_grad_cos_total": float("nan"), "utility_signal_raw": raw,
            "utility_signal_transformed": transformed}


# ---------------------------------------------------------------------------
# loss-pressure gate for event-triggered replay
# ---------------------------------------------------------------------------
class LossTriggeredReplayDecision:
    """One gate evaluation.  The eight numbers stay on the device in one tensor
    and travel to pinned host memory with one asynchronous copy; reading a field
    waits for that copy only if it has not landed yet, so a loop that looks at
    the decision one step later never stalls (runner_fast_path.py:6035-6132)."""

    FIELDS = ("local_loss", "ema_loss", "local_ratio", "local_pressure", "global_pressure", "fire_count",
              "local_fire", "triggered")

    def __init__(self, packed: torch.Tensor) -> None:
        self._event = None
        if packed.is_cuda:
            self._host = torch.empty(packed.shape, dtype=packed.dtype, pin_memory=True)
            self._host.copy_(packed, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()
        else:
            self._host = packed.detach().clone()

    def ready(self) -> bool:
        return self._event is None or bool(self._event.query())

    def _get(self, i: int) -> float:
        if self._event is not None:
            self._event.synchronize()
            self._event = None
        return float(self._host[i])

    local_loss = property(lambda self: self._get(0))
    ema_loss = property(lambda self: self._get(1))
    local_ratio = property(lambda self: self._get(2))
    local_pressure = property(lambda self: self._get(3))
    global_pressure = property(lambda self: self._get(4))
    fire_count = property(lambda self: int(round(self._get(5))))
    local_fire = property(lambda self: self._get(6) > 0.5)
    triggered = property(lambda self: self._get(7) > 0.5)


class LossTriggeredReplayEMA:
    """Schedules NEXT-step replay from the just-finished loss: pressure is how far
    ``loss / ema`` exceeds ``threshold``; ranks average their pressure with one
    two-element all-reduce and all agree on ``triggered``
    (runner_fast_path.py:6135-6210).  Returns ``None`` during warm-up."""

    def __init__(self, *, decay: float = 0.99, warmup_steps: int = 32, eps: float = 1e-8) -> None:
        if not 0.0 <= float(decay) < 1.0:
            raise ValueError(f"decay must be in [0, 1), got {decay}")
        if int(warmup_steps) < 0:
            raise ValueError(f"warmup_steps must be >= 0, got {warmup_steps}")
        self.decay, self.warmup_steps, self.eps = float(decay), int(warmup_steps), float(eps)
        self.value: Optional[torch.Tensor] = None
        self.observations = 0

    def update(self, loss: torch.Tensor, *, threshold: float = 1.10, pressure_threshold: float = 0.05,
               ddp_active: bool = False, world_size: int = 1, group=None) -> Optional[LossTriggeredReplayDecision]:
        cur = loss.detach().float().reshape(())
        if self.value is None:
            self.value, self.observations = cur.clone(), 1
            return None
        before = self.value
        self.value = self.decay * before + (1.0 - self.decay) * cur
        self.observations += 1
        if self.observations <= self.warmup_steps:
            return None
        ratio = cur / before.clamp_min(self.eps)
        pressure = (ratio - float(threshold)).clamp_min(0.0)
        fire = (pressure > 0).float()
        both = torch.stack((pressure, fire))
        if ddp_active and int(world_size) > 1:
            import torch.distributed as dist
            dist.all_reduce(both, op=dist.ReduceOp.SUM, group=group)
            both = torch.stack((both[0] / float(world_size), both[1]))
        triggered = (both[0] > float(pressure_threshold)).float()
        return LossTriggeredReplayDecision(torch.stack((cur, before, ratio, pressure, both[0], both[1], fire,
                                                        triggered)))
