"""CRCT teacher runtime: which rank plays which role, the scoring payloads, the
two teacher transports, and the memory rank's service loop.

Parity map (experiments/23_fast_path/runner_fast_path.py of the reference):

* ``crct_rank_topology``                    rank roles of the "N-1 train + 1 memory" world (``:1879-1910``)
* ``score_payload_inline`` / ``packet_payload_inline``   exact and approximate payloads (``:1298-1477``)
* ``broadcast_params_coalesced``            flat parameter broadcast to the teacher rank (``:880-905``)
* ``collect_teacher_payload_sync``          gather ids -> score on the memory rank -> broadcast (``:5931-6032``)
* ``TeacherMailbox``                        same-node mailbox: request/result rings, payload slab and a
                                            double-buffered weight-snapshot region in POSIX shared memory
                                            (``:3191-3260``, ``:3656-3740``, ``:4339-5077``, ``:5120-5890``)
* ``memory_rank_should_stop`` / ``memory_rank_defer_stop``   wall-clock stop with a shutdown grace window
                                            (``:1796-1844``)
* ``CrctRuntime``                           what the training loop talks to

Design notes.  The mailbox never makes a train rank wait for the teacher: a
request is a device->host copy on a side stream whose ring record is pushed only
once its event has completed, a result is taken only if it is already in the
ring, and a missing or stale result is a fail-open step (plain loss, no
residual).  Shared-memory regions are page-locked on CUDA ranks so both copy
directions are DMA.  With a flat parameter arena a weight snapshot is one copy
of one buffer.
"""
from __future__ import annotations

import os
import time
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Any, Optional

import numpy as np
import torch
import torch.distributed as dist

from .cache_utility import (CrctGradientConflictMonitor, ScarcityAwareMemoryOptimizer, alpha_ramp,
                            rank3_score_batch_causal)
from .utils.arena import get_arena
from .wake_cache import TransactionalWakeCache

__all__ = ["crct_rank_topology", "crct_full_input_ids", "crct_valid_mask", "score_payload_inline",
           "packet_payload_inline", "broadcast_params_coalesced", "collect_teacher_payload_sync",
           "TeacherMailbox", "memory_rank_should_stop", "memory_rank_defer_stop", "CrctRuntime",
           "TEACHER_RESULT_SLICE_NAMES", "weighted_row_scale", "crct_train_step", "SlotCommitPeerLane"]

TEACHER_RESULT_SLICE_NAMES = ("target", "confidence", "loss_weight", "utility", "memory_residual", "memory_gate",
                              "plasticity_coverage", "plasticity_confidence", "plasticity_budget")
_REQ_EVENT, _RES_EVENT = 6, 7
_FLAG_SHUTDOWN = 1
_FLAG_GATE_ALIASES_TARGET = 2
_DTYPE_CODE = {torch.int32: 1, torch.float32: 2, torch.float16: 3, torch.bfloat16: 4}
_CODE_DTYPE = {v: k for k, v in _DTYPE_CODE.items()}


# ---------------------------------------------------------------------------
# roles
# ---------------------------------------------------------------------------
def crct_rank_topology(*, world_size: int, split_memory_ranks: bool = False) -> dict[str, Any]:
    """Last rank serves packets and runs maintenance; with ``split_memory_ranks``
    (and at least three ranks) the last two ranks take one role each."""
    world = int(world_size)
    if world < 1:
        raise ValueError(f"world_size must be positive, got {world_size!r}")
    split = bool(split_memory_ranks) and world >= 3
    packet, maint = world - (2 if split else 1), world - 1
    memory = sorted({packet, maint}) if world > 1 else []
    train = [r for r in range(world) if r not in memory]
    return {"split_memory_ranks": split, "packet_rank": packet, "maintenance_rank": maint, "memory_ranks": memory,
            "train_ranks": train, "grad_world_size": len(train),
            "memory_owner": "split_packet_and_maintenance" if split else "packet_and_maintenance_shared"}


def crct_full_input_ids(inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """The ``[B, T+1]`` continuation a next-token batch was cut from."""
    return torch.cat([inputs[:, :1].long(), targets.long()], dim=1)


def crct_valid_mask(input_ids: torch.Tensor) -> torch.Tensor:
    """Training batches are dense continuations: every position is valid."""
    return torch.ones_like(input_ids, dtype=torch.bool)


def weighted_row_scale(loss_weight: torch.Tensor) -> torch.Tensor:
    """Per-row factors ``w * R / max(sum w, 1)`` so that ``mean(ce * factor)``
    equals the weighted loss ``sum(ce * w) / max(sum w, 1)``."""
    w = loss_weight.reshape(-1).float()
    return w * (w.numel() / w.sum().clamp_min(1.0))


# ---------------------------------------------------------------------------
# payloads
# ---------------------------------------------------------------------------
def _stash_probe(model: Any, input_ids: torch.Tensor, valid: torch.Tensor, step: int) -> None:
    model._last_crct_probe_input_ids = input_ids.detach()
    model._last_crct_probe_valid_mask = valid.detach()
    model._last_crct_probe_step = int(step)


def score_payload_inline(*, model: Any, cache: TransactionalWakeCache,
                         scarcity_optimizer: Optional[ScarcityAwareMemoryOptimizer], inputs: torch.Tensor,
                         targets: torch.Tensor, step: int, total_steps: Optional[int], tau: float, strength: float,
                         w_max: float, alpha_max: float, memory_write_tokens: int,
                         gradient_conflict_monitor: Optional[CrctGradientConflictMonitor] = None,
                         update_model_memory_after: bool = False,
                         record_stage_seconds: Optional[dict[str, float]] = None) -> dict[str, Any]:
    """Exact off/force-on contrast of one batch -> per-token teacher labels
    (runner_fast_path.py:1298-1379).  The reweighting strength follows the
    alpha ramp; the scarcity optimizer takes one dual step on the realised read
    rate."""
    ids = crct_full_input_ids(inputs, targets)
    valid = crct_valid_mask(ids)
    _stash_probe(model, ids, valid, step)
    alpha = alpha_ramp(int(step), int(total_steps or 0), alpha_max=float(alpha_max))
    score = rank3_score_batch_causal(model=model, cache=cache, input_ids=ids, valid_mask=valid,
                                     scarcity_optimizer=scarcity_optimizer, tau=float(tau),
                                     strength=float(strength) * float(alpha), w_max=float(w_max),
                                     update_model_memory_after=bool(update_model_memory_after),
                                     memory_write_tokens=int(memory_write_tokens),
                                     gradient_conflict_monitor=gradient_conflict_monitor, step=int(step),
                                     record_stage_seconds=record_stage_seconds)
    cue = getattr(model, "_last_outer_cue", None)
    if cue is not None:
        model._last_crct_probe_outer_cue = cue.detach()
    if scarcity_optimizer is not None:
        tgt, m = score["controller_target"], valid[:, 1:].to(score["controller_target"].device)
        scarcity_optimizer.dual_step(actual_read_rate=float(tgt[m].mean()) if bool(m.any()) else 0.0)
    out: dict[str, Any] = {"step_id_int": int(step), "target": score["controller_target"].detach().clone(),
                           "confidence": score["confidence"].detach().clone(),
                           "loss_weight": score["loss_weight"].detach().clone(),
                           "utility": score["utility"].detach().clone()}
    for k in ("plasticity_coverage", "plasticity_confidence", "plasticity_budget", "loss_reweight_diagnostics"):
        v = score.get(k)
        if isinstance(v, torch.Tensor):
            out[k] = v.detach().clone()
    if "memory_residual" in score and "memory_gate" in score:
        out["memory_residual"] = score["memory_residual"].detach().clone()
        out["memory_gate"] = score["memory_gate"].detach().clone()
        out["memory_gate_alias_target"] = True           # the gate is the controller target: ship it once
    if isinstance(score.get("memory_write_records"), list):
        out["memory_write_records"] = score["memory_write_records"]
    return out


@torch.inference_mode()
def packet_payload_inline(*, model: Any, cache: TransactionalWakeCache, inputs: torch.Tensor, targets: torch.Tensor,
                          step: int, memory_write_tokens: int) -> dict[str, Any]:
    """Low-latency packet: the current episodic residual with neutral labels, no
    off/force-on contrast (runner_fast_path.py:1382-1477).  Bootstraps the
    store by appending up to ``memory_write_tokens`` source tokens."""
    ids = crct_full_input_ids(inputs, targets)
    valid = crct_valid_mask(ids)
    _stash_probe(model, ids, valid, step)
    build = getattr(model, "build_episodic_packet", None)
    if not callable(build):
        raise ValueError("approximate CRCT packet serving requires model.build_episodic_packet(...)")
    txn = cache.begin_batch()
    mask = valid[:, 1:].to(device=inputs.device, dtype=torch.float32)
    packet = build(ids[:, :-1].to(torch.int32), cache_read_cutoff=txn.read_cutoff)
    cue = getattr(model, "_last_outer_cue", None)
    if cue is not None:
        model._last_crct_probe_outer_cue = cue.detach()
    residual, gate = packet.get("memory_residual"), packet.get("memory_gate")
    if not isinstance(residual, torch.Tensor) or not isinstance(gate, torch.Tensor):
        raise TypeError("build_episodic_packet must return memory_residual and memory_gate tensors")
    gate = gate.to(device=inputs.device, dtype=torch.float32) * mask
    records = None
    if int(memory_write_tokens) > 0:
        append = getattr(model, "append_memory_from_hidden", None)
        src = packet.get("packet_source_hidden")
        if append is None or not isinstance(src, torch.Tensor):
            raise ValueError("approximate CRCT packet serving requires packet_source_hidden and "
                             "model.append_memory_from_hidden(...) for cache bootstrap")
        ws = packet.get("packet_write_score")
        if isinstance(ws, torch.Tensor):
            ws = ws.to(device=src.device, dtype=torch.float32)
            if ws.shape == mask.shape:
                ws = ws * mask.to(src.device)
        else:
            ws = None
        n = min(int(src.shape[0] * src.shape[1]), int(memory_write_tokens))
        records = append(src.detach(), bucket_ids=packet.get("packet_source_bucket_ids"), score=ws,
                         max_tokens=int(memory_write_tokens),
                         event_ids=cache.reserve_event_ids(n, device=src.device))
        if not isinstance(records, list):
            raise TypeError("append_memory_from_hidden must return generation-stamped records")
    cache.commit(txn)
    zero = torch.zeros_like(mask)
    out: dict[str, Any] = {"step_id_int": int(step), "target": zero.clone(), "confidence": zero.clone(),
                           "loss_weight": mask.clone(), "utility": zero.clone(),
                           "memory_residual": residual.detach().clone(), "memory_gate": gate.detach().clone(),
                           "memory_gate_alias_target": False,
                           "packet_source_count": int(packet.get("packet_source_count", 0)),
                           "packet_approximate": True}
    if records is not None:
        out["memory_write_records"] = records
        out["approx_memory_write_records"] = len(records)
    return out


# ---------------------------------------------------------------------------
# train step with a teacher packet
# ---------------------------------------------------------------------------
def crct_train_step(model: torch.nn.Module, inputs: torch.Tensor, targets: torch.Tensor,
                    payload: Optional[dict[str, Any]], *, precision: str = "bf16",
                    lm_head_backward_mode: str = "fused_streaming_cached",
                    lm_head_tile_size: int = 8192) -> torch.Tensor:
    """Forward + backward of a train rank under CRCT (runner_fast_path.py:9770-9870).
    The packet's residual and gate enter through the fixed pre-recurrence lane of
    ``encode(memory_mode="packet")``; without a packet that lane is an exact no-op.
    The packet's per-token weights turn the loss into
    ``sum(ce * w) / max(sum w, 1)``.  A bare trunk with weights but no residual
    stays on the kernel engine (per-row weights in the fused head's epilogue)."""
    from .precision import autocast_context
    from .train_ssm import _FUSED_LM_HEAD_BACKENDS, _engine_for, fused_lm_head_backward
    residual = payload.get("memory_residual") if payload else None
    gate = payload.get("memory_gate") if payload else None
    w = payload.get("loss_weight") if payload else None
    fused = str(lm_head_backward_mode).strip().lower() in _FUSED_LM_HEAD_BACKENDS
    if residual is None and fused and precision in ("bf16", "fp8_fused") and model.training:
        engine = _engine_for(model)
        if engine is not None:
            loss = engine.step(inputs, targets,
                               row_weight=None if w is None else weighted_row_scale(w.to(inputs.device)))
            engine.arena.materialize_grads()
            return loss
    with autocast_context(precision, device_type=inputs.device.type):
        if residual is not None and gate is not None:
            hidden = model.encode(inputs, memory_mode="packet", episodic_residual=residual, episodic_gate=gate)
        else:
            hidden = model.encode(inputs, memory_mode="packet")
        if w is None and fused:
            return fused_lm_head_backward(hidden, model.final_norm, model.lm_head, targets,
                                          tile_size=int(lm_head_tile_size))
        if fused:
            from .kernels.lm_head_loss import fused_linear_cross_entropy_weighted
            loss, _ = fused_linear_cross_entropy_weighted(model.final_norm(hidden), model.lm_head.weight,
                                                          targets.reshape(-1),
                                                          w.to(device=hidden.device, dtype=torch.float32),
                                                          tile_size=int(lm_head_tile_size))
        else:
            logits = model.lm_head(model.final_norm(hidden))
            ce = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(),
                                                   targets.reshape(-1), reduction="none").reshape(targets.shape)
            loss = ce.mean() if w is None else (ce * w.reshape(ce.shape)).sum() / w.sum().clamp_min(1.0)
        loss.backward()
        return loss.detach()


# ---------------------------------------------------------------------------
# collective transport
# ---------------------------------------------------------------------------
def broadcast_params_coalesced(model: torch.nn.Module, *, src: int, group=None) -> int:
    """Parameters and floating buffers from ``src`` to the group in as few
    broadcasts as dtypes (one, when the model lives in a flat arena).  Returns
    the number of collectives issued."""
    arena = get_arena(model)
    n = 0
    done: set[int] = set()
    if arena is not None:
        dist.broadcast(arena.flat_param, src=src, group=group)
        done = {p.data_ptr() for p in arena.params.values()}
        n += 1
    rest = [t for _, t in _weights_to_sync(model) if t.data_ptr() not in done]
    by_kind: "OrderedDict[tuple, list[torch.Tensor]]" = OrderedDict()
    for t in rest:
        by_kind.setdefault((t.device, t.dtype), []).append(t.data)
    for ts in by_kind.values():
        flat = torch._utils._flatten_dense_tensors(ts)
        dist.broadcast(flat, src=src, group=group)
        for t, s in zip(ts, torch._utils._unflatten_dense_tensors(flat, ts)):
            t.copy_(s)
        n += 1
    return n


def collect_teacher_payload_sync(*, model: Any, cache: TransactionalWakeCache,
                                 scarcity_optimizer: Optional[ScarcityAwareMemoryOptimizer], inputs: torch.Tensor,
                                 targets: torch.Tensor, rank: int, world_size: int, group, step: int,
                                 total_steps: Optional[int], tau: float, strength: float, w_max: float,
                                 alpha_max: float, memory_write_tokens: int,
                                 gradient_conflict_monitor: Optional[CrctGradientConflictMonitor] = None,
                                 memory_rank: Optional[int] = None) -> Optional[dict[str, Any]]:
    """Lock-step teacher (runner_fast_path.py:5931-6032): every rank contributes
    its ``[B, T+1]`` ids with one gather, the memory rank scores the train
    ranks' batches as one concatenated batch, and the four label planes come
    back stacked in ONE broadcast.  Returns ``None`` on the memory rank.  A
    single process scores the batch in place."""
    kw = dict(model=model, cache=cache, scarcity_optimizer=scarcity_optimizer, step=step, total_steps=total_steps,
              tau=tau, strength=strength, w_max=w_max, alpha_max=alpha_max,
              memory_write_tokens=int(memory_write_tokens), gradient_conflict_monitor=gradient_conflict_monitor)
    if int(world_size) < 2 or not dist.is_initialized():
        return score_payload_inline(inputs=inputs, targets=targets, update_model_memory_after=False, **kw)
    mem = int(world_size) - 1 if memory_rank is None else int(memory_rank)
    ids = crct_full_input_ids(inputs, targets).to(torch.int32).contiguous()
    gathered = [torch.empty_like(ids) for _ in range(world_size)] if rank == mem else None
    dist.gather(ids, gather_list=gathered, dst=mem, group=group)
    train = [r for r in range(world_size) if r != mem]
    B, T = ids.shape[0], ids.shape[1] - 1
    planes = torch.empty(4, len(train), B, T, dtype=torch.float32, device=inputs.device)
    if rank == mem:
        cat = torch.cat([gathered[r] for r in train], dim=0)
        scored = score_payload_inline(inputs=cat[:, :-1].to(inputs.dtype), targets=cat[:, 1:].to(targets.dtype),
                                      update_model_memory_after=True, **kw)
        for i, k in enumerate(("target", "confidence", "loss_weight", "utility")):
            planes[i] = scored[k].reshape(len(train), B, T)
    dist.broadcast(planes, src=mem, group=group)
    if rank == mem:
        return None
    i = train.index(rank)
    return {"step_id_int": int(step), "target": planes[0, i], "confidence": planes[1, i],
            "loss_weight": planes[2, i], "utility": planes[3, i]}


# ---------------------------------------------------------------------------
# stop predicates of a memory rank
# ---------------------------------------------------------------------------
def memory_rank_should_stop(*, steps: int, elapsed_s: float, budget_seconds: float, stop_margin_seconds: float,
                            max_steps: Optional[int] = None) -> bool:
    """A memory rank counts served packets, not trunk steps, and may serve none:
    it stops on its own wall clock (or ``max_steps`` served)."""
    if max_steps is not None and int(steps) >= int(max_steps):
        return True
    return float(elapsed_s) >= max(0.0, float(budget_seconds) - float(stop_margin_seconds))


def memory_rank_defer_stop(*, local_stop: bool, elapsed_s: float, budget_seconds: float, stop_margin_seconds: float,
                           shutdown_requested: bool) -> bool:
    """Keep polling for the train ranks' shutdown record for a bounded grace
    window past the budget so teardown is not mistaken for a timeout."""
    if not local_stop or shutdown_requested:
        return False
    return float(elapsed_s) < float(budget_seconds) + max(5.0, float(stop_margin_seconds))


# ---------------------------------------------------------------------------
# mailbox
# ---------------------------------------------------------------------------
def _align64(n: int) -> int:
    return (int(n) + 63) & ~63


def _pin(region: np.ndarray) -> bool:
    """Page-lock a shared-memory mapping so CUDA copies to and from it are DMA."""
    if not torch.cuda.is_available():
        return False
    try:
        rc = torch.cuda.cudart().cudaHostRegister(region.ctypes.data, region.nbytes, 0)
        return int(rc) == 0
    except Exception:                                       # registration is an optimisation only
        return False


def _unpin(region: Optional[np.ndarray]) -> None:
    if region is not None and torch.cuda.is_available():
        try:
            torch.cuda.cudart().cudaHostUnregister(region.ctypes.data)
        except Exception:
            pass


def _weights_to_sync(model: torch.nn.Module) -> list[tuple[str, torch.Tensor]]:
    """Parameters plus floating buffers, except the episodic store's own buffers:
    slots live on the memory rank and are never overwritten from a train rank."""
    out = [(n, p.data) for n, p in model.named_parameters()]
    out += [(n, b) for n, b in model.named_buffers()
            if b.is_floating_point() and not n.startswith("outer_model.")]
    return out


def _snapshot_tensors(model: torch.nn.Module, scope: str) -> list[tuple[str, torch.Tensor]]:
    """Ordered ``(name, tensor)`` list a weight snapshot carries when the model
    has no arena: parameters and floating buffers, optionally only the names the
    packet path reads."""
    keep = None
    if scope == "packet":
        fn = getattr(model, "packet_forward_state_keys", None)
        keep = set(fn()) if callable(fn) else None
    return [(n, t) for n, t in _weights_to_sync(model) if keep is None or n in keep]


@dataclass
class _PendingSubmit:
    record: np.ndarray
    event: Any
    kind: str


@dataclass
class MailboxMetrics:
    requests_submitted: int = 0
    requests_dropped_full: int = 0
    requests_served: int = 0
    requests_skipped_stale: int = 0
    results_received: int = 0
    results_dropped_stale: int = 0
    results_dropped_unknown_step: int = 0
    weight_snapshots_published: int = 0
    weight_snapshots_applied: int = 0
    weight_snapshots_torn: int = 0
    score_seconds: float = 0.0
    max_result_lag_steps: int = 0
    extra: dict = field(default_factory=dict)

    def as_dict(self) -> dict[str, Any]:
        d = {k: v for k, v in self.__dict__.items() if k != "extra"}
        d.update(self.extra)
        return d


class TeacherMailbox:
    """One side of the same-node teacher mailbox.

    ``role="train"`` submits ``[B, T+1]`` id batches and takes finished label
    packets; ``role="memory"`` serves them.  Four POSIX shared-memory objects
    named ``<name>_req``, ``<name>_res`` (SPSC rings of 72-byte requests and
    456-byte results), ``<name>_slab`` (tensor payloads addressed by the 40-byte
    slices inside those records) and ``<name>_w`` (96-byte header + two weight
    buffers).  The train side creates, the memory side attaches; whoever created
    unlinks.

    Slot reuse: record ``i`` of a direction owns payload slot ``i mod 2*capacity``;
    a ring holds at most ``capacity`` unread records and a reader copies a slot
    out right after popping its record, so a writer never reaches a live slot.
    """

    def __init__(self, *, name: str, role: str, batch_size: int, seq_len: int, hidden_dim: int, device: torch.device,
                 payload_dtype: torch.dtype = torch.float32, capacity: int = 8, max_local_batches: int = 8,
                 max_payload_lag_steps: int = 8, score_interval_steps: int = 1, weight_bytes: int = 0,
                 weight_snapshot_scope: str = "full", source_rank: int = 0, attach_timeout_s: float = 30.0) -> None:
        from .episodic import native as N
        if role not in ("train", "memory"):
            raise ValueError(f"role must be 'train' or 'memory', got {role!r}")
        if weight_snapshot_scope not in ("full", "packet"):
            raise ValueError(f"weight_snapshot_scope must be 'full' or 'packet'; got {weight_snapshot_scope!r}")
        if payload_dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise ValueError(f"payload_dtype must be fp32, fp16 or bf16; got {payload_dtype}")
        self._N = N
        self.name, self.role, self.device = str(name), role, torch.device(device)
        self.B, self.T, self.D = int(batch_size), int(seq_len), int(hidden_dim)
        self.payload_dtype = payload_dtype
        self.capacity = max(2, int(capacity))
        self.slots = 2 * self.capacity
        self.max_local_batches = max(1, int(max_local_batches))
        self.max_payload_lag_steps = max(0, int(max_payload_lag_steps))
        self.score_interval_steps = max(1, int(score_interval_steps))
        self.scope = weight_snapshot_scope
        self.source_rank = int(source_rank)
        self.metrics = MailboxMetrics()
        self.shutdown_requested = False
        es = torch.empty((), dtype=payload_dtype).element_size()
        self._req_bytes = _align64(self.B * (self.T + 1) * 4)
        plane, vec = _align64(self.B * self.T * es), _align64(self.D * 4)
        self._res_layout = [plane] * 4 + [_align64(self.B * self.D * es), plane, vec, vec, vec]
        self._res_bytes = sum(self._res_layout)
        self._res_base = self.slots * self._req_bytes
        slab_bytes = self._res_base + self.slots * self._res_bytes
        self._wbuf = _align64(weight_bytes)
        create = role == "train"
        t_end = time.monotonic() + float(attach_timeout_s)
        while True:
            opened: list = []
            try:
                self._req = N.Ring(N.TEACHER_REQUEST, self.capacity, shm_name=f"{name}_req", create=create)
                opened.append(self._req)
                self._res = N.Ring(N.TEACHER_RESULT, self.capacity, shm_name=f"{name}_res", create=create)
                opened.append(self._res)
                self._slab = N.ShmBytes(f"{name}_slab", slab_bytes if create else 0, create=create)
                opened.append(self._slab)
                self._w = N.ShmBytes(f"{name}_w", 128 + 2 * self._wbuf if create else 0, create=create)
                break
            except ValueError:
                for o in opened:
                    o.close()
                if create or time.monotonic() > t_end:
                    raise
                time.sleep(0.01)                            # the creating side has not opened them yet
        if self._slab.array.size < slab_bytes or self._w.array.size < 128 + 2 * self._wbuf:
            raise ValueError("teacher mailbox regions are smaller than this side's layout: both sides must be "
                             "built with the same batch, sequence, hidden and weight sizes")
        self._pinned = self.device.type == "cuda" and _pin(self._slab.array) and _pin(self._w.array)
        self._slab_t = torch.from_numpy(self._slab.array)
        self._w_t = torch.from_numpy(self._w.array)
        self._side = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self._next_req = 0
        self._next_res = 0
        self._pending: deque[_PendingSubmit] = deque()
        self._local: "OrderedDict[int, tuple[torch.Tensor, torch.Tensor]]" = OrderedDict()
        self._w_version_published = 0
        self._w_version_applied = 0
        self._w_inflight: Optional[tuple[Any, dict]] = None

    # -- slab access -----------------------------------------------------
    def _typed(self, region: torch.Tensor, off: int, nbytes: int, dtype: torch.dtype) -> torch.Tensor:
        return region[off: off + nbytes].view(dtype)

    def _slice(self, rec_slice, off: int, t: Optional[torch.Tensor]) -> None:
        if t is None:
            rec_slice["nbytes"] = 0
            return
        rec_slice["offset_bytes"], rec_slice["nbytes"] = off, t.numel() * t.element_size()
        rec_slice["dtype"], rec_slice["rank"] = _DTYPE_CODE[t.dtype], t.dim()
        shape = list(t.shape) + [0] * (4 - t.dim())
        rec_slice["shape"] = shape

    def _copy_in(self, off: int, t: torch.Tensor) -> None:
        dst = self._typed(self._slab_t, off, t.numel() * t.element_size(), t.dtype)
        dst.copy_(t.reshape(-1), non_blocking=self._pinned)

    def _copy_out(self, rec_slice, *, dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        n = int(rec_slice["nbytes"])
        if n == 0:
            return None
        dt = _CODE_DTYPE[int(rec_slice["dtype"])]
        shape = [int(s) for s in rec_slice["shape"][: int(rec_slice["rank"])]]
        src = self._typed(self._slab_t, int(rec_slice["offset_bytes"]), n, dt).reshape(shape)
        out = src.to(self.device, non_blocking=self._pinned)
        if self.device.type == "cpu":
            out = out.clone()
        return out if dtype is None else out.to(dtype)

    # -- train side --------------------------------------------------------
    def _flush_pending(self) -> None:
        while self._pending:
            p = self._pending[0]
            if p.event is not None and not p.event.query():
                return
            if p.kind == "request":
                if not self._req.push(p.record):
                    self.metrics.requests_dropped_full += 1
                else:
                    self.metrics.requests_submitted += 1
            self._pending.popleft()

    def _submit(self, inputs: torch.Tensor, targets: torch.Tensor, step: int) -> None:
        if len(self._req) + len(self._pending) >= self.capacity:
            self.metrics.requests_dropped_full += 1
            return
        ids = crct_full_input_ids(inputs, targets).to(torch.int32)
        off = (self._next_req % self.slots) * self._req_bytes
        rec = np.zeros((), dtype=self._N.TEACHER_REQUEST)
        rec["event_type"], rec["source_rank"], rec["slice_count"] = _REQ_EVENT, self.source_rank, 1
        rec["request_id"], rec["step"] = self._next_req, int(step)
        rec["weight_snapshot_version"] = self._w_version_published
        self._slice(rec["full_ids"], off, ids)
        ev = None
        if self._side is not None:
            self._side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._side):
                self._copy_in(off, ids)
                ids.record_stream(self._side)
                ev = torch.cuda.Event()
                ev.record(self._side)
        else:
            self._copy_in(off, ids)
        self._next_req += 1
        self._pending.append(_PendingSubmit(rec, ev, "request"))

    def _take_results(self, step: int) -> Optional[tuple[dict[str, Any], torch.Tensor, torch.Tensor]]:
        best = None
        while True:
            rec = self._res.pop()
            if rec is None:
                break
            self.metrics.results_received += 1
            s = int(rec["step"])
            if s not in self._local:
                self.metrics.results_dropped_unknown_step += 1
                continue
            if int(step) - s > self.max_payload_lag_steps:
                self.metrics.results_dropped_stale += 1
                self._local.pop(s, None)
                continue
            best = rec                                       # newest wins; older complete results are superseded
        if best is None:
            return None
        s = int(best["step"])
        payload: dict[str, Any] = {"step_id_int": s, "weight_snapshot_version": int(best["weight_snapshot_version"]),
                                   "score_seconds": float(best["score_seconds"])}
        for i, k in enumerate(TEACHER_RESULT_SLICE_NAMES):
            t = self._copy_out(best["slices"][i], dtype=torch.float32)
            if t is not None:
                payload[k] = t
        if int(best["flags"]) & _FLAG_GATE_ALIASES_TARGET and "memory_residual" in payload:
            payload["memory_gate"] = payload["target"]
        inputs, targets = self._local.pop(s)
        for old in [k for k in self._local if k < s]:
            self._local.pop(old)
        self.metrics.max_result_lag_steps = max(self.metrics.max_result_lag_steps, int(step) - s)
        return payload, inputs, targets

    def begin_step(self, *, inputs: torch.Tensor, targets: torch.Tensor,
                   step: int) -> Optional[tuple[dict[str, Any], torch.Tensor, torch.Tensor]]:
        """Train side, once per step.  Publishes this batch to the teacher (every
        ``score_interval_steps``), returns the newest finished packet together
        with the batch it was scored on, or ``None`` (fail open)."""
        assert self.role == "train"
        self._flush_pending()
        self._finish_weight_publish()
        if int(step) % self.score_interval_steps == 0:
            self._local[int(step)] = (inputs, targets)
            while len(self._local) > self.max_local_batches:
                self._local.popitem(last=False)
            self._submit(inputs, targets, step)
            self._flush_pending()
        return self._take_results(step)

    def request_shutdown(self) -> None:
        """Tell the memory side to stop; waits (bounded) for copies in flight first."""
        if self.role != "train":
            return
        t_end = time.monotonic() + 2.0
        while self._pending and time.monotonic() < t_end:
            self._flush_pending()
            time.sleep(0.001)
        rec = np.zeros((), dtype=self._N.TEACHER_REQUEST)
        rec["event_type"], rec["source_rank"], rec["flags"] = _REQ_EVENT, self.source_rank, _FLAG_SHUTDOWN
        rec["request_id"] = self._next_req
        while not self._req.push(rec) and time.monotonic() < t_end:
            time.sleep(0.001)

    # -- weight snapshot ---------------------------------------------------
    def _weight_source(self, model: torch.nn.Module) -> list[torch.Tensor]:
        arena = get_arena(model)
        if arena is not None:
            return [arena.flat_param]
        return [t for _, t in _snapshot_tensors(model, self.scope)]

    def _header(self) -> np.ndarray:
        return self._w.array[:96].view(self._N.WEIGHT_SNAPSHOT_HEADER)

    def maybe_publish_weight_snapshot(self, model: torch.nn.Module, *, step: int, interval: int) -> bool:
        """Train side: every ``interval`` steps copy the weights into the inactive
        buffer; the header flips to it once the copy has completed."""
        if self.role != "train" or interval <= 0 or int(step) % int(interval) != 0 or self._w_inflight is not None:
            return False
        src = self._weight_source(model)
        total = sum(t.numel() * t.element_size() for t in src)
        if total > self._wbuf:
            raise ValueError(f"weight snapshot needs {total} bytes, the mailbox was sized for {self._wbuf}")
        version = self._w_version_published + 1
        buf = version & 1
        base = 128 + buf * self._wbuf

        def copy_all() -> None:
            off = base
            for t in src:
                n = t.numel() * t.element_size()
                self._typed(self._w_t, off, n, t.dtype).copy_(t.detach().reshape(-1), non_blocking=self._pinned)
                off += n
        ev = None
        if self._side is not None:
            self._side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._side):
                copy_all()
                ev = torch.cuda.Event()
                ev.record(self._side)
        else:
            copy_all()
        self._w_inflight = (ev, {"version": version, "buf": buf, "step": int(step), "total": total,
                                 "count": len(src)})
        self._finish_weight_publish()
        return True

    def _finish_weight_publish(self) -> None:
        if self._w_inflight is None:
            return
        ev, info = self._w_inflight
        if ev is not None and not ev.query():
            return
        h = self._header()
        h["magic"], h["wire_version"], h["header_bytes"] = self._N.WEIGHT_SNAPSHOT_MAGIC, 1, 96
        h["step"], h["total_bytes"], h["tensor_count"] = info["step"], info["total"], info["count"]
        h["active_buffer"] = info["buf"]
        h["checksum"] = (info["total"] * 0x9E3779B97F4A7C15 + info["version"]) & 0xFFFFFFFFFFFFFFFF
        h["snapshot_version"] = info["version"]              # written last: readers key on it
        self._w_version_published = info["version"]
        self._w_inflight = None
        self.metrics.weight_snapshots_published += 1

    def poll_weight_snapshot(self, model: torch.nn.Module) -> bool:
        """Memory side: load the newest published weights, if newer than applied.
        A snapshot that was overwritten while being read is discarded."""
        h = self._header()[0]
        magic, v, total = int(h["magic"]), int(h["snapshot_version"]), int(h["total_bytes"])
        checksum, active = int(h["checksum"]), int(h["active_buffer"])
        if magic != self._N.WEIGHT_SNAPSHOT_MAGIC or v <= self._w_version_applied:
            return False
        if checksum != (total * 0x9E3779B97F4A7C15 + v) & 0xFFFFFFFFFFFFFFFF:
            self.metrics.weight_snapshots_torn += 1         # header caught mid-update: next poll
            return False
        dst = self._weight_source(model)
        if sum(t.numel() * t.element_size() for t in dst) != total:
            raise ValueError("weight snapshot layout differs between the train and the memory rank")
        base = 128 + active * self._wbuf
        staged, off = [], base
        for t in dst:
            n = t.numel() * t.element_size()
            staged.append(self._typed(self._w_t, off, n, t.dtype).reshape(t.shape).to(t.device, copy=True))
            off += n
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        v2 = int(self._header()[0]["snapshot_version"])
        if v2 >= v + 2:                                      # lapped: this buffer was being rewritten
            self.metrics.weight_snapshots_torn += 1
            return False
        with torch.no_grad():
            for t, s in zip(dst, staged):
                t.copy_(s)
        self._w_version_applied = v
        self.metrics.weight_snapshots_applied += 1
        return True

    # -- memory side -------------------------------------------------------
    def pop_request(self) -> Optional[tuple[int, int, torch.Tensor]]:
        """Newest waiting request as ``(request_id, step, ids[B, T+1])``; older
        ones are skipped (drop, don't queue).  Sets ``shutdown_requested``."""
        assert self.role == "memory"
        newest = None
        while True:
            rec = self._req.pop()
            if rec is None:
                break
            if int(rec["flags"]) & _FLAG_SHUTDOWN:
                self.shutdown_requested = True
                continue
            if newest is not None:
                self.metrics.requests_skipped_stale += 1
            newest = rec
        if newest is None:
            return None
        ids = self._copy_out(newest["full_ids"])
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        return int(newest["request_id"]), int(newest["step"]), ids

    def push_result(self, *, request_id: int, step: int, scored: dict[str, Any], score_seconds: float) -> bool:
        assert self.role == "memory"
        if len(self._res) >= self.capacity:
            return False
        rec = np.zeros((), dtype=self._N.TEACHER_RESULT)
        rec["event_type"], rec["source_rank"] = _RES_EVENT, self.source_rank
        rec["request_id"], rec["step"] = int(request_id), int(step)
        rec["weight_snapshot_version"], rec["payload_version"] = self._w_version_applied, self._next_res
        rec["score_seconds"] = float(score_seconds)
        rec["target_token_count"], rec["hidden_dim"] = self.B * self.T, self.D
        alias = bool(scored.get("memory_gate_alias_target")) and "memory_residual" in scored
        off = self._res_base + (self._next_res % self.slots) * self._res_bytes
        n_slices = 0
        for i, k in enumerate(TEACHER_RESULT_SLICE_NAMES):
            t = scored.get(k)
            if k == "memory_gate" and alias:
                t = None
            if isinstance(t, torch.Tensor):
                plane = k in ("target", "confidence", "loss_weight", "utility", "memory_residual", "memory_gate")
                t = t.detach().to(self.payload_dtype if plane else torch.float32).contiguous()
                if t.numel() * t.element_size() > self._res_layout[i]:
                    raise ValueError(f"teacher result {k} {tuple(t.shape)} does not fit its mailbox slot")
                self._copy_in(off, t)
                self._slice(rec["slices"][i], off, t)
                n_slices += 1
                if k.startswith("plasticity"):
                    rec["plasticity_dim"] = t.numel()
            off += self._res_layout[i]
        rec["slice_count"] = n_slices
        if alias:
            rec["flags"] = int(rec["flags"]) | _FLAG_GATE_ALIASES_TARGET
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        ok = self._res.push(rec)
        if ok:
            self._next_res += 1
            self.metrics.requests_served += 1
            self.metrics.score_seconds += float(score_seconds)
        return ok

    # -- teardown ----------------------------------------------------------
    def close(self, *, unlink: Optional[bool] = None) -> None:
        unlink = (self.role == "train") if unlink is None else bool(unlink)
        if self._side is not None:
            self._side.synchronize()
        if self._pinned:
            _unpin(self._slab.array)
            _unpin(self._w.array)
            self._pinned = False
        self._slab_t = self._w_t = None
        for r in (self._req, self._res):
            r.close(unlink=unlink)
        for r in (self._slab, self._w):
            r.close(unlink=unlink)


# ---------------------------------------------------------------------------
# slot-commit lane between two memory ranks
# ---------------------------------------------------------------------------
_LANE_MAGIC = 0x4343424C414E4531
_LANE_FIELDS = 16
_SURVIVAL_SCALE = 1_000_000


class SlotCommitPeerLane:
    """Lane that carries ``SlotCommit`` records between the packet-serving rank
    and the maintenance rank of a split-memory topology (role of
    runner_fast_path.py:1942-2455).  The packet rank publishes its APPEND
    commits, the maintenance rank publishes confirmed maintenance commits back;
    train ranks never touch it.

    A commit is a few hundred bytes that the host produces and the host
    consumes (the slot table is host-managed), so the lane is a pair of SPSC
    rings in POSIX shared memory, ``<name>_p2m`` and ``<name>_m2p``, not a device
    send: nothing to match, nothing to abandon at shutdown, and a poll is exact.
    Record: 16 int64 ``[magic, version, seq, slot_id, action, step,
    base_generation (-1 = none), new_generation, bucket_id, event_id,
    survival * 1e6, dtype code, numel, rows, cols, 0]`` plus ``max_payload_bytes``
    of tensor data.  A full ring drops the oldest queued commit on the sending
    side (``queue_overwrites``); a commit against a generation the mirror has
    moved past is dropped on the receiving side (``stale_generation_drops``).
    The packet rank creates the rings, the maintenance rank attaches."""

    def __init__(self, *, name: str, rank: int, packet_rank: int, maintenance_rank: int,
                 ring_capacity: int = 1024, queue_capacity: int = 1024, max_payload_bytes: int = 4096,
                 attach_timeout_s: float = 30.0) -> None:
        from .episodic import native as N
        self.rank, self.packet_rank, self.maintenance_rank = int(rank), int(packet_rank), int(maintenance_rank)
        self.participant = self.rank in (self.packet_rank, self.maintenance_rank)
        self.capacity = max(1, int(queue_capacity))
        self.max_payload = int(max_payload_bytes)
        self._dtype = np.dtype([("hdr", "<i8", (_LANE_FIELDS,)), ("payload", "u1", (self.max_payload,))])
        self._q: deque = deque()
        self._seq = 0
        self._tx = self._rx = None
        self.metrics: dict[str, Any] = {
            "mode": "slot_commit_shm_ring", "participant": self.participant, "submitted": 0,
            "queue_overwrites": 0, "sent": 0, "received": 0, "applied": 0, "dropped": 0,
            "stale_generation_drops": 0, "append_commits_applied": 0, "maintenance_commits_applied": 0,
            "oversize_drops": 0, "last_drop_reason": ""}
        if not self.participant:
            return
        creator = self.rank == self.packet_rank
        self._creator = creator
        self._names = (f"{name}_p2m", f"{name}_m2p")
        t_end = time.monotonic() + float(attach_timeout_s)
        while True:
            opened: list = []
            try:
                for nm in self._names:
                    opened.append(N.Ring(self._dtype, int(ring_capacity), shm_name=nm, create=creator))
                break
            except ValueError:
                for o in opened:
                    o.close()
                if creator or time.monotonic() > t_end:
                    raise
                time.sleep(0.01)
        p2m, m2p = opened
        self._tx, self._rx = (p2m, m2p) if creator else (m2p, p2m)

    def _record(self, c) -> Optional[np.ndarray]:
        from .slot_commit import slot_commit_dtype_code
        rec = np.zeros((), dtype=self._dtype)
        t = None if c.tensor is None else c.tensor.detach().cpu().contiguous()
        rows = cols = nbytes = 0
        if t is not None:
            rows, cols = t.reshape(-1, t.shape[-1]).shape if t.dim() else (1, 1)
            nbytes = t.numel() * t.element_size()
            if nbytes > self.max_payload:
                return None
            rec["payload"][:nbytes] = t.reshape(-1).view(torch.uint8).numpy()
        rec["hdr"] = [_LANE_MAGIC, 1, self._seq, c.slot_id, int(c.action), c.step,
                      -1 if c.base_generation is None else c.base_generation, c.new_generation, c.bucket_id,
                      c.event_id, int(round(float(c.survival_factor) * _SURVIVAL_SCALE)),
                      0 if t is None else slot_commit_dtype_code(t.dtype), 0 if t is None else t.numel(),
                      rows, cols, nbytes]
        return rec

    def submit(self, commit) -> None:
        if not self.participant:
            return
        if len(self._q) >= self.capacity:
            self._q.popleft()
            self.metrics["queue_overwrites"] += 1
        self._q.append(commit)
        self.metrics["submitted"] += 1

    def pump(self, model: Any) -> int:
        """Push queued commits while the ring has room, then apply every commit
        that has arrived.  Returns how many were applied."""
        if not self.participant or self._tx is None:
            return 0
        while self._q:
            rec = self._record(self._q[0])
            if rec is None:
                self._q.popleft()
                self.metrics["oversize_drops"] += 1
                continue
            if not self._tx.push(rec):
                break
            self._q.popleft()
            self._seq += 1
            self.metrics["sent"] += 1
        applied = 0
        while True:
            rec = self._rx.pop()
            if rec is None:
                break
            self.metrics["received"] += 1
            applied += self._apply(model, rec)
        return applied

    def _apply(self, model: Any, rec) -> int:
        from .slot_commit import (SlotCommit, SlotCommitAction, apply_append_slot_commit_to_model,
                                  apply_slot_commit_to_model, slot_commit_dtype_from_code)
        m = [int(v) for v in rec["hdr"]]
        if m[0] != _LANE_MAGIC:
            self.metrics["dropped"] += 1
            self.metrics["last_drop_reason"] = "bad_magic"
            return 0
        tensor = None
        if m[12] > 0:
            raw = torch.from_numpy(np.array(rec["payload"][: m[15]], copy=True))
            tensor = raw.view(slot_commit_dtype_from_code(m[11])).reshape(m[13], m[14])
            dev = next(model.parameters()).device
            tensor = tensor.to(dev)
        action = SlotCommitAction(m[4])
        c = SlotCommit(slot_id=m[3], action=action, step=m[5], base_generation=None if m[6] < 0 else m[6],
                       new_generation=m[7], bucket_id=m[8], event_id=m[9],
                       survival_factor=m[10] / _SURVIVAL_SCALE, tensor=tensor)
        append = action is SlotCommitAction.APPEND
        ok, why = (apply_append_slot_commit_to_model if append else apply_slot_commit_to_model)(model, c)
        if ok:
            self.metrics["applied"] += 1
            self.metrics["append_commits_applied" if append else "maintenance_commits_applied"] += 1
            return 1
        self.metrics["dropped"] += 1
        self.metrics["last_drop_reason"] = why
        if why == "stale_generation":
            self.metrics["stale_generation_drops"] += 1
        return 0

    def close(self, model: Any = None) -> None:
        """Drain what has already arrived, then release (and, on the creating side, unlink) the rings."""
        if not self.participant or self._tx is None:
            return
        if model is not None:
            self.pump(model)
        for r in (self._tx, self._rx):
            r.close(unlink=self._creator)
        self._tx = self._rx = None
        self.participant = False


# ---------------------------------------------------------------------------
# runtime object the training loop talks to
# ---------------------------------------------------------------------------
def _weight_bytes(model: torch.nn.Module, scope: str) -> int:
    arena = get_arena(model)
    if arena is not None:
        return arena.flat_param.numel() * arena.flat_param.element_size()
    return sum(t.numel() * t.element_size() for _, t in _snapshot_tensors(model, scope))


class CrctRuntime:
    """Everything ``crct_enabled`` adds to a training run.

    Transport modes (``crct_teacher_transport_mode``):

    * ``"inline"`` (forced when there is one rank): the training rank scores its
      own batch every ``crct_score_interval_steps``.
    * ``"sync"``: lock-step gather/score/broadcast with the memory rank.
    * ``"async_rank0_memory_mailbox"``: train rank 0 and the memory rank talk
      through :class:`TeacherMailbox`; the other train ranks bypass the teacher.

    With more than one rank the last rank is the memory rank: it runs
    :meth:`run_memory_rank` instead of the training loop and never joins the
    gradient group.
    """

    def __init__(self, *, model: torch.nn.Module, config: dict[str, Any], rank: int, world_size: int,
                 device: torch.device, batch_size: int, seq_len: int, total_steps: Optional[int] = None,
                 all_group=None) -> None:
        get = config.get
        outer = getattr(model, "outer_model", None)
        if outer is None or not callable(getattr(model, "append_memory_from_hidden", None)):
            raise ValueError("crct_enabled needs a model with an append-only multi-slot episodic store "
                             "(outer_model_dim > 0, outer_model_type='multislot', buffer_mode='append_only')")
        self.model, self.rank, self.world_size, self.device = model, int(rank), int(world_size), device
        self.total_steps = total_steps
        self.topology = crct_rank_topology(world_size=world_size,
                                           split_memory_ranks=bool(get("crct_split_memory_ranks", False)))
        self.memory_rank = self.topology["packet_rank"] if world_size > 1 else -1     # the sync teacher
        self.is_memory_rank = world_size > 1 and rank in self.topology["memory_ranks"]
        mode = get("crct_teacher_transport_mode")
        if mode is None:
            # the reference's pair of keys: asynchronous transport on / off, and which carrier
            if not bool(get("crct_async_teacher_transport", True)):
                mode = "sync"
            else:
                backend = str(get("crct_async_teacher_transport_backend", "mailbox")).strip().lower()
                if backend in ("mailbox", "file", "file_mailbox"):
                    mode = "async_rank0_memory_mailbox"
                elif backend in ("collective", "broadcast", "nccl"):
                    mode = "sync"                      # lock-step collectives with the memory rank
                else:
                    raise ValueError("crct_async_teacher_transport_backend must be one of 'collective' or 'mailbox'; "
                                     f"got {backend!r}")
        mode = str(mode).strip().lower()
        if world_size == 1:
            mode = "inline"
        if mode not in ("inline", "sync", "async_rank0_memory_mailbox"):
            raise ValueError("crct_teacher_transport_mode must be inline, sync or async_rank0_memory_mailbox; "
                             f"got {mode!r}")
        if self.topology["split_memory_ranks"] and mode != "async_rank0_memory_mailbox":
            raise ValueError("split memory ranks need the mailbox transport")
        self.mode = mode
        def first(*names, default):
            """First key that the config carries: the reference's key names and this package's own."""
            for n in names:
                if n in config and config[n] is not None:
                    return config[n]
            return default
        self.tau = float(get("crct_lm_weight_tau", 0.10))
        self.strength = float(get("crct_lm_weight_strength", 0.10))
        self.w_max = float(get("crct_lm_weight_w_max", 1.20))
        self.alpha_max = float(get("crct_lm_weight_alpha_max", 0.15))
        self.write_tokens = int(get("crct_memory_write_tokens_per_step", 256))
        self.score_interval = max(1, int(first("crct_teacher_score_interval_steps", "crct_score_interval_steps", default=1)))
        self.param_sync_interval = int(first("crct_teacher_param_sync_interval_steps", "crct_teacher_param_sync_interval",
                                             default=16))
        # per-stage seconds of the scoring pass, summed over the run (off by default: the timers synchronise)
        self.stage_timing = bool(get("crct_score_stage_timing_enabled", False))
        self.stage_seconds: dict[str, float] = {}
        self.stage_samples = 0
        self.plasticity_strength = float(get("crct_plasticity_budget_strength", 0.25))
        self.plasticity_applied = self.plasticity_missing = 0
        self.approximate_packets = bool(get("crct_approximate_packets", False))
        self.cache = TransactionalWakeCache()
        self.scarcity = (ScarcityAwareMemoryOptimizer(tau=self.tau,
                                                      target_read_rate=float(get("crct_target_read_rate", 0.25)),
                                                      target_write_rate=float(get("crct_target_write_rate", 0.10)),
                                                      dual_lr=float(get("crct_dual_lr", 0.01)),
                                                      ema_beta=float(get("crct_ema_beta", 0.95)),
                                                      max_price=float(get("crct_max_price", 0.50)))
                         if bool(get("crct_scarcity_enabled", True)) else None)
        self.conflict = None
        if bool(get("crct_gradient_conflict_enabled", False)):
            opts = {k: config[f"crct_gradient_conflict_{k}"] for k in
                    ("ema_beta", "catastrophic_threshold", "soft_gate_strength", "soft_gate_floor", "trace_path",
                     "trace_stride", "trace_max_rows", "trace_flush_rows")
                    if config.get(f"crct_gradient_conflict_{k}") is not None}
            self.conflict = CrctGradientConflictMonitor(enabled=True, **opts)
        topo = self.topology
        split = topo["split_memory_ranks"]
        self.packet_rank, self.maint_rank = topo["packet_rank"], topo["maintenance_rank"]
        self.is_packet_rank = world_size > 1 and rank == self.packet_rank
        self.is_maintenance_rank = world_size > 1 and rank == self.maint_rank
        self.replay_loop = None
        if bool(get("replay_eviction_enabled", False)) and (self.is_maintenance_rank or world_size == 1):
            from .replay_eviction import ReplayEvictionLoop
            kw = {k[len("replay_eviction_"):]: v for k, v in config.items()
                  if k.startswith("replay_eviction_") and k != "replay_eviction_enabled" and v is not None}
            # the reference's runner keys for five of the loop's options
            for ref_key, own in (("mode", "action_mode"), ("threshold", "eviction_threshold"),
                                 ("ema_beta", "eviction_ema_beta"), ("min_age_steps", "min_slot_age_steps"),
                                 ("max_seconds", "max_seconds_per_tick")):
                if ref_key in kw:
                    kw.setdefault(own, kw.pop(ref_key))
            self.replay_loop = ReplayEvictionLoop(**kw)
        # process groups: every rank must take part in every new_group call, in the same order
        self.all_group = all_group
        self.train_group = self.teacher_group = self.maint_group = self.peer_group = None
        if world_size > 1:
            backend = "nccl" if device.type == "cuda" else "gloo"
            self.train_group = dist.new_group(topo["train_ranks"], backend=backend)
            self.teacher_group = dist.new_group(sorted({0, self.packet_rank}), backend=backend)
            if split:
                self.maint_group = dist.new_group(sorted({0, self.maint_rank}), backend=backend)
                self.peer_group = dist.new_group([self.packet_rank, self.maint_rank], backend=backend)
        self.grad_world_size = topo["grad_world_size"] if world_size > 1 else 1
        self.mailbox: Optional[TeacherMailbox] = None           # rank 0 <-> packet rank
        self.maint_mailbox: Optional[TeacherMailbox] = None     # rank 0 -> maintenance rank (split topology)
        self.lane: Optional[SlotCommitPeerLane] = None
        if self.mode == "async_rank0_memory_mailbox" and rank in (0, self.packet_rank, self.maint_rank):
            name = str(get("crct_mailbox_name", "") or
                       f"/ccb_crct_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}")
            hidden = int(getattr(model, "dim", 0) or get("model_dim", 0))
            dt = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[
                str(first("crct_async_teacher_payload_dtype", "crct_async_payload_dtype", default="fp32")).lower()]
            scope = "packet" if split else "full"

            def open_box(box_name: str, role: str, box_scope: str) -> TeacherMailbox:
                return TeacherMailbox(
                    name=box_name, role=role, batch_size=batch_size, seq_len=seq_len, hidden_dim=hidden,
                    device=device, payload_dtype=dt, capacity=int(get("crct_mailbox_capacity", 8)),
                    max_local_batches=int(first("crct_async_teacher_pending_batches", "crct_max_local_batches", default=8)),
                    max_payload_lag_steps=int(first("crct_async_teacher_max_lag_steps", "crct_max_payload_lag_steps",
                                                    default=8)),
                    score_interval_steps=self.score_interval, weight_bytes=_weight_bytes(model, box_scope),
                    weight_snapshot_scope=box_scope, source_rank=rank)
            # rank 0 creates the regions, the memory side attaches after a barrier on their two-rank group
            if rank == 0:
                self.mailbox = open_box(name, "train", scope)
                dist.barrier(group=self.teacher_group)
                if split:
                    self.maint_mailbox = open_box(name + "_m", "train", "full")
                    dist.barrier(group=self.maint_group)
            else:
                if rank == self.packet_rank:
                    dist.barrier(group=self.teacher_group)
                    self.mailbox = open_box(name, "memory", scope)
                if split and rank == self.maint_rank:
                    dist.barrier(group=self.maint_group)
                    self.maint_mailbox = open_box(name + "_m", "memory", "full")
                if split:
                    if rank == self.maint_rank:              # attach after the packet rank has created the rings
                        dist.barrier(group=self.peer_group)
                    self.lane = SlotCommitPeerLane(name=name + "_lane", rank=rank, packet_rank=self.packet_rank,
                                                   maintenance_rank=self.maint_rank,
                                                   queue_capacity=int(get("crct_slot_commit_queue", 1024)))
                    if rank == self.packet_rank:
                        dist.barrier(group=self.peer_group)
        self._mailbox_final: Optional[dict[str, Any]] = None
        self.teacher_requests = 0
        self.teacher_payloads = 0
        self.teacher_fail_open = 0
        self.teacher_bypass_steps = 0
        self.packets_served = 0
        self.param_syncs = 0

    # -- shared kwargs ------------------------------------------------------
    def _score_kw(self, step: int) -> dict[str, Any]:
        return dict(model=self.model, cache=self.cache, scarcity_optimizer=self.scarcity, step=int(step),
                    total_steps=self.total_steps, tau=self.tau, strength=self.strength, w_max=self.w_max,
                    alpha_max=self.alpha_max, memory_write_tokens=self.write_tokens,
                    gradient_conflict_monitor=self.conflict)

    def _score(self, inputs: torch.Tensor, targets: torch.Tensor, step: int) -> dict[str, Any]:
        was_training = self.model.training
        self.model.eval()
        try:
            if self.approximate_packets:
                return packet_payload_inline(model=self.model, cache=self.cache, inputs=inputs, targets=targets,
                                             step=step, memory_write_tokens=self.write_tokens)
            stages: Optional[dict[str, float]] = {} if self.stage_timing else None
            with torch.no_grad():
                out = score_payload_inline(inputs=inputs, targets=targets, update_model_memory_after=True,
                                           record_stage_seconds=stages, **self._score_kw(step))
            if stages:
                self.stage_samples += 1
                for k, v in stages.items():
                    if not k.startswith("_"):                     # underscore keys carry the problem shape
                        self.stage_seconds[k] = self.stage_seconds.get(k, 0.0) + float(v)
            return out
        finally:
            self.model.train(was_training)

    def _feed_maintenance(self, step: int) -> None:
        if self.replay_loop is None:
            return
        ids = getattr(self.model, "_last_crct_probe_input_ids", None)
        if ids is not None and getattr(self.model, "_last_crct_probe_step", None) == int(step):
            self.replay_loop.cache_probe(input_ids=ids, valid_mask=self.model._last_crct_probe_valid_mask,
                                         cue=getattr(self.model, "_last_crct_probe_outer_cue", None),
                                         cache_read_cutoff=None, step=int(step))

    def _publish_appends(self, scored: dict[str, Any], step: int) -> None:
        """Packet rank of a split topology: its slot appends go to the maintenance replica."""
        if self.lane is None:
            return
        from .slot_commit import SlotCommit, SlotCommitAction
        for r in scored.get("memory_write_records") or []:
            self.lane.submit(SlotCommit(slot_id=int(r["slot_id"]), action=SlotCommitAction.APPEND, step=int(step),
                                        base_generation=None, new_generation=int(r["generation"]),
                                        bucket_id=int(r["bucket_id"]), event_id=int(r["event_id"]),
                                        tensor=r["tensor"]))

    def _maintenance_tick(self, step: int) -> None:
        out = self.replay_loop.tick(model=self.model, step=step)
        if self.lane is not None:                            # confirmed decisions go to the packet rank's mirror
            for c in out.slot_commits:
                self.lane.submit(c)

    # -- train rank ----------------------------------------------------------
    def begin_step(self, inputs: torch.Tensor, targets: torch.Tensor,
                   step: int) -> tuple[Optional[dict[str, Any]], torch.Tensor, torch.Tensor]:
        """``(payload or None, inputs, targets)`` for this step.  With the mailbox
        the returned batch is the one the payload was scored on."""
        payload = None
        if self.mode == "inline":
            if step % self.score_interval == 0:
                self.teacher_requests += 1
                payload = self._score(inputs, targets, step)
                self._feed_maintenance(step)
        elif self.mode == "sync":
            self.teacher_requests += 1
            payload = collect_teacher_payload_sync(inputs=inputs, targets=targets, rank=self.rank,
                                                   world_size=self.world_size, group=self.all_group,
                                                   memory_rank=self.memory_rank, **self._score_kw(step))
        elif self.mailbox is None:
            self.teacher_bypass_steps += 1
            return None, inputs, targets
        else:
            self.teacher_requests += 1
            if self.maint_mailbox is not None:                # probe frames for the maintenance rank
                self.maint_mailbox.begin_step(inputs=inputs, targets=targets, step=step)
            ready = self.mailbox.begin_step(inputs=inputs, targets=targets, step=step)
            if ready is not None:
                payload, inputs, targets = ready
        if payload is None:
            self.teacher_fail_open += 1
        else:
            self.teacher_payloads += 1
        return payload, inputs, targets

    def apply_plasticity_budget(self, optimizer: Any, payload: Optional[dict[str, Any]]) -> bool:
        """Before the optimizer step: hand the packet's per-channel plasticity budget to an optimizer that
        takes one (``set_plasticity_budget``, e.g. Muon), so channels whose memory residual tracked utility
        move faster this step (runner_fast_path.py:1727-1751 of the reference).  Counts what was applied and
        what arrived without a budget."""
        setter = getattr(optimizer, "set_plasticity_budget", None)
        budget = payload.get("plasticity_budget") if isinstance(payload, dict) else None
        if not callable(setter) or not isinstance(budget, torch.Tensor):
            if payload is not None:
                self.plasticity_missing += 1
            return False
        conf = payload.get("plasticity_confidence")
        step = payload.get("step_id_int")
        if not isinstance(step, int) and isinstance(payload.get("step_id"), torch.Tensor):
            step = int(payload["step_id"].detach().cpu().item())
        setter(budget.detach(), confidence=conf.detach() if isinstance(conf, torch.Tensor) else None,
               strength=self.plasticity_strength, step=step if isinstance(step, int) else None)
        self.plasticity_applied += 1
        return True

    def after_optimizer_step(self, step: int) -> None:
        """Train side: weight hand-off to the teacher; inline maintenance."""
        if self.mode == "async_rank0_memory_mailbox" and self.mailbox is not None:
            if self.mailbox.maybe_publish_weight_snapshot(self.model, step=step, interval=self.param_sync_interval):
                self.param_syncs += 1
            if self.maint_mailbox is not None:
                self.maint_mailbox.maybe_publish_weight_snapshot(self.model, step=step,
                                                                 interval=self.param_sync_interval)
        elif self.mode == "sync" and self.param_sync_interval > 0 and step % self.param_sync_interval == 0:
            if self.rank in (0, self.memory_rank):
                self.param_syncs += broadcast_params_coalesced(self.model, src=0, group=self.teacher_group)
        elif self.mode == "inline" and self.replay_loop is not None:
            self.replay_loop.tick(model=self.model, step=step)

    # -- memory rank ---------------------------------------------------------
    def run_memory_rank(self, *, budget_seconds: float, stop_margin_seconds: float, max_steps: Optional[int],
                        batch_shape: tuple[int, int], input_dtype: torch.dtype = torch.int32,
                        time_fn=time.perf_counter, idle_sleep_s: float = 0.0005) -> dict[str, Any]:
        """Service loop of the memory rank.  Mailbox: poll weights, serve the
        newest request, otherwise run one maintenance tick; stop on the
        shutdown record or the wall clock (+ grace).  Sync: mirror the train
        ranks' collectives step for step until they signal stop."""
        t0 = time_fn()
        self.model.eval()
        served = 0
        ticks = 0
        if self.mode == "sync":
            B, T = batch_shape
            dummy_in = torch.zeros(B, T, dtype=input_dtype, device=self.device)
            dummy_tg = torch.zeros(B, T, dtype=torch.long, device=self.device)
            step = 0
            while True:
                flag = torch.zeros(1, device=self.device)
                dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.all_group)
                if flag.item() > 0.5:
                    break
                with torch.no_grad():
                    collect_teacher_payload_sync(inputs=dummy_in, targets=dummy_tg, rank=self.rank,
                                                 world_size=self.world_size, group=self.all_group,
                                                 memory_rank=self.memory_rank, **self._score_kw(step))
                self._feed_maintenance(step)
                served += 1
                if self.param_sync_interval > 0 and step % self.param_sync_interval == 0:
                    self.param_syncs += broadcast_params_coalesced(self.model, src=0, group=self.teacher_group)
                if self.replay_loop is not None:
                    self.replay_loop.tick(model=self.model, step=step)
                    ticks += 1
                step += 1
        else:
            serves = self.mailbox is not None and self.is_packet_rank
            mb = self.mailbox if serves else self.maint_mailbox
            assert mb is not None
            last_step = 0
            while True:
                elapsed = time_fn() - t0
                stop = memory_rank_should_stop(steps=served, elapsed_s=elapsed, budget_seconds=budget_seconds,
                                               stop_margin_seconds=stop_margin_seconds, max_steps=None)
                if mb.shutdown_requested:
                    break
                if stop and not memory_rank_defer_stop(local_stop=True, elapsed_s=elapsed,
                                                       budget_seconds=budget_seconds,
                                                       stop_margin_seconds=stop_margin_seconds,
                                                       shutdown_requested=False):
                    break
                mb.poll_weight_snapshot(self.model)
                if self.lane is not None:
                    self.lane.pump(self.model)
                req = mb.pop_request()
                if req is None:
                    if self.replay_loop is not None and self.replay_loop.has_probe():
                        self._maintenance_tick(last_step)
                        ticks += 1
                    else:
                        time.sleep(idle_sleep_s)
                    continue
                rid, step, ids = req
                last_step = step
                if not serves:                               # maintenance-only rank: the batch is a probe frame
                    if self.replay_loop is not None:
                        full = ids.long()
                        self.replay_loop.cache_probe(input_ids=full, valid_mask=crct_valid_mask(full), cue=None,
                                                     cache_read_cutoff=None, step=int(step))
                    served += 1
                    continue
                ts = time_fn()
                scored = self._score(ids[:, :-1].to(input_dtype), ids[:, 1:].long(), step)
                self._feed_maintenance(step)
                self._publish_appends(scored, step)
                if mb.push_result(request_id=rid, step=step, scored=scored, score_seconds=time_fn() - ts):
                    served += 1
            if self.lane is not None:
                self.lane.close(self.model)
        self.packets_served = served
        out = self.diagnostics()
        out.update({"steps": served, "elapsed_s": time_fn() - t0, "rank": self.rank, "world_size": self.world_size,
                    "role": "memory", "maintenance_ticks": ticks})
        return out

    # -- teardown ------------------------------------------------------------
    def signal_stop_sync(self, stop: bool) -> bool:
        """Sync mode: the per-step continue/stop flag every rank joins."""
        flag = torch.tensor([1.0 if stop else 0.0], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.all_group)
        return flag.item() > 0.5

    def close(self) -> None:
        if self.mailbox is not None:
            self.mailbox.request_shutdown()
            self._mailbox_final = self.mailbox.metrics.as_dict()
            self.mailbox.close()
            self.mailbox = None
        if self.maint_mailbox is not None:
            self.maint_mailbox.request_shutdown()
            if self._mailbox_final is None:
                self._mailbox_final = self.maint_mailbox.metrics.as_dict()
            self.maint_mailbox.close()
            self.maint_mailbox = None
        if self.replay_loop is not None:
            self.replay_loop.close()

    def diagnostics(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "enabled": True, "transport_mode": self.mode, "topology": self.topology,
            "teacher_requests": self.teacher_requests, "teacher_payloads": self.teacher_payloads,
            "teacher_fail_open": self.teacher_fail_open, "teacher_bypass_steps": self.teacher_bypass_steps,
            "packets_served": self.packets_served, "param_syncs": self.param_syncs,
            "lm_weight_tau": self.tau, "lm_weight_strength": self.strength, "lm_weight_w_max": self.w_max,
            "lm_weight_alpha_max": self.alpha_max, "plasticity_budget_strength": self.plasticity_strength,
            "plasticity_budget_payloads_applied": self.plasticity_applied,
            "plasticity_budget_payloads_missing": self.plasticity_missing}
        if self.stage_timing:
            d["score_stage_seconds"] = {"samples": self.stage_samples, **{k: float(v) for k, v in self.stage_seconds.items()}}
        if self.mailbox is not None:
            d["mailbox"] = self.mailbox.metrics.as_dict()
        elif self._mailbox_final is not None:
            d["mailbox"] = self._mailbox_final
        if self.lane is not None:
            d["slot_commit_lane"] = dict(self.lane.metrics)
        if self.scarcity is not None:
            d["scarcity"] = {k: float(v) for k, v in vars(self.scarcity).items() if isinstance(v, (int, float))}
        if self.replay_loop is not None:
            d["replay_eviction"] = self.replay_loop.diagnostics()
        return d
