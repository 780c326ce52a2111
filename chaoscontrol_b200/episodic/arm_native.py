"""Python face of ``native/arm.cpp``: the maintenance scheduler, the fused CPU
RMSNorm -> LM-head NLL, the evidence engine and the per-slot SSM controller learner
(what the reference exposes from its C++ extension as ``ArmMaintenanceScheduler``,
``amx_bf16_nll``, ``CpuEvidenceEngine`` and ``OnlineLearningController``:
kernels/_cpu_ssm_controller/src/cpu_ssm_controller.cpp:1390-1888, online_learning.h:39-123).
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Optional, Sequence

import numpy as np
import torch

from . import native

__all__ = ["ArmMaintenanceScheduler", "PackedLmHead", "rms_lmhead_nll", "CpuEvidenceEngine",
           "OnlineLearningController", "ssm_forward_step", "ssm_flat", "CUE_TOKENS"]

CUE_TOKENS = 32
NO_SLOT = (1 << 64) - 1
_bound = False


def _L() -> C.CDLL:
    global _bound
    L = native.lib()
    if not _bound:
        vp, u32, u64, i32, f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float
        L.ccbc_arm_sched_new.restype = vp
        L.ccbc_arm_sched_new.argtypes = [u32] * 4
        L.ccbc_arm_sched_free.argtypes = [vp]
        L.ccbc_arm_sched_ingest.argtypes = [vp, u64, u64, u32, u64]
        L.ccbc_arm_sched_next_job.argtypes = [vp, u64, vp, i32, vp]
        L.ccbc_arm_sched_record.argtypes = [vp, vp]
        L.ccbc_arm_sched_diag.argtypes = [vp, vp, vp]
        L.ccbc_lmhead_pack.restype = vp
        L.ccbc_lmhead_pack.argtypes = [vp, vp, i32, i32]
        L.ccbc_lmhead_free.argtypes = [vp]
        L.ccbc_rms_lmhead_nll.argtypes = [vp, vp, vp, i32, f32, vp]
        L.ccbc_rms_lmhead_nll_mode.argtypes = [vp, vp, vp, i32, f32, vp, i32]
        L.ccbc_evidence_new.restype = vp
        L.ccbc_evidence_new.argtypes = [u32, u32]
        L.ccbc_evidence_free.argtypes = [vp]
        L.ccbc_evidence_set_lm_head.argtypes = [vp, vp, vp, i32]
        L.ccbc_evidence_ingest.argtypes = [vp, vp, vp, u64, u64, u32]
        L.ccbc_evidence_shutdown.argtypes = [vp]
        L.ccbc_evidence_diag.argtypes = [vp] * 6
        L.ccbc_ssm_flat_size.restype = C.c_int64
        L.ccbc_ssm_flat_size.argtypes = [i32] * 3
        L.ccbc_ssm_forward_step.restype = f32
        L.ccbc_ssm_forward_step.argtypes = [i32] * 3 + [vp] * 6
        L.ccbc_ssm_learner_new.restype = vp
        L.ccbc_ssm_learner_new.argtypes = [u32, u32, f32, f32, f32, u32, f32, u64]
        L.ccbc_ssm_learner_free.argtypes = [vp]
        L.ccbc_ssm_learner_init.argtypes = [vp, i32, i32, i32, vp]
        L.ccbc_ssm_learner_record.argtypes = [vp, u32, u64, u32, f32, C.c_uint8, vp, i32, vp, i32, vp, i32]
        L.ccbc_ssm_learner_outcome.argtypes = [vp, vp]
        L.ccbc_ssm_learner_weights.argtypes = [vp, i32, vp]
        L.ccbc_ssm_learner_telemetry.argtypes = [vp, vp, vp]
        L.ccbc_ssm_learner_history_size.restype = C.c_int64
        L.ccbc_ssm_learner_history_size.argtypes = [vp, u32]
        L.ccbc_ssm_learner_mark_evicted.argtypes = [vp, u32, u64]
        L.ccbc_ssm_learner_is_evicted.argtypes = [vp, u32]
        L.ccbc_ssm_learner_gc.argtypes = [vp, u64, u64]
        _bound = True
    return L


# ---------------------------------------------------------------- scheduler
class ArmMaintenanceScheduler:
    _COUNTERS = ("frames_ingested", "frames_completed", "frames_dropped_stale", "frames_dropped_overflow",
                 "duplicate_frames", "jobs_emitted", "results_recorded", "slots_scheduled_total", "slots_scored_total",
                 "actions_confirmed_total", "actions_rejected_total", "result_errors", "skipped_no_frame",
                 "skipped_no_slots", "skipped_inflight", "queue_depth_max", "queue_depth")

    def __init__(self, memory_streams: int = 8, slot_work_chunk_size: int = 16, frame_ttl_steps: int = 256,
                 max_frames: int = 32) -> None:
        self._cfg = dict(memory_streams=max(1, memory_streams), slot_work_chunk_size=min(max(1, slot_work_chunk_size), 16),
                         frame_ttl_steps=frame_ttl_steps, max_frames=max(1, max_frames))
        self._h = _L().ccbc_arm_sched_new(memory_streams, slot_work_chunk_size, frame_ttl_steps, max_frames)

    def ingest_frame(self, frame_id: int, step: int, stream_id: int, cache_read_cutoff: Optional[int]) -> bool:
        cut = NO_SLOT if cache_read_cutoff is None else int(cache_read_cutoff)
        return bool(_L().ccbc_arm_sched_ingest(self._h, int(frame_id), int(step), int(stream_id), cut))

    def next_job(self, step: int, visible_slots: Sequence[int], cache_read_cutoff: Optional[int] = None
                 ) -> Optional[dict[str, Any]]:
        """The next ``ArmMaintenanceJob`` as a dict (``slot_ids`` trimmed to ``slot_count``), or ``None``."""
        vis = np.ascontiguousarray(list(visible_slots), dtype=np.uint64)
        job = np.zeros((), dtype=native.ARM_JOB)
        if not _L().ccbc_arm_sched_next_job(self._h, int(step), vis.ctypes.data, int(vis.size), job.ctypes.data):
            return None
        d = {k: job[k].item() for k in job.dtype.names if k != "slot_ids"}
        d["slot_ids"] = [int(s) for s in job["slot_ids"][: d["slot_count"]]]
        d["cache_read_cutoff"] = None if d["cache_read_cutoff"] == NO_SLOT else d["cache_read_cutoff"]
        return d

    def record_result(self, result: dict[str, Any]) -> None:
        r = np.zeros((), dtype=native.ARM_RESULT)
        r["event_type"], r["job_type"] = 5, int(result.get("job_type", 1))
        for k in ("stream_id", "status", "slot_count", "job_id", "frame_id", "step", "slots_scored",
                  "actions_confirmed", "actions_rejected", "probe_seconds", "oracle_seconds", "cpu_seconds",
                  "frame_age_seconds"):
            if k in result:
                r[k] = result[k]
        ids = list(result.get("slot_ids", []))[:16]
        r["slot_ids"][:] = NO_SLOT
        r["slot_ids"][: len(ids)] = ids
        _L().ccbc_arm_sched_record(self._h, r.ctypes.data)

    def diagnostics(self) -> dict[str, Any]:
        c = np.zeros(17, np.uint64)
        s = np.zeros(4, np.float64)
        _L().ccbc_arm_sched_diag(self._h, c.ctypes.data, s.ctypes.data)
        out: dict[str, Any] = {"enabled": True, **self._cfg, **{k: int(v) for k, v in zip(self._COUNTERS, c)}}
        out.update(probe_seconds_total=float(s[0]), oracle_seconds_total=float(s[1]), cpu_seconds_total=float(s[2]),
                   frame_age_seconds_max=float(s[3]))
        return out

    def close(self) -> None:
        if self._h:
            _L().ccbc_arm_sched_free(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------- fused CPU NLL
def _bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().to("cpu", torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)


class PackedLmHead:
    """Final-norm weight + LM-head matrix repacked once into vocabulary tiles of ``W^T``."""

    def __init__(self, norm_weight: torch.Tensor, lm_head_weight: torch.Tensor) -> None:
        self.V, self.D = int(lm_head_weight.shape[0]), int(lm_head_weight.shape[1])
        nw = np.ascontiguousarray(norm_weight.detach().float().cpu().numpy())
        W = _bf16_bits(lm_head_weight)
        self._h = _L().ccbc_lmhead_pack(nw.ctypes.data, W.ctypes.data, self.V, self.D)

    def close(self) -> None:
        if self._h:
            _L().ccbc_lmhead_free(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def rms_lmhead_nll(head: PackedLmHead, hidden: torch.Tensor, targets: torch.Tensor, eps: float = 1e-6, *,
                   packed_amx: bool = True) -> tuple[torch.Tensor, bool]:
    """``(per-token NLL [T] fp32, used_amx)`` of ``lm_head(RMSNorm(hidden))`` computed on the host cores from
    bf16 operands; the vocabulary is streamed in tiles with an online log-sum-exp.

    On CPUs with AMX the default path multiplies straight out of the VNNI tile cache that
    ``PackedLmHead`` built once and folds each 16 x 16 logits tile into the running (max, sum);
    ``packed_amx=False`` takes the generic tile-matmul path instead (the oracle for the fused one)."""
    h = _bf16_bits(hidden.reshape(-1, head.D))
    y = np.ascontiguousarray(targets.detach().cpu().numpy().reshape(-1).astype(np.int64))
    out = np.zeros(h.shape[0], np.float32)
    used = _L().ccbc_rms_lmhead_nll_mode(head._h, h.ctypes.data, y.ctypes.data, int(h.shape[0]), float(eps),
                                         out.ctypes.data, 0 if packed_amx else 1)
    return torch.from_numpy(out), bool(used)


class CpuEvidenceEngine:
    def __init__(self, lanes: int = 8, d_model: int = 384) -> None:
        self.lanes, self.d_model = max(1, int(lanes)), max(1, int(d_model))
        self._h = _L().ccbc_evidence_new(self.lanes, self.d_model)

    def set_lm_head(self, norm_weight: torch.Tensor, lm_head_weight: torch.Tensor) -> None:
        if norm_weight.shape != (self.d_model,) or lm_head_weight.dim() != 2 or lm_head_weight.shape[1] != self.d_model:
            raise ValueError(f"set_lm_head: expected norm [{self.d_model}] and weight [V, {self.d_model}]")
        nw = np.ascontiguousarray(norm_weight.detach().float().cpu().numpy())
        W = _bf16_bits(lm_head_weight)
        _L().ccbc_evidence_set_lm_head(self._h, nw.ctypes.data, W.ctypes.data, int(lm_head_weight.shape[0]))

    def ingest_frame(self, cue_hidden: torch.Tensor, cue_targets: torch.Tensor, *, frame_id: int, step: int,
                     stream_id: int) -> None:
        if cue_hidden.dtype != torch.bfloat16 or tuple(cue_hidden.shape) != (CUE_TOKENS, self.d_model):
            raise ValueError(f"cue_hidden must be bf16 [{CUE_TOKENS}, {self.d_model}]; got {cue_hidden.dtype} "
                             f"{tuple(cue_hidden.shape)}")
        if cue_targets.dtype != torch.int32 or tuple(cue_targets.shape) != (CUE_TOKENS,):
            raise ValueError(f"cue_targets must be int32 [{CUE_TOKENS}]")
        h = _bf16_bits(cue_hidden)
        y = np.ascontiguousarray(cue_targets.cpu().numpy())
        if _L().ccbc_evidence_ingest(self._h, h.ctypes.data, y.ctypes.data, int(frame_id), int(step), int(stream_id)):
            raise RuntimeError("CpuEvidenceEngine.ingest_frame called after shutdown")

    def shutdown(self) -> None:
        _L().ccbc_evidence_shutdown(self._h)

    def diagnostics(self) -> dict[str, Any]:
        u, f = np.zeros(8, np.uint64), np.zeros(7, np.float64)
        la, lw, ls = np.zeros(self.lanes, np.uint64), np.zeros(self.lanes, np.uint64), np.zeros(self.lanes, np.float64)
        _L().ccbc_evidence_diag(self._h, u.ctypes.data, f.ctypes.data, la.ctypes.data, lw.ctypes.data, ls.ctypes.data)
        key = lambda a: {str(i): (float(v) if a.dtype.kind == "f" else int(v)) for i, v in enumerate(a)}
        return {"enabled": not bool(u[7]), "lanes": self.lanes, "t_probe_max": CUE_TOKENS, "k_tile": 64,
                "d_model": self.d_model, "frames_ingested": int(u[0]), "last_frame_id": int(u[1]),
                "last_step": int(u[2]), "last_stream_id": int(u[3]), "lm_head_set": bool(u[4]),
                "lm_head_set_count": int(u[4]), "cue_nll_calls_total": int(u[5]), "used_amx": bool(u[6]),
                "cue_nll_seconds_total": float(f[0]), "last_cue_nll_seconds": float(f[1]),
                "cue_nll_mean_ema": float(f[2]), "cue_nll_finite_fraction_ema": float(f[3]),
                "last_cue_nll_mean": float(f[4]), "last_cue_nll_max": float(f[5]),
                "last_cue_nll_finite_fraction": float(f[6]), "lane_tile_advances_total": key(la),
                "lane_work_items_emitted_total": key(lw), "lane_cue_nll_seconds_total": key(ls)}

    def close(self) -> None:
        if self._h:
            _L().ccbc_evidence_free(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------- per-slot SSM controller
_ORDER = ("w_global_in", "w_slot_in", "decay_global", "decay_slot", "w_global_out", "w_slot_out", "bias")


def ssm_flat(weights: Any) -> tuple[np.ndarray, int, int, int]:
    """Flat fp32 vector of a ``CpuSsmControllerWeights`` in the native layout, with ``(F, G, S)``."""
    d = weights.to_dict()
    flat = np.concatenate([d[k].numpy().reshape(-1) for k in _ORDER]).astype(np.float32)
    return np.ascontiguousarray(flat), weights.feature_dim, weights.global_dim, weights.slot_dim


def _unflat(flat: np.ndarray, F: int, G: int, S: int) -> dict[str, torch.Tensor]:
    sizes = (G * F, S * F, G, S, G, S, 1)
    shapes = ((G, F), (S, F), (G,), (S,), (G,), (S,), ())
    out, pos = {}, 0
    for k, n, shp in zip(_ORDER, sizes, shapes):
        out[k] = torch.from_numpy(flat[pos:pos + n].copy()).reshape(shp)
        pos += n
    return out


def ssm_forward_step(weights: Any, features, global_state, slot_state) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One native controller step: ``(new_global, new_slot, logit)``."""
    flat, F, G, S = ssm_flat(weights)
    f = np.ascontiguousarray(np.asarray(features, np.float32).reshape(F))
    g = np.ascontiguousarray(np.asarray(global_state, np.float32).reshape(G))
    s = np.ascontiguousarray(np.asarray(slot_state, np.float32).reshape(S))
    ng, ns = np.zeros(G, np.float32), np.zeros(S, np.float32)
    logit = _L().ccbc_ssm_forward_step(F, G, S, flat.ctypes.data, f.ctypes.data, g.ctypes.data, s.ctypes.data,
                                       ng.ctypes.data, ns.ctypes.data)
    return torch.from_numpy(ng), torch.from_numpy(ns), torch.tensor(float(logit))


class OnlineLearningController:
    """Per-slot action history + delayed credit for the diagonal-SSM slot controller."""
    TELEMETRY = ("replay_outcomes", "history_appends", "credited_actions", "nonzero_credit_actions",
                 "backward_skipped_missing_weights", "backward_skipped_bad_shape", "invalid_slot_skips", "sgd_steps",
                 "ema_blends")

    def __init__(self, num_slots: int = 4096, max_entries_per_slot: int = 64, gamma: float = 0.995,
                 gerber_c: float = 0.5, learning_rate: float = 1e-3, sgd_interval: int = 256,
                 ema_alpha: float = 0.25, ema_interval: int = 64) -> None:
        self._h = _L().ccbc_ssm_learner_new(num_slots, max_entries_per_slot, gamma, gerber_c, learning_rate,
                                            sgd_interval, ema_alpha, ema_interval)
        self._dims: Optional[tuple[int, int, int]] = None

    def initialize_weights(self, weights: Any) -> None:
        flat, F, G, S = ssm_flat(weights)
        _L().ccbc_ssm_learner_init(self._h, F, G, S, flat.ctypes.data)
        self._dims = (F, G, S)

    @property
    def weights_initialized(self) -> bool:
        return self._dims is not None

    def record_replay_selection(self, *, slot_id: int, gpu_step: int, policy_version: int, output_logit: float,
                                selected_rank: int, features, global_state, slot_state) -> None:
        f, g, s = (np.ascontiguousarray(np.asarray(v, np.float32).reshape(-1)) for v in (features, global_state, slot_state))
        _L().ccbc_ssm_learner_record(self._h, int(slot_id), int(gpu_step), int(policy_version), float(output_logit),
                                     int(selected_rank) & 0xFF, f.ctypes.data, f.size, g.ctypes.data, g.size,
                                     s.ctypes.data, s.size)

    def on_replay_outcome(self, ev: np.ndarray) -> None:
        rec = np.ascontiguousarray(ev, dtype=native.REPLAY_OUTCOME)
        _L().ccbc_ssm_learner_outcome(self._h, rec.ctypes.data)

    def _weights(self, slow: bool) -> dict[str, torch.Tensor]:
        if self._dims is None:
            raise RuntimeError("weights are not initialised")
        F, G, S = self._dims
        flat = np.zeros(int(_L().ccbc_ssm_flat_size(F, G, S)), np.float32)
        _L().ccbc_ssm_learner_weights(self._h, int(slow), flat.ctypes.data)
        return _unflat(flat, F, G, S)

    def fast_weights(self) -> dict[str, torch.Tensor]:
        return self._weights(False)

    def slow_weights(self) -> dict[str, torch.Tensor]:
        return self._weights(True)

    def telemetry(self) -> dict[str, Any]:
        t, c = np.zeros(9, np.uint64), np.zeros(1, np.float32)
        _L().ccbc_ssm_learner_telemetry(self._h, t.ctypes.data, c.ctypes.data)
        return {**{k: int(v) for k, v in zip(self.TELEMETRY, t)}, "last_credit_sum": float(c[0])}

    def history_size(self, slot_id: int) -> int:
        return int(_L().ccbc_ssm_learner_history_size(self._h, int(slot_id)))

    def mark_evicted(self, slot_id: int, current_event_id: int) -> None:
        _L().ccbc_ssm_learner_mark_evicted(self._h, int(slot_id), int(current_event_id))

    def is_evicted(self, slot_id: int) -> bool:
        return bool(_L().ccbc_ssm_learner_is_evicted(self._h, int(slot_id)))

    def gc(self, current_event_id: int, gc_lookahead: int) -> None:
        _L().ccbc_ssm_learner_gc(self._h, int(current_event_id), int(gc_lookahead))

    def close(self) -> None:
        if self._h:
            _L().ccbc_ssm_learner_free(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
