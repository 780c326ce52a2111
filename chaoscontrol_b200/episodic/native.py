"""Python face of the C++ control plane (``libccb200_ctrl.so``): wire-record
dtypes, SPSC / shared-memory rings, credit helpers, the simplex policy and its
online learner, the CSWG reader, CPU math and the controller loop.

The numpy structured dtypes below mirror ``native/wire_format.h`` field by
field; :func:`check_wire_sizes` compares them with the sizes compiled into the
library (the reference pins the same numbers: WriteEvent 568 B, QueryEvent
736 B, ReplayOutcome 96 B, ...).
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libccb200_ctrl.so"
_lib: Optional[C.CDLL] = None

KEY_REP_DIM, SPAN_LENGTH, SIMPLEX_CANDIDATES, ARM_SLOT_CAPACITY = 256, 4, 16, 16
TEACHER_RESULT_SLICES = 9
WEIGHT_SNAPSHOT_MAGIC = 0x53574343

TENSOR_SLICE = np.dtype([("offset_bytes", "<u8"), ("nbytes", "<u8"), ("dtype", "<u4"), ("rank", "<u4"),
                         ("shape", "<u4", (4,))])
WRITE_EVENT = np.dtype([
    ("event_type", "u1"), ("source_rank", "u1"), ("write_bucket", "u1"), ("pad0", "u1", (5,)),
    ("candidate_id", "<u8"), ("gpu_step", "<u8"), ("key_fp", "<u8"),
    ("key_rep", "<u2", (KEY_REP_DIM,)), ("value_tok_ids", "<u2", (SPAN_LENGTH,)),
    ("value_anchor_id", "<u4"), ("pressure_at_write", "<f4"), ("pre_write_ce", "<f4"), ("pad1", "u1", (4,))])
QUERY_EVENT = np.dtype([
    ("event_type", "u1"), ("source_rank", "u1"), ("bucket", "u1"), ("pad0", "u1", (5,)),
    ("query_id", "<u8"), ("gpu_step", "<u8"), ("query_rep", "<u2", (KEY_REP_DIM,)),
    ("pressure", "<f4"), ("pre_query_ce", "<f4"),
    ("candidate_slot_ids", "<u8", (SIMPLEX_CANDIDATES,)), ("candidate_cosines", "<f4", (SIMPLEX_CANDIDATES,))])
REPLAY_OUTCOME = np.dtype([
    ("event_type", "u1"), ("selected_rank", "u1"), ("outcome_status", "u1"), ("pad0", "u1", (5,)),
    ("replay_id", "<u8"), ("gpu_step", "<u8"), ("query_event_id", "<u8"), ("source_write_id", "<u8"),
    ("slot_id", "<u4"), ("policy_version", "<u4"), ("selection_step", "<u8"),
    ("teacher_score", "<f4"), ("controller_logit", "<f4"), ("ce_before_replay", "<f4"),
    ("ce_after_replay", "<f4"), ("ce_delta_raw", "<f4"), ("bucket_baseline", "<f4"),
    ("reward_shaped", "<f4"), ("grad_cos_rare", "<f4"), ("grad_cos_total", "<f4"),
    ("flags", "<u2"), ("pad1", "u1", (2,))])
ARM_JOB = np.dtype([
    ("event_type", "u1"), ("job_type", "u1"), ("stream_id", "u1"), ("flags", "u1"), ("slot_count", "<u4"),
    ("job_id", "<u8"), ("frame_id", "<u8"), ("step", "<u8"), ("cache_read_cutoff", "<u8"),
    ("slot_ids", "<u8", (ARM_SLOT_CAPACITY,))])
ARM_RESULT = np.dtype([
    ("event_type", "u1"), ("job_type", "u1"), ("stream_id", "u1"), ("status", "u1"), ("slot_count", "<u4"),
    ("job_id", "<u8"), ("frame_id", "<u8"), ("step", "<u8"),
    ("slots_scored", "<u4"), ("actions_confirmed", "<u4"), ("actions_rejected", "<u4"), ("pad0", "<u4"),
    ("probe_seconds", "<f4"), ("oracle_seconds", "<f4"), ("cpu_seconds", "<f4"), ("frame_age_seconds", "<f4"),
    ("slot_ids", "<u8", (ARM_SLOT_CAPACITY,))])
TEACHER_REQUEST = np.dtype([
    ("event_type", "u1"), ("source_rank", "u1"), ("status", "u1"), ("flags", "u1"), ("slice_count", "<u4"),
    ("request_id", "<u8"), ("step", "<u8"), ("weight_snapshot_version", "<u8"), ("full_ids", TENSOR_SLICE)])
TEACHER_RESULT = np.dtype([
    ("event_type", "u1"), ("source_rank", "u1"), ("status", "u1"), ("flags", "u1"), ("slice_count", "<u4"),
    ("request_id", "<u8"), ("step", "<u8"), ("weight_snapshot_version", "<u8"), ("payload_version", "<u8"),
    ("score_seconds", "<f4"), ("packet_seconds", "<f4"), ("target_token_count", "<u4"),
    ("hidden_dim", "<u4"), ("plasticity_dim", "<u4"), ("fast_slow_mode", "<u4"),
    ("fast_slow_accepted", "<u4"), ("fast_slow_step", "<u8"), ("fast_slow_alpha", "<f4"),
    ("fast_slow_gate", "<f4"), ("fast_slow_effective_alpha", "<f4"), ("fast_slow_reason", "<u4"),
    ("pad0", "<u4"), ("slices", TENSOR_SLICE, (TEACHER_RESULT_SLICES,))])
WEIGHT_SNAPSHOT_HEADER = np.dtype([
    ("magic", "<u4"), ("wire_version", "<u4"), ("header_bytes", "<u4"), ("flags", "<u4"),
    ("step", "<u8"), ("snapshot_version", "<u8"), ("total_bytes", "<u8"), ("checksum", "<u8"),
    ("tensor_count", "<u4"), ("active_buffer", "<u4"), ("fast_slow_mode", "<u4"),
    ("fast_slow_accepted", "<u4"), ("fast_slow_step", "<u8"), ("fast_slow_alpha", "<f4"),
    ("fast_slow_gate", "<f4"), ("fast_slow_effective_alpha", "<f4"), ("fast_slow_reason", "<u4"),
    ("reserved0", "<u8")])

WIRE_DTYPES = {0: TENSOR_SLICE, 1: WRITE_EVENT, 2: QUERY_EVENT, 3: REPLAY_OUTCOME, 4: ARM_JOB,
               5: ARM_RESULT, 6: TEACHER_REQUEST, 7: TEACHER_RESULT, 8: WEIGHT_SNAPSHOT_HEADER}
EXPECTED_SIZES = {0: 40, 1: 568, 2: 736, 3: 96, 4: 168, 5: 192, 6: 72, 7: 456, 8: 96}


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(f"{_LIB_PATH} missing: run `python -m chaoscontrol_b200._build`")
        L = C.CDLL(str(_LIB_PATH))
        L.ccbc_last_error.restype = C.c_char_p
        L.ccbc_wire_sizeof.restype = C.c_int64
        L.ccbc_ring_capacity.restype = C.c_int64
        for n in ("ccbc_ring_create_local", "ccbc_ring_open_shm", "ccbc_shm_open", "ccbc_shm_ptr",
                  "ccbc_rolling_new", "ccbc_learner_new"):
            getattr(L, n).restype = C.c_void_p
        L.ccbc_ring_create_local.argtypes = [C.c_int64, C.c_int64]
        L.ccbc_ring_open_shm.argtypes = [C.c_char_p, C.c_int64, C.c_int64, C.c_int]
        L.ccbc_ring_push.argtypes = [C.c_void_p, C.c_void_p]
        L.ccbc_ring_pop.argtypes = [C.c_void_p, C.c_void_p]
        L.ccbc_ring_size.argtypes = [C.c_void_p]
        L.ccbc_ring_size.restype = C.c_int64
        L.ccbc_ring_close.argtypes = [C.c_void_p]
        L.ccbc_shm_unlink.argtypes = [C.c_char_p]
        L.ccbc_shm_open.argtypes = [C.c_char_p, C.c_int64, C.c_int]
        L.ccbc_shm_ptr.argtypes = [C.c_void_p]
        L.ccbc_shm_size.argtypes = [C.c_void_p]
        L.ccbc_shm_size.restype = C.c_int64
        L.ccbc_shm_close.argtypes = [C.c_void_p]
        L.ccbc_recency_decay.argtypes = [C.c_float, C.c_uint64, C.c_uint64, C.c_float]
        L.ccbc_recency_decay.restype = C.c_float
        L.ccbc_gerber_weight.argtypes = [C.c_float] * 3
        L.ccbc_gerber_weight.restype = C.c_float
        L.ccbc_rolling_new.argtypes = [C.c_float]
        L.ccbc_rolling_update.argtypes = [C.c_void_p, C.c_float]
        L.ccbc_rolling_mean.argtypes = [C.c_void_p]
        L.ccbc_rolling_mean.restype = C.c_float
        L.ccbc_rolling_std.argtypes = [C.c_void_p]
        L.ccbc_rolling_std.restype = C.c_float
        L.ccbc_rolling_free.argtypes = [C.c_void_p]
        L.ccbc_sgd_apply.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float]
        L.ccbc_ema_blend.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float]
        L.ccbc_simplex_flat_size.argtypes = [C.c_int] * 3
        L.ccbc_simplex_flat_size.restype = C.c_int64
        L.ccbc_simplex_forward.argtypes = [C.c_int] * 4 + [C.c_float] + [C.c_void_p] * 6
        L.ccbc_simplex_grad.argtypes = ([C.c_int] * 4 + [C.c_float] + [C.c_void_p] * 4 +
                                        [C.c_int, C.c_float, C.c_float, C.c_void_p])
        L.ccbc_simplex_flat_size_ex.argtypes = [C.c_int] * 7
        L.ccbc_simplex_flat_size_ex.restype = C.c_int64
        L.ccbc_simplex_forward_ex.argtypes = [C.c_int] * 8 + [C.c_float] + [C.c_void_p] * 7
        L.ccbc_simplex_grad_ex.argtypes = ([C.c_int] * 8 + [C.c_float] + [C.c_void_p] * 4 +
                                           [C.c_int, C.c_float, C.c_float, C.c_void_p])
        L.ccbc_forward_pretrain_model.argtypes = [C.c_int] * 5 + [C.c_void_p] * 13
        L.ccbc_learner_init_ex.argtypes = [C.c_void_p] + [C.c_int] * 8 + [C.c_float, C.c_void_p]
        L.ccbc_learner_new.argtypes = [C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_float,
                                       C.c_int64, C.c_float, C.c_float]
        L.ccbc_learner_free.argtypes = [C.c_void_p]
        L.ccbc_learner_init.argtypes = [C.c_void_p] + [C.c_int] * 4 + [C.c_float, C.c_void_p]
        L.ccbc_learner_record.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_float,
                                          C.c_void_p, C.c_void_p, C.c_void_p]
        L.ccbc_learner_outcome.argtypes = [C.c_void_p, C.c_void_p]
        L.ccbc_learner_weights.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.ccbc_learner_telemetry.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.ccbc_learner_history_size.argtypes = [C.c_void_p, C.c_int]
        L.ccbc_learner_history_size.restype = C.c_int64
        L.ccbc_learner_set_trace.argtypes = [C.c_void_p, C.c_char_p]
        L.ccbc_cswg_load.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_int64]
        L.ccbc_cswg_load.restype = C.c_int64
        L.ccbc_half_to_float.argtypes = [C.c_uint16]
        L.ccbc_half_to_float.restype = C.c_float
        L.ccbc_float_to_half.argtypes = [C.c_float]
        L.ccbc_float_to_half.restype = C.c_uint16
        L.ccbc_controller_main.argtypes = [C.c_char_p] * 5 + [C.c_void_p, C.c_void_p]
        L.ccbc_controller_main.restype = C.c_int64
        L.ccbc_cpu_features.argtypes = [C.c_void_p]
        L.ccbc_matvec.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3
        L.ccbc_diag_step.argtypes = [C.c_void_p] * 3 + [C.c_int] * 2
        L.ccbc_bf16_matmul.argtypes = [C.c_void_p] * 3 + [C.c_int] * 4
        _lib = L
    return _lib


def _err() -> str:
    return lib().ccbc_last_error().decode(errors="replace")


def check_wire_sizes() -> dict[int, int]:
    """Sizes compiled into the library; raises if they differ from the Python dtypes."""
    out = {}
    for kind, dt in WIRE_DTYPES.items():
        n = int(lib().ccbc_wire_sizeof(kind))
        if n != dt.itemsize or n != EXPECTED_SIZES[kind]:
            raise AssertionError(f"wire kind {kind}: native {n}, numpy {dt.itemsize}, expected {EXPECTED_SIZES[kind]}")
        out[kind] = n
    return out


class Ring:
    """SPSC ring of fixed-size records; process-local or POSIX-shm backed."""

    def __init__(self, dtype: np.dtype, capacity: int, *, shm_name: Optional[str] = None,
                 create: bool = True) -> None:
        self.dtype = np.dtype(dtype)
        self.capacity = int(capacity)
        self.shm_name = shm_name
        L = lib()
        if shm_name is None:
            h = L.ccbc_ring_create_local(self.dtype.itemsize, self.capacity)
        else:
            h = L.ccbc_ring_open_shm(shm_name.encode(), self.dtype.itemsize, self.capacity, int(create))
        if not h:
            raise ValueError(_err())
        self._h = h

    def push(self, record: np.ndarray) -> bool:
        rec = np.ascontiguousarray(record, dtype=self.dtype).reshape(1)
        return bool(lib().ccbc_ring_push(self._h, rec.ctypes.data))

    def pop(self) -> Optional[np.ndarray]:
        out = np.zeros(1, dtype=self.dtype)
        return out[0] if lib().ccbc_ring_pop(self._h, out.ctypes.data) else None

    def __len__(self) -> int:
        return int(lib().ccbc_ring_size(self._h))

    def close(self, unlink: bool = False) -> None:
        if self._h:
            lib().ccbc_ring_close(self._h)
            self._h = None
        if unlink and self.shm_name:
            lib().ccbc_shm_unlink(self.shm_name.encode())


class ShmBytes:
    """A named shared-memory byte region (exit flags, stats counters)."""

    def __init__(self, name: str, size: int = 0, create: bool = True) -> None:
        self.name = name
        h = lib().ccbc_shm_open(name.encode(), size, int(create))
        if not h:
            raise ValueError(_err())
        self._h = h
        n = int(lib().ccbc_shm_size(h))
        self.array = np.ctypeslib.as_array(C.cast(lib().ccbc_shm_ptr(h), C.POINTER(C.c_uint8)), shape=(n,))

    def close(self, unlink: bool = False) -> None:
        if self._h:
            self.array = None
            lib().ccbc_shm_close(self._h)
            self._h = None
        if unlink:
            lib().ccbc_shm_unlink(self.name.encode())


def recency_decay(reward: float, t: int, p: int, gamma: float) -> float:
    return float(lib().ccbc_recency_decay(reward, t, p, gamma))


def gerber_weight(then: float, now: float, threshold: float) -> float:
    return float(lib().ccbc_gerber_weight(then, now, threshold))


class RollingStddev:
    def __init__(self, decay: float = 0.99) -> None:
        self._h = lib().ccbc_rolling_new(decay)

    def update(self, x: float) -> None:
        lib().ccbc_rolling_update(self._h, x)

    def mean(self) -> float:
        return float(lib().ccbc_rolling_mean(self._h))

    def stddev(self) -> float:
        return float(lib().ccbc_rolling_std(self._h))

    def __del__(self):
        try:
            lib().ccbc_rolling_free(self._h)
        except Exception:
            pass


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class SimplexPolicy:
    """Dimension bundle + flat fp32 weights ``[W_vp | b_vp | W_lh | b_lh | W_sb | alpha]``."""

    def __init__(self, N: int = 16, K_v: int = 16, K_s: int = 4, H: int = 32, temperature: float = 1.0,
                 seed: int = 0) -> None:
        self.N, self.K_v, self.K_s, self.H, self.temperature = N, K_v, K_s, H, float(temperature)
        n = int(lib().ccbc_simplex_flat_size(K_v, K_s, H))
        rng = np.random.default_rng(seed)
        self.flat = (rng.standard_normal(n) * 0.1).astype(np.float32)

    def forward(self, V, E, feats):
        V, E, feats = _f32(V), _f32(E), _f32(feats)
        p = np.zeros(self.N, np.float32)
        logits = np.zeros(self.N, np.float32)
        rc = lib().ccbc_simplex_forward(self.N, self.K_v, self.K_s, self.H, self.temperature,
                                        self.flat.ctypes.data, V.ctypes.data, E.ctypes.data,
                                        feats.ctypes.data, p.ctypes.data, logits.ctypes.data)
        if rc:
            raise ValueError(_err())
        return p, logits

    def grad(self, V, E, feats, chosen: int, advantage: float, entropy_beta: float = 0.0) -> np.ndarray:
        V, E, feats = _f32(V), _f32(E), _f32(feats)
        g = np.zeros_like(self.flat)
        rc = lib().ccbc_simplex_grad(self.N, self.K_v, self.K_s, self.H, self.temperature,
                                     self.flat.ctypes.data, V.ctypes.data, E.ctypes.data,
                                     feats.ctypes.data, chosen, advantage, entropy_beta, g.ctypes.data)
        if rc:
            raise ValueError(_err())
        return g


class SimplexPolicyV3(SimplexPolicy):
    """The policy with its optional parts: ``K_e`` edge features per vertex pair, ``n_heads`` residual
    attention heads over the vertices (learned H x H query / key / value projections, per-head
    edge bias, averaged per-vertex logits scaled by ``lambda_hxh``) and a stored bucket-embedding
    table (simplex_policy.h:27-53 of the reference).  Flat layout: the base block, then
    ``[lambda | W_q | W_k | W_v | W_o | W_e]`` when ``n_heads > 0``, then ``bucket_embed``."""

    def __init__(self, N: int = 16, K_v: int = 16, K_e: int = 1, K_s: int = 4, H: int = 32, n_heads: int = 0,
                 n_buckets: int = 0, embed_dim: int = 0, temperature: float = 1.0, seed: int = 0) -> None:
        self.N, self.K_v, self.K_e, self.K_s, self.H = N, K_v, K_e, K_s, H
        self.n_heads, self.n_buckets, self.embed_dim = n_heads, n_buckets, embed_dim
        self.temperature = float(temperature)
        n = int(lib().ccbc_simplex_flat_size_ex(K_v, K_e, K_s, H, n_heads, n_buckets, embed_dim))
        self.flat = (np.random.default_rng(seed).standard_normal(n) * 0.1).astype(np.float32)

    def _dims(self):
        return (self.N, self.K_v, self.K_e, self.K_s, self.H, self.n_heads, self.n_buckets, self.embed_dim)

    def forward(self, V, E, feats, with_branch: bool = False):
        V, E, feats = _f32(V), _f32(E), _f32(feats)
        p, logits, hxh = (np.zeros(self.N, np.float32) for _ in range(3))
        rc = lib().ccbc_simplex_forward_ex(*self._dims(), self.temperature, self.flat.ctypes.data, V.ctypes.data,
                                           E.ctypes.data, feats.ctypes.data, p.ctypes.data, logits.ctypes.data,
                                           hxh.ctypes.data)
        if rc:
            raise ValueError(_err())
        return (p, logits, hxh) if with_branch else (p, logits)

    def grad(self, V, E, feats, chosen: int, advantage: float, entropy_beta: float = 0.0) -> np.ndarray:
        V, E, feats = _f32(V), _f32(E), _f32(feats)
        g = np.zeros_like(self.flat)
        rc = lib().ccbc_simplex_grad_ex(*self._dims(), self.temperature, self.flat.ctypes.data, V.ctypes.data,
                                        E.ctypes.data, feats.ctypes.data, chosen, advantage, entropy_beta,
                                        g.ctypes.data)
        if rc:
            raise ValueError(_err())
        return g


def forward_pretrain_model(features, weights: dict):
    """``(logits [B, D_slot], value [B])`` of the offline-pretrained controller trunk from features
    ``[B, F]`` and a weight dict with the reference's names (``trunk.in_proj.weight`` ... ``value_head.bias``,
    cpu_ssm_controller.cpp:309-355)."""
    x = _f32(features)
    w = {k: _f32(v) for k, v in weights.items()}
    Dg, F = w["trunk.in_proj.weight"].shape
    L = w["trunk.decay"].shape[0]
    Ds = w["policy_head.weight"].shape[0]
    if x.ndim != 2 or x.shape[1] != F:
        raise ValueError(f"features must be [B, {F}], got {x.shape}")
    for name, shape in (("trunk.in_proj.bias", (Dg,)), ("trunk.decay", (L, Dg)), ("trunk.w_in", (L, Dg, Dg)),
                        ("trunk.w_out", (L, Dg, Dg)), ("trunk.bias", (L, Dg)), ("policy_head.weight", (Ds, Dg)),
                        ("policy_head.bias", (Ds,)), ("value_head.weight", (1, Dg)), ("value_head.bias", (1,))):
        if tuple(w[name].shape) != shape:
            raise ValueError(f"{name} must have shape {shape}, got {tuple(w[name].shape)}")
    B = x.shape[0]
    logits = np.zeros((B, Ds), np.float32)
    value = np.zeros(B, np.float32)
    rc = lib().ccbc_forward_pretrain_model(
        B, F, Dg, L, Ds, x.ctypes.data, w["trunk.in_proj.weight"].ctypes.data, w["trunk.in_proj.bias"].ctypes.data,
        w["trunk.decay"].ctypes.data, w["trunk.w_in"].ctypes.data, w["trunk.w_out"].ctypes.data,
        w["trunk.bias"].ctypes.data, w["policy_head.weight"].ctypes.data, w["policy_head.bias"].ctypes.data,
        w["value_head.weight"].ctypes.data, w["value_head.bias"].ctypes.data, logits.ctypes.data, value.ctypes.data)
    if rc:
        raise ValueError(_err())
    return logits, value


class SimplexOnlineLearner:
    TELEMETRY_INT = ("replay_outcomes", "history_appends", "credited_actions", "gerber_accepted",
                     "gerber_rejected", "skipped_missing_state", "invalid_slot_skips", "sgd_steps",
                     "ema_blends")
    TELEMETRY_FLOAT = ("last_advantage_raw", "last_advantage_standardized", "last_gerber_weight",
                       "last_entropy", "last_grad_l2")

    def __init__(self, num_slots=4096, max_entries_per_slot=64, gamma=0.995, learning_rate=1e-3,
                 sgd_interval=256, ema_alpha=0.25, ema_interval=64, gerber_c=0.5, entropy_beta=0.0):
        self._h = lib().ccbc_learner_new(num_slots, max_entries_per_slot, gamma, learning_rate,
                                         sgd_interval, ema_alpha, ema_interval, gerber_c, entropy_beta)
        self._policy: Optional[SimplexPolicy] = None

    @property
    def handle(self):
        return self._h

    def initialize(self, policy: SimplexPolicy) -> None:
        rc = lib().ccbc_learner_init(self._h, policy.N, policy.K_v, policy.K_s, policy.H,
                                     policy.temperature, policy.flat.ctypes.data)
        if rc:
            raise ValueError(_err())
        self._policy = policy

    def record_decision(self, slot_id: int, gpu_step: int, chosen: int, p_chosen: float, V, E, feats):
        V, E, feats = _f32(V), _f32(E), _f32(feats)
        rc = lib().ccbc_learner_record(self._h, slot_id, gpu_step, chosen, p_chosen, V.ctypes.data,
                                       E.ctypes.data, feats.ctypes.data)
        if rc:
            raise ValueError(_err())

    def on_replay_outcome(self, ev: np.ndarray) -> None:
        rec = np.ascontiguousarray(ev, dtype=REPLAY_OUTCOME).reshape(1)
        lib().ccbc_learner_outcome(self._h, rec.ctypes.data)

    def weights(self, slow: bool = False) -> np.ndarray:
        out = np.zeros_like(self._policy.flat)
        if lib().ccbc_learner_weights(self._h, int(slow), out.ctypes.data):
            raise ValueError(_err())
        return out

    def telemetry(self) -> dict:
        a = np.zeros(9, np.uint64)
        b = np.zeros(5, np.float32)
        lib().ccbc_learner_telemetry(self._h, a.ctypes.data, b.ctypes.data)
        d = {k: int(v) for k, v in zip(self.TELEMETRY_INT, a)}
        d.update({k: float(v) for k, v in zip(self.TELEMETRY_FLOAT, b)})
        return d

    def history_size(self, slot: int) -> int:
        return int(lib().ccbc_learner_history_size(self._h, slot))

    def set_trace_path(self, path: str) -> None:
        lib().ccbc_learner_set_trace(self._h, path.encode())

    def close(self) -> None:
        if self._h:
            lib().ccbc_learner_free(self._h)
            self._h = None


def load_cswg(path: str):
    """Returns ``(header dict, fp32 payload)`` of a CSWG controller weight file."""
    hdr = np.zeros(6, np.uint32)
    n = int(lib().ccbc_cswg_load(str(path).encode(), hdr.ctypes.data, None, 0))
    if n < 0:
        raise ValueError(_err())
    payload = np.zeros(n, np.float32)
    lib().ccbc_cswg_load(str(path).encode(), hdr.ctypes.data, payload.ctypes.data, n)
    keys = ("version", "n_layers", "d_global", "d_slot", "feature_dim", "dtype")
    return dict(zip(keys, (int(v) for v in hdr))), payload


def write_cswg(path: str, payload: np.ndarray, *, n_layers: int, d_global: int, d_slot: int,
               feature_dim: int) -> None:
    with open(path, "wb") as f:
        f.write(b"CSWG")
        f.write(np.asarray([1, n_layers, d_global, d_slot, feature_dim, 1], "<u4").tobytes())
        f.write(np.asarray(payload, np.float16).astype("<f2").tobytes())


def cpu_features() -> dict:
    out = np.zeros(5, np.int32)
    lib().ccbc_cpu_features(out.ctypes.data)
    return dict(zip(("avx2", "avx512f", "amx_tile", "amx_bf16", "amx_enabled"), (bool(v) for v in out)))


def matvec(W, x, force_scalar: bool = False) -> np.ndarray:
    W, x = _f32(W), _f32(x)
    y = np.zeros(W.shape[0], np.float32)
    lib().ccbc_matvec(W.ctypes.data, x.ctypes.data, y.ctypes.data, W.shape[0], W.shape[1], int(force_scalar))
    return y


def diag_step(decay, x, h, force_scalar: bool = False) -> np.ndarray:
    decay, x = _f32(decay), _f32(x)
    h = _f32(h).copy()
    lib().ccbc_diag_step(decay.ctypes.data, x.ctypes.data, h.ctypes.data, h.size, int(force_scalar))
    return h


def bf16_matmul(A_bits: np.ndarray, B_bits: np.ndarray, force_scalar: bool = False):
    """``A`` / ``B`` as uint16 bf16 bit patterns; returns ``(C fp32, used_amx)``."""
    A = np.ascontiguousarray(A_bits, np.uint16)
    B = np.ascontiguousarray(B_bits, np.uint16)
    M, K = A.shape
    N = B.shape[1]
    Cm = np.zeros((M, N), np.float32)
    used = lib().ccbc_bf16_matmul(A.ctypes.data, B.ctypes.data, Cm.ctypes.data, M, N, K, int(force_scalar))
    return Cm, bool(used)


def run_controller(write_rings: Sequence[str], query_ring: str, replay_ring: str, exit_flag: str,
                   stats_shm: str = "", learner: Optional[SimplexOnlineLearner] = None) -> dict:
    """Blocking controller loop (run it in a thread or a child process)."""
    counts = np.zeros(3, np.uint64)
    total = lib().ccbc_controller_main("\n".join(write_rings).encode(), query_ring.encode(),
                                       replay_ring.encode(), exit_flag.encode(), stats_shm.encode(),
                                       learner.handle if learner else None, counts.ctypes.data)
    if total < 0:
        raise RuntimeError(_err())
    return {"total": int(total), "writes": int(counts[0]), "queries": int(counts[1]), "replays": int(counts[2])}


def controller_thread(*args, **kw) -> tuple[threading.Thread, dict]:
    box: dict = {}

    def _run():
        try:
            box["result"] = run_controller(*args, **kw)
        except Exception as exc:  # surfaced by the caller
            box["error"] = exc

    th = threading.Thread(target=_run, daemon=True)
    th.start()
    return th, box
