"""Diagonal-SSM controller that scores cache slots on the CPU: one global recurrent
state plus one state per slot, a linear read-out of both (contract of
src/chaoscontrol/episodic/cpu_ssm_controller.py:26-267).

    g' = decay_global * g + W_global_in f        s' = decay_slot * s + W_slot_in f
    logit = <g', w_global_out> + <s', w_slot_out> + bias

The native path runs the two mat-vecs and recurrences through the control-plane
library's AVX-512 kernels (``native/matops.cpp``); the PyTorch statement is the
fallback and the oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np
import torch

_FIELDS = ("w_global_in", "w_slot_in", "decay_global", "decay_slot", "w_global_out", "w_slot_out", "bias")

__all__ = ["CpuSsmControllerWeights", "CpuSsmControllerState", "CpuSsmControllerStep",
           "CpuSsmControllerDecision", "CpuSsmControllerRuntime", "cpp_available", "require_cpp", "forward_step"]


def _native():
    try:
        from . import native
        native.lib()
        return native
    except Exception:
        return None


def cpp_available() -> bool:
    return _native() is not None


def require_cpp() -> None:
    if _native() is None:  # pragma: no cover - depends on the local build
        raise ImportError("the C++ control-plane library is not built; run the in-tree build first")


def _cpu_f32(t: Any, *, expected_shape: tuple[int, ...]) -> torch.Tensor:
    out = torch.as_tensor(t, dtype=torch.float32, device="cpu").contiguous()
    if tuple(out.shape) != expected_shape:
        raise ValueError(f"expected shape {expected_shape}; got {tuple(out.shape)}")
    return out


@dataclass(frozen=True)
class CpuSsmControllerWeights:
    w_global_in: torch.Tensor       # [D_global, F]
    w_slot_in: torch.Tensor         # [D_slot, F]
    decay_global: torch.Tensor      # [D_global]
    decay_slot: torch.Tensor        # [D_slot]
    w_global_out: torch.Tensor      # [D_global]
    w_slot_out: torch.Tensor        # [D_slot]
    bias: torch.Tensor              # scalar

    def __post_init__(self) -> None:
        if self.w_global_in.dim() != 2:
            raise ValueError("w_global_in must be [D_global, F]")
        if self.w_slot_in.dim() != 2:
            raise ValueError("w_slot_in must be [D_slot, F]")
        if self.w_slot_in.shape[1] != self.w_global_in.shape[1]:
            raise ValueError("w_global_in and w_slot_in must share feature dim")
        want = {"decay_global": (self.global_dim,), "decay_slot": (self.slot_dim,),
                "w_global_out": (self.global_dim,), "w_slot_out": (self.slot_dim,), "bias": ()}
        for name, shape in want.items():
            if tuple(getattr(self, name).shape) != shape:
                raise ValueError(f"{name} must have shape {shape}; got {tuple(getattr(self, name).shape)}")

    @property
    def feature_dim(self) -> int:
        return int(self.w_global_in.shape[1])

    @property
    def global_dim(self) -> int:
        return int(self.w_global_in.shape[0])

    @property
    def slot_dim(self) -> int:
        return int(self.w_slot_in.shape[0])

    def to_dict(self) -> dict[str, torch.Tensor]:
        out = {k: getattr(self, k).detach().to("cpu", torch.float32).contiguous() for k in _FIELDS}
        out["bias"] = out["bias"].reshape(())
        return out

    @classmethod
    def from_dict(cls, blob: dict[str, Any]) -> "CpuSsmControllerWeights":
        missing = [k for k in _FIELDS if k not in blob]
        if missing:
            raise KeyError(f"missing CPU SSM controller weight field(s): {missing}")
        return cls(**{k: torch.as_tensor(blob[k], dtype=torch.float32, device="cpu").contiguous() for k in _FIELDS})

    def save(self, path: Path | str) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        torch.save(self.to_dict(), path)

    @classmethod
    def load(cls, path: Path | str) -> "CpuSsmControllerWeights":
        return cls.from_dict(torch.load(path, map_location="cpu", weights_only=False))


@dataclass(frozen=True)
class CpuSsmControllerState:
    global_state: torch.Tensor
    slot_state: torch.Tensor


@dataclass(frozen=True)
class CpuSsmControllerStep:
    global_state: torch.Tensor
    slot_state: torch.Tensor
    logit: torch.Tensor


@dataclass(frozen=True)
class CpuSsmControllerDecision:
    """What delayed replay credit needs from decision time: the features and the states BEFORE the step."""
    features: torch.Tensor
    global_state: torch.Tensor
    slot_state: torch.Tensor
    logit: torch.Tensor


def forward_step(features: torch.Tensor, state: CpuSsmControllerState, weights: CpuSsmControllerWeights, *,
                 prefer_cpp: bool = True) -> CpuSsmControllerStep:
    f = _cpu_f32(features, expected_shape=(weights.feature_dim,))
    g = _cpu_f32(state.global_state, expected_shape=(weights.global_dim,))
    s = _cpu_f32(state.slot_state, expected_shape=(weights.slot_dim,))
    w = weights.to_dict()
    if prefer_cpp and _native() is not None:
        from .arm_native import ssm_forward_step
        out_g, out_s, logit = ssm_forward_step(weights, f, g, s)      # one native call: both mat-vecs, both recurrences
        return CpuSsmControllerStep(out_g, out_s, logit.reshape(()))
    out_g = w["decay_global"] * g + torch.mv(w["w_global_in"], f)
    out_s = w["decay_slot"] * s + torch.mv(w["w_slot_in"], f)
    logit = out_g.dot(w["w_global_out"]) + out_s.dot(w["w_slot_out"]) + w["bias"]
    return CpuSsmControllerStep(out_g.contiguous(), out_s.contiguous(), logit.reshape(()))


class CpuSsmControllerRuntime:
    """Owns the global state and ``capacity`` per-slot states for online scoring."""

    def __init__(self, weights: CpuSsmControllerWeights, *, capacity: int, prefer_cpp: bool = True) -> None:
        if capacity <= 0:
            raise ValueError(f"capacity must be positive; got {capacity}")
        self.weights, self.prefer_cpp = weights, bool(prefer_cpp)
        self.global_state = torch.zeros(weights.global_dim, dtype=torch.float32)
        self.slot_state = torch.zeros(int(capacity), weights.slot_dim, dtype=torch.float32)

    def score_slot_with_snapshot(self, features: torch.Tensor, *, slot: int) -> CpuSsmControllerDecision:
        slot = int(slot)
        if not 0 <= slot < self.slot_state.shape[0]:
            raise IndexError(f"slot {slot} out of range")
        f = _cpu_f32(features, expected_shape=(self.weights.feature_dim,))
        before = CpuSsmControllerState(self.global_state.clone(), self.slot_state[slot].clone())
        out = forward_step(f, before, self.weights, prefer_cpp=self.prefer_cpp)
        self.global_state.copy_(out.global_state)
        self.slot_state[slot].copy_(out.slot_state)
        return CpuSsmControllerDecision(f.clone(), before.global_state, before.slot_state, out.logit)

    def score_slot(self, features: torch.Tensor, *, slot: int) -> torch.Tensor:
        return self.score_slot_with_snapshot(features, slot=slot).logit
