"""Recurrent-state persistence across chunks / documents, trainable initial
states, the delta / log_a modulation context and the adapt-set selector
(cf. src/chaoscontrol/eval_stream/persistence.py, delta_mod.py, ttt_runner.py)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..models.core import CareSSMCore

PERSISTENCE_MODES = ("reset", "carry_state", "carry_weights", "carry_both", "trainable_h0",
                     "trainable_h0+carry")

ADAPT_SET_PATTERNS: dict[str, list[str]] = {
    "none": [],
    "log_a": ["substr:log_a"],
    "delta_proj": ["substr:delta_proj"],
    "log_a+delta_proj": ["substr:log_a", "substr:delta_proj"],
    "B_side": ["substr:in_proj", "substr:select_proj"],
    "C_side": ["substr:out_proj", "substr:gate_proj"],
    "embed_rows_seen": ["exact:embed.weight"],
    "lm_head": ["substr:lm_head"],
    "lora_r8": ["substr:lora_"],
    "trainable_h0": ["substr:_trainable_h0"],
    "all": ["*"],
}


def _matches(name: str, patterns: list[str]) -> bool:
    for pat in patterns:
        kind, _, body = pat.partition(":")
        if kind == "exact" and name == body:
            return True
        if kind == "substr" and body in name:
            return True
        if ":" not in pat and pat in name:
            return True
    return False


def select_adapt_params(module: nn.Module, *, adapt_set: str) -> list[nn.Parameter]:
    if adapt_set not in ADAPT_SET_PATTERNS:
        raise ValueError(f"unknown adapt_set: {adapt_set}")
    pats = ADAPT_SET_PATTERNS[adapt_set]
    if not pats:
        return []
    if pats == ["*"]:
        return list(module.parameters())
    out, seen = [], set()
    for name, p in module.named_parameters():
        if _matches(name, pats) and id(p) not in seen:
            out.append(p)
            seen.add(id(p))
    return out


class StateManager:
    """Per-block recurrence state across chunks and document boundaries."""

    def __init__(self, model: nn.Module, *, persistence_mode: str) -> None:
        if persistence_mode not in PERSISTENCE_MODES:
            raise ValueError(f"unknown persistence_mode: {persistence_mode}")
        self.model = model
        self.mode = persistence_mode
        self._cores = [m for m in model.modules() if isinstance(m, CareSSMCore)]
        self._state: list[torch.Tensor] = []
        self._doc_idx = -1

    def _zeros(self, batch_size: int) -> list[torch.Tensor]:
        ref = next(self.model.parameters())
        return [torch.zeros(batch_size, c.dim, device=ref.device, dtype=ref.dtype) for c in self._cores]

    def start_doc(self, *, doc_id: int, batch_size: int) -> None:
        self._doc_idx += 1
        if self.mode in ("reset", "carry_weights"):
            self._state = self._zeros(batch_size)
        elif self.mode in ("carry_state", "carry_both"):
            if not self._state:
                self._state = self._zeros(batch_size)
        elif self.mode == "trainable_h0" or (self.mode == "trainable_h0+carry" and self._doc_idx == 0):
            self._state = [c._trainable_h0.expand(batch_size, -1) for c in self._cores]

    def get_state(self) -> list[torch.Tensor]:
        return self._state

    def set_state(self, state: list[torch.Tensor]) -> None:
        self._state = state


def attach_trainable_h0(model: nn.Module) -> None:
    """Give every recurrence core a trainable initial state (evaluation only)."""
    for core in model.modules():
        if isinstance(core, CareSSMCore) and not hasattr(core, "_trainable_h0"):
            ref = next(core.parameters())
            core._trainable_h0 = nn.Parameter(torch.zeros(1, core.dim, device=ref.device, dtype=ref.dtype))


def detach_trainable_h0(model: nn.Module) -> None:
    for core in model.modules():
        if isinstance(core, CareSSMCore) and hasattr(core, "_trainable_h0"):
            del core._trainable_h0


class DeltaModulator:
    """Context manager: scale every core's delta projection output and / or shift
    ``log_a`` for the enclosed forwards; everything is restored on exit.  Shifting
    ``log_a`` while adapting ``log_a`` is refused (the exit would undo the updates)."""

    def __init__(self, module: nn.Module, *, delta_scale: float = 1.0, log_a_shift: float = 0.0,
                 adapt_set_hint: Optional[str] = None) -> None:
        self.module = module
        self.delta_scale = float(delta_scale)
        self.log_a_shift = float(log_a_shift)
        self._hint = adapt_set_hint
        self._handles: list = []
        self._saved: list[tuple[nn.Parameter, torch.Tensor]] = []

    def __enter__(self):
        if self.log_a_shift != 0.0 and self._hint in ("log_a", "log_a+delta_proj", "all"):
            raise ValueError("DeltaModulator.log_a_shift is incompatible with adapting log_a "
                             "(log_a_shift reverts log_a on exit).")
        for core in (m for m in self.module.modules() if isinstance(m, CareSSMCore)):
            if self.delta_scale != 1.0:
                self._handles.append(core.delta_proj.register_forward_hook(
                    lambda _m, _i, out, s=self.delta_scale: out * s))
            if self.log_a_shift != 0.0 and hasattr(core, "log_a"):
                self._saved.append((core.log_a, core.log_a.detach().clone()))
                with torch.no_grad():
                    core.log_a.add_(self.log_a_shift)
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles.clear()
        with torch.no_grad():
            for p, orig in self._saved:
                p.copy_(orig)
        self._saved.clear()
