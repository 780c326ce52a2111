"""Core modules of the diagonal-SSM trunk: RMSNorm, FeedForward, the recurrence
core (diag / paired / full transition modes) and the recurrence backends.

Parameter names and math follow the reference so its checkpoints load with
``strict=True`` (src/chaoscontrol/core.py:316-357 for RMSNorm / FeedForward /
LowRankDeltaProjection, core.py:360-799 for the core).  Differences by design:

* there is one recurrence implementation per device (the native scan on CUDA,
  the chunked fp64 form on CPU) instead of an environment-selected backend;
* a non-zero ``initial_state`` stays on the parallel scan path: the kernels
  take ``h0`` natively, where the reference drops to a per-token Python loop
  (core.py:689-728).
"""
from __future__ import annotations

import math
from contextlib import contextmanager
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.scan import diag_recurrence_chunked, diag_recurrence_reference, ssm_scan

_DEFAULT_CHUNK_SIZE = 32


def get_diag_recurrence_backend(device: Optional[torch.device] = None) -> str:
    """Name of the recurrence implementation used for tensors on ``device``."""
    if device is not None and torch.device(device).type == "cuda":
        return "ssm_scan"
    return "chunked"


def verify_diag_recurrence(device: torch.device | str = "cpu") -> dict[str, Any]:
    """Run the active backend on a tiny problem and compare with the serial loop."""
    dev = torch.device(device)
    g = torch.Generator().manual_seed(0)
    decay = torch.rand(2, 17, 8, generator=g).to(dev)
    update = torch.randn(2, 17, 8, generator=g).to(dev)
    got = _diag_recurrence(decay, update)
    ref = diag_recurrence_reference(decay, update)
    err = float((got.float() - ref).abs().max())
    if err > 1e-4:
        raise RuntimeError(f"diag recurrence backend mismatch on {dev}: max err {err}")
    return {"backend": get_diag_recurrence_backend(dev), "max_err": err}


def _diag_recurrence(decay: torch.Tensor, update: torch.Tensor,
                     initial_state: Optional[torch.Tensor] = None) -> torch.Tensor:
    if update.is_cuda:
        return ssm_scan(decay.contiguous(), update.contiguous(), initial_state)
    return diag_recurrence_chunked(decay, update, _DEFAULT_CHUNK_SIZE, initial_state).to(update.dtype)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.float32))
        self.eps = eps

    #: set by the block-scaled fp8 promotion: the norm also emits the e4m3 copy its consumers read
    emit_fp8_blocks = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.emit_fp8_blocks and x.is_cuda and x.dtype == torch.bfloat16 and x.size(-1) % 128 == 0:
            from ..ops.fp8_block import rmsnorm_quant
            return rmsnorm_quant(x, self.weight, self.eps)
        normed = F.rms_norm(x.float(), (x.size(-1),), eps=self.eps)
        return normed.to(x.dtype) * self.weight


class FeedForward(nn.Module):
    def __init__(self, dim: int, mult: int) -> None:
        super().__init__()
        hidden = dim * mult
        self.fc = nn.Linear(dim, hidden, bias=False)
        self.proj = nn.Linear(hidden, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(F.silu(self.fc(x)))


class LowRankDeltaProjection(nn.Module):
    """``up(down(x))``: the D x D timescale projection factored to rank ``r``."""

    def __init__(self, dim: int, rank: int) -> None:
        super().__init__()
        if rank <= 0:
            raise ValueError(f"rank must be positive, got {rank}")
        self.dim = int(dim)
        self.rank = int(rank)
        self.down = nn.Linear(dim, rank, bias=False)
        self.up = nn.Linear(rank, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.up(self.down(x))


def _is_zero_state(state: torch.Tensor) -> bool:
    return (not state.requires_grad) and bool((state == 0).all())


class CareSSMCore(nn.Module):
    """Recurrence core.  ``diag`` is the production mode; ``paired`` (2x2
    rotation blocks) and ``full`` (matrix exponential of skew + low-rank A) are
    diagnostics that run as plain PyTorch loops."""

    def __init__(self, dim: int, *, a_mode: str = "diag", a_full_rank: int = 8,
                 a_full_gamma: float = 0.05, delta_rank: int = 0) -> None:
        super().__init__()
        self.dim = dim
        self.a_mode = a_mode
        self.a_full_rank = a_full_rank
        self.delta_rank = int(delta_rank)
        self._capture_states_enabled = False
        self._captured_states: Optional[torch.Tensor] = None

        self.in_proj = nn.Linear(dim, dim, bias=False)
        self.select_proj = nn.Linear(dim, dim, bias=False)
        self.gate_proj = nn.Linear(dim, dim, bias=False)
        self.out_proj = nn.Linear(dim, dim, bias=False)

        if a_mode == "diag":
            if 0 < self.delta_rank < dim:
                self.delta_proj: nn.Module = LowRankDeltaProjection(dim, self.delta_rank)
            else:
                self.delta_rank = 0
                self.delta_proj = nn.Linear(dim, dim, bias=False)
            self.log_a = nn.Parameter(torch.zeros((dim,), dtype=torch.float32))
        elif a_mode == "paired":
            if dim % 2:
                raise AssertionError(f"paired mode requires even dim, got {dim}")
            n_pairs = dim // 2
            self.delta_proj = nn.Linear(dim, dim, bias=False)
            self.log_r = nn.Parameter(torch.zeros((n_pairs,), dtype=torch.float32))
            self.theta = nn.Parameter(torch.linspace(0.0, math.pi, n_pairs, dtype=torch.float32))
        elif a_mode == "full":
            self.delta_proj = nn.Linear(dim, 1, bias=False)
            n_skew = dim * (dim - 1) // 2
            self.skew_params = nn.Parameter(torch.zeros((n_skew,), dtype=torch.float32))
            self.log_gamma = nn.Parameter(torch.full((), math.log(a_full_gamma), dtype=torch.float32))
            rank = min(a_full_rank, dim)
            self.U = nn.Parameter(torch.randn(dim, rank) * 0.01)
            self.V = nn.Parameter(torch.randn(dim, rank) * 0.01)
        else:
            raise ValueError(f"unsupported a_mode: {a_mode}")

    # -- helpers ---------------------------------------------------------
    def _content_terms(self, x: torch.Tensor):
        return (torch.sigmoid(self.select_proj(x)), torch.tanh(self.in_proj(x)),
                torch.sigmoid(self.gate_proj(x)))

    def _diag_terms(self, x: torch.Tensor):
        a_base = torch.sigmoid(self.log_a).to(dtype=x.dtype)[None, None, :]
        delta = F.softplus(self.delta_proj(x)).clamp_min(1e-4)
        decay = torch.exp(-delta * a_base)
        select, candidate, gate = self._content_terms(x)
        return decay, select * candidate, gate

    def _build_skew_symmetric(self) -> torch.Tensor:
        S = torch.zeros(self.dim, self.dim, dtype=self.skew_params.dtype,
                        device=self.skew_params.device)
        idx = torch.triu_indices(self.dim, self.dim, offset=1)
        S[idx[0], idx[1]] = self.skew_params
        return S - S.T

    def _get_A_full(self) -> torch.Tensor:
        S = self._build_skew_symmetric()
        gamma = torch.exp(self.log_gamma)
        return S - gamma * torch.eye(self.dim, device=S.device, dtype=S.dtype) + self.U @ self.V.T

    @contextmanager
    def capture_states(self):
        """Record the ``[B, T, D]`` state trajectory of enclosed diag forwards."""
        if self.a_mode != "diag":
            raise NotImplementedError(
                f"capture_states() is only implemented for a_mode='diag'; got a_mode={self.a_mode!r}.")
        self._capture_states_enabled = True
        self._captured_states = None
        try:
            yield lambda: self._captured_states
        finally:
            self._capture_states_enabled = False
            self._captured_states = None

    # -- single step -----------------------------------------------------
    def _update(self, inp, state, rich_b):
        if rich_b is not None:
            return rich_b(inp, state)
        return torch.sigmoid(self.select_proj(inp)) * torch.tanh(self.in_proj(inp))

    def step(self, inp: torch.Tensor, state: torch.Tensor, *, rich_b: Any = None):
        """One token: ``(batch, dim)`` input and state -> ``(output, new_state)``."""
        if self.a_mode == "diag":
            a_base = torch.sigmoid(self.log_a).to(dtype=inp.dtype)[None, :]
            delta = F.softplus(self.delta_proj(inp)).clamp_min(1e-4)
            new_state = torch.exp(-delta * a_base) * state + self._update(inp, state, rich_b)
        elif self.a_mode == "paired":
            batch, n_pairs = inp.shape[0], self.dim // 2
            delta = F.softplus(self.delta_proj(inp)).clamp_min(1e-4)
            r = torch.exp(-F.softplus(self.log_r)).to(dtype=inp.dtype)
            cos_t = torch.cos(self.theta).to(dtype=inp.dtype)
            sin_t = torch.sin(self.theta).to(dtype=inp.dtype)
            delta_pairs = (delta[:, 0::2] + delta[:, 1::2]) * 0.5
            eff = torch.exp(-delta_pairs * (1.0 - r[None, :]))
            s = state.view(batch, n_pairs, 2)
            s0, s1 = s[:, :, 0], s[:, :, 1]
            n0 = eff * (cos_t[None, :] * s0 - sin_t[None, :] * s1)
            n1 = eff * (sin_t[None, :] * s0 + cos_t[None, :] * s1)
            decayed = torch.stack([n0, n1], dim=-1).view(batch, self.dim)
            new_state = decayed + self._update(inp, state, rich_b)
        elif self.a_mode == "full":
            A_c = self._get_A_full().to(dtype=inp.dtype)
            delta = F.softplus(self.delta_proj(inp)).clamp(1e-4, 2.0)
            A_d = torch.matrix_exp(delta.mean() * A_c)
            new_state = state @ A_d.T + self._update(inp, state, rich_b)
        else:
            raise ValueError(f"unsupported a_mode: {self.a_mode}")
        out = torch.sigmoid(self.gate_proj(inp)) * new_state
        return self.out_proj(out), new_state

    # -- sequence --------------------------------------------------------
    def forward(self, x: torch.Tensor, *, rich_b: Any = None, return_jacobian_stats: bool = False,
                initial_state: Optional[torch.Tensor] = None, return_final_state: bool = False):
        """Run the recurrence over ``(batch, seq, dim)``.

        Returns ``y`` optionally followed by a Jacobian-stats dict and / or the
        final state, in the reference's order (core.py:622-799).
        """
        batch, seq, dim = x.shape

        def bundle(y, stats, final_state):
            if return_jacobian_stats and return_final_state:
                return y, stats, final_state
            if return_jacobian_stats:
                return y, stats
            if return_final_state:
                return y, final_state
            return y

        if self.a_mode == "diag" and rich_b is None:
            h0 = None
            if initial_state is not None and not _is_zero_state(initial_state):
                h0 = initial_state.to(device=x.device)
            decay, update, gate = self._diag_terms(x)
            states = _diag_recurrence(decay, update, h0)
            if self._capture_states_enabled:
                self._captured_states = states.detach()
            y = self.out_proj(gate * states)
            stats = ({"lambda_max": torch.tensor(0.0), "sv_log_var": torch.tensor(0.0)}
                     if return_jacobian_stats else None)
            return bundle(y, stats, states[:, -1] if return_final_state else None)

        state = (initial_state.to(dtype=x.dtype, device=x.device) if initial_state is not None
                 else x.new_zeros((batch, dim)))
        outputs = []
        lam, svv = [], []
        for idx in range(seq):
            out, state = self.step(x[:, idx, :], state, rich_b=rich_b)
            outputs.append(out)
            if return_jacobian_stats and self.a_mode == "full":
                with torch.no_grad():
                    A_c = self._get_A_full().float()
                    delta = F.softplus(self.delta_proj(x[:, idx, :])).clamp(1e-4, 2.0).mean().float()
                    sv = torch.linalg.svdvals(torch.matrix_exp(delta * A_c))
                    lam.append(torch.log(sv.max()))
                    svv.append(torch.log(sv).var())
        y = torch.stack(outputs, dim=1)
        stats = None
        if return_jacobian_stats:
            if lam:
                stats = {"lambda_max": torch.stack(lam).mean(), "sv_log_var": torch.stack(svv).mean()}
            else:
                stats = {"lambda_max": torch.tensor(0.0), "sv_log_var": torch.tensor(0.0)}
        return bundle(y, stats, state)


def criticality_loss(jacobian_stats: dict, *, alpha: float = 0.01, beta: float = 0.001,
                     target_log_sv: float = -0.13) -> torch.Tensor:
    """``alpha * (lambda_max - target)^2 + beta * Var(log sv)``: keep the
    transition slightly sub-critical (target log singular value ~ log 0.88);
    same contract as src/chaoscontrol/core.py:802-818."""
    lam = jacobian_stats["lambda_max"]
    sv_var = jacobian_stats["sv_log_var"]
    return alpha * (lam - target_log_sv).pow(2) + beta * sv_var
