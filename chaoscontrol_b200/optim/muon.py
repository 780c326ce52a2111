"""Muon with a decoupled-AdamW fallback for non-matrix parameters.

Same constructor, classification rule (2-D tensors except ``delta_proj``),
hyper-parameters and per-parameter state layout as the reference optimizer
(src/chaoscontrol/optim/muon.py:20-124, 390-660).  Three execution paths:

``arena``   parameters live in a :class:`~chaoscontrol_b200.utils.arena.ParamArena`:
            momentum / normalise / apply are single launches over flat ranges,
            each shape group's Newton-Schulz iteration is three batched
            tcgen05 GEMMs, AdamW is one launch per contiguous range.
``fused``   any parameter set: stack by shape, one batched NS per group (PyTorch).
``plain``   per-parameter loop (the oracle).
"""
from __future__ import annotations

from typing import Any, Callable, Iterable, Optional

import torch
from torch import Tensor

from ..ops import _lib
from ..ops.gemm import gemm

_NS_COEFFS = (3.4445, -4.7750, 2.0315)


def _ns_torch(X: Tensor, steps: int) -> Tensor:
    a, b, c = _NS_COEFFS
    for _ in range(steps):
        A = X @ X.mT
        X = a * X + (b * A + c * (A @ A)) @ X
    return X


def _ns_kernels(X: Tensor, steps: int) -> Tensor:
    """Newton-Schulz on a normalised bf16 batch ``[G, r, c]`` with the tcgen05 GEMM.

    Wide / square matrices iterate ``X <- aX + (bA + cA^2) X`` with ``A = X X^T``;
    tall ones use ``A = X^T X`` and ``X <- aX + X (bA + cA^2)`` so nothing is ever
    transposed in memory.
    """
    a, b, c = _NS_COEFFS
    G, r, cdim = X.shape
    tall = r > cdim
    k = cdim if tall else r
    A = torch.empty(G, k, k, dtype=torch.bfloat16, device=X.device)
    B = torch.empty_like(A)
    Y = torch.empty_like(X)
    for _ in range(steps):
        if tall:
            kblocks = (r + 63) // 64
            splits = 1
            if kblocks >= 64:
                splits = 16
                while kblocks % splits:
                    splits //= 2
            if splits > 1:
                part = gemm(X, X, a_mn=True, b_mn=True, splits=splits, out_dtype=torch.float32)
                A.copy_(part.sum(0))
            else:
                gemm(X, X, a_mn=True, b_mn=True, out=A)
        else:
            gemm(X, X, out=A)
        gemm(A, A, out=B, alpha=c, beta=b, cin=A)
        if tall:
            gemm(X, B, out=Y, alpha=1.0, beta=a, cin=X)
        else:
            gemm(B, X, b_mn=True, out=Y, alpha=1.0, beta=a, cin=X)
        X, Y = Y, X
    return X


def _kernel_ns_ok(X: Tensor) -> bool:
    return (X.is_cuda and X.dtype == torch.bfloat16 and _lib.available() and
            X.shape[-1] % 8 == 0 and X.shape[-2] % 8 == 0)


def newton_schulz_orthogonalize(grad: Tensor, steps: int = 5, eps: float = 1e-7,
                                compute_dtype: Optional[torch.dtype] = None) -> Tensor:
    """Quintic Newton-Schulz iteration pushing ``grad`` toward its orthogonal factor.

    2-D input or a batch; bf16 on CUDA, fp32 on CPU unless ``compute_dtype`` says
    otherwise.  On CUDA/bf16 the matmuls are the library's tcgen05 GEMMs.
    """
    if compute_dtype is None:
        compute_dtype = torch.bfloat16 if grad.is_cuda else torch.float32
    was_flat = grad.ndim == 2
    X = (grad.unsqueeze(0) if was_flat else grad).to(compute_dtype)
    lead = X.shape[:-2]
    X = X.reshape(-1, X.shape[-2], X.shape[-1])
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + eps)
    if _kernel_ns_ok(X):
        X = _ns_kernels(X.contiguous(), steps)
    else:
        tall = X.size(-2) > X.size(-1)
        if tall:
            X = X.mT
        X = _ns_torch(X, steps)
        if tall:
            X = X.mT
    X = X.reshape(*lead, X.shape[-2], X.shape[-1])
    return X.squeeze(0) if was_flat else X


def _default_is_matrix(param: Tensor, name: Optional[str]) -> bool:
    if name and (name.endswith(".delta_proj.weight") or ".delta_proj." in name):
        return False
    return param.ndim == 2


class Muon(torch.optim.Optimizer):
    def __init__(self, params: Iterable[Tensor] | Iterable[dict[str, Any]], lr: float = 0.02,
                 momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5,
                 weight_decay: float = 0.0, adamw_betas: tuple[float, float] = (0.9, 0.95),
                 adamw_eps: float = 1e-8, adamw_lr: Optional[float] = None,
                 adamw_weight_decay: Optional[float] = None,
                 matrix_param_names: Optional[set[str]] = None,
                 is_matrix: Optional[Callable[[Tensor, Optional[str]], bool]] = None,
                 fused: bool = False, compute_dtype: Optional[torch.dtype] = None,
                 log_a_beta_coupling: bool = False, log_a_beta_ema: float = 0.99,
                 log_a_beta_min: float = 0.5) -> None:
        if lr <= 0.0 or ns_steps <= 0 or not 0.0 <= momentum < 1.0:
            raise ValueError(f"invalid Muon hparams: lr={lr} momentum={momentum} ns_steps={ns_steps}")
        if not 0.0 <= float(log_a_beta_min) < 1.0:
            raise ValueError(f"log_a_beta_min must be in [0, 1), got {log_a_beta_min}")
        if not 0.0 <= float(log_a_beta_ema) < 1.0:
            raise ValueError(f"log_a_beta_ema must be in [0, 1), got {log_a_beta_ema}")
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        weight_decay=weight_decay, adamw_betas=adamw_betas, adamw_eps=adamw_eps,
                        adamw_lr=lr if adamw_lr is None else adamw_lr,
                        adamw_weight_decay=(weight_decay if adamw_weight_decay is None
                                            else adamw_weight_decay))
        super().__init__(params, defaults)
        # an empty set is a legitimate override: "nothing is a matrix"
        self._matrix_param_names = set(matrix_param_names) if matrix_param_names is not None else None
        self._is_matrix_fn = is_matrix if is_matrix is not None else _default_is_matrix
        self._fused = fused
        self._compute_dtype = compute_dtype
        self._param_name_by_id: dict[int, str] = {}
        self._plasticity_multiplier: Optional[Tensor] = None
        self._plasticity_multiplier_views: dict = {}
        self._plasticity_step = -1
        self._plasticity_strength = 0.0
        self._plasticity_updates = 0
        self._plasticity_last_dim = 0
        self._plasticity_last_budget: Optional[Tensor] = None
        self._plasticity_last_confidence: Optional[Tensor] = None
        self._log_a_beta_coupling = bool(log_a_beta_coupling)
        self._log_a_beta_ema = float(log_a_beta_ema)
        self._log_a_beta_min = float(log_a_beta_min)
        self._log_a_beta_updates = 0
        self._log_a_beta_last: Optional[Tensor] = None
        self._arena = None
        self._arena_state: dict[str, Any] = {}
        self.ns_calls = 0          # batched NS invocations (one per shape group when fused)

    # -- wiring ----------------------------------------------------------
    def bind_param_names(self, named_params: Iterable[tuple[str, Tensor]]) -> None:
        self._param_name_by_id = {id(p): n for n, p in named_params}

    def bind_arena(self, arena) -> None:
        """Use the flat-buffer kernel path for a model whose parameters live in ``arena``."""
        self._arena = arena
        self._param_name_by_id = {id(p): n for n, p in arena.params.items()}

    def set_arena_shard(self, shard: Optional[dict]) -> None:
        """Restrict the matrix (Muon) update to an owned sub-batch of every arena
        shape group: ``shard[group_index] = (first, end)``.  ``None`` restores the
        full update.  Non-matrix (AdamW) parameters are always updated: they are
        replicated.  Used by the distributed optimizer, which gathers the owned
        results afterwards.  Momentum buffers stay full-size so ``state_dict()``
        keeps its layout; only the owned slices are touched."""
        self._arena_shard = None if shard is None else {int(k): (int(v[0]), int(v[1])) for k, v in shard.items()}
        self._owned_ids = None
        if self._arena_shard is not None and self._arena is not None:
            owned = set()
            for gi, g in enumerate(self._arena.muon_groups):
                a, b = self._arena_shard.get(gi, (0, 0))
                owned.update(id(self._arena.params[n]) for n in g.names[a:b])
            self._owned_ids = owned

    def _owns(self, p: Tensor) -> bool:
        ids = getattr(self, "_owned_ids", None)
        return ids is None or id(p) in ids

    def _is_matrix_param(self, p: Tensor) -> bool:
        name = self._param_name_by_id.get(id(p))
        if self._matrix_param_names is not None and name is not None:
            return name in self._matrix_param_names
        return self._is_matrix_fn(p, name)

    # -- log_a beta coupling / plasticity (research knobs) ------------------
    def _uses_log_a_beta(self, p: Tensor) -> bool:
        if not self._log_a_beta_coupling:
            return False
        return p.ndim == 1 and self._param_name_by_id.get(id(p), "").endswith(".log_a")

    def _log_a_beta_for(self, p: Tensor, state: dict, beta1: float):
        if not self._uses_log_a_beta(p):
            return None
        ema = state.get("log_a_slow_ema")
        cur = p.detach().float()
        if ema is None:
            ema = cur.clone()
            state["log_a_slow_ema"] = ema
        else:
            ema.mul_(self._log_a_beta_ema).add_(cur, alpha=1.0 - self._log_a_beta_ema)
        floor = min(self._log_a_beta_min, float(beta1))
        beta_vec = (floor + (float(beta1) - floor) * torch.sigmoid(ema)).float()
        prod = state.get("log_a_beta1_prod")
        if prod is None:
            prod = beta_vec.clone()
            state["log_a_beta1_prod"] = prod
        else:
            prod.mul_(beta_vec)
        bias1 = (1.0 - prod).clamp_min(1e-12)
        self._log_a_beta_updates += 1
        self._log_a_beta_last = beta_vec.detach()
        return beta_vec.to(p.dtype), bias1.to(p.dtype)

    @torch.no_grad()
    def set_plasticity_budget(self, budget: Tensor, *, confidence: Optional[Tensor] = None,
                              strength: float = 0.25, step: Optional[int] = None) -> None:
        """Per-channel update multiplier ``1 + strength * budget`` for core parameters."""
        b = budget.detach().float().reshape(-1).clamp(0.0, 1.0)
        c = torch.ones_like(b) if confidence is None else confidence.detach().float().reshape(-1).clamp(0.0, 1.0)
        if c.numel() != b.numel():
            raise ValueError("plasticity confidence must match budget shape; got "
                             f"{tuple(c.shape)} vs {tuple(b.shape)}")
        self._plasticity_multiplier = 1.0 + float(strength) * b
        self._plasticity_multiplier_views.clear()
        self._plasticity_step = -1 if step is None else int(step)
        self._plasticity_strength = float(strength)
        self._plasticity_updates += 1
        self._plasticity_last_dim = int(b.numel())
        self._plasticity_last_budget = b
        self._plasticity_last_confidence = c

    def plasticity_budget_trace(self) -> dict:
        mult, budget, conf = (self._plasticity_multiplier, self._plasticity_last_budget,
                              self._plasticity_last_confidence)
        if mult is None or mult.numel() == 0:
            return {"enabled": False, "updates": self._plasticity_updates, "step": self._plasticity_step,
                    "dim": 0, "strength": self._plasticity_strength, "budget_mean": 0.0,
                    "budget_max": 0.0, "confidence_mean": 0.0, "lr_multiplier_min": 1.0,
                    "lr_multiplier_mean": 1.0, "lr_multiplier_max": 1.0,
                    "budget_nonzero_fraction": 0.0, "confidence_max": 0.0, "top_channels": [],
                    "top_budget": []}
        k = min(8, int(budget.numel()))
        vals, idx = torch.topk(budget, k=k)
        return {"enabled": True, "updates": self._plasticity_updates, "step": self._plasticity_step,
                "dim": self._plasticity_last_dim, "strength": self._plasticity_strength,
                "budget_mean": float(budget.mean()), "budget_max": float(budget.max()),
                "confidence_mean": float(conf.mean()), "confidence_max": float(conf.max()),
                "budget_nonzero_fraction": float((budget > 0).float().mean()),
                "lr_multiplier_min": float(mult.min()), "lr_multiplier_mean": float(mult.mean()),
                "lr_multiplier_max": float(mult.max()),
                "top_channels": [int(i) for i in idx.cpu()], "top_budget": [float(v) for v in vals.cpu()]}

    def ssm_role_trace(self) -> dict:
        beta = self._log_a_beta_last
        out = {"log_a_beta_coupling": self._log_a_beta_coupling,
               "log_a_beta_updates": self._log_a_beta_updates, "log_a_beta_ema": self._log_a_beta_ema,
               "log_a_beta_min_config": self._log_a_beta_min, "log_a_beta_min": 0.0,
               "log_a_beta_mean": 0.0, "log_a_beta_max": 0.0}
        if beta is not None and beta.numel():
            out.update(log_a_beta_min=float(beta.min()), log_a_beta_mean=float(beta.mean()),
                       log_a_beta_max=float(beta.max()))
        return out

    def _plasticity_multiplier_for(self, p: Tensor) -> Optional[Tensor]:
        mult = self._plasticity_multiplier
        if mult is None:
            return None
        name = self._param_name_by_id.get(id(p), "")
        if not name.startswith("layers.") or ".core." not in name:
            return None
        key = (p.device, p.dtype)
        m = self._plasticity_multiplier_views.get(key)
        if m is None:
            m = mult.to(device=p.device, dtype=p.dtype)
            self._plasticity_multiplier_views[key] = m
        d = m.numel()
        if p.ndim == 1 and p.numel() == d and name.endswith((".log_a", ".log_r", ".theta")):
            return m.reshape_as(p)
        if p.ndim != 2:
            return None
        if name.endswith((".in_proj.weight", ".select_proj.weight", ".gate_proj.weight",
                          ".delta_proj.weight", ".delta_proj.up.weight")) and p.shape[0] == d:
            return m.view(d, 1)
        if name.endswith((".delta_proj.down.weight", ".out_proj.weight")) and p.shape[1] == d:
            return m.view(1, d)
        return None

    # -- AdamW fallback ----------------------------------------------------
    def _adamw_update_param(self, *, p, state, grad, beta1, beta2, adamw_eps, adamw_lr, adamw_wd):
        if "step" not in state:
            state["step"] = 0
            state["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        state["step"] += 1
        t = state["step"]
        exp_avg, exp_avg_sq = state["exp_avg"], state["exp_avg_sq"]
        pair = self._log_a_beta_for(p, state, beta1)
        if pair is None:
            exp_avg.mul_(beta1).add_(grad, alpha=1.0 - beta1)
            bias1: Any = 1.0 - beta1 ** t
        else:
            beta_vec, bias1 = pair
            exp_avg.mul_(beta_vec).add_(grad * (1.0 - beta_vec))
        exp_avg_sq.mul_(beta2).addcmul_(grad, grad, value=1.0 - beta2)
        bias2 = 1.0 - beta2 ** t
        denom = (exp_avg_sq.sqrt() / (bias2 ** 0.5)).add_(adamw_eps)
        if adamw_wd > 0.0:
            p.data.mul_(1.0 - adamw_lr * adamw_wd)
        mult = self._plasticity_multiplier_for(p)
        if isinstance(bias1, Tensor):
            upd = exp_avg / denom / bias1
            p.data.add_(upd if mult is None else upd * mult, alpha=-adamw_lr)
        elif mult is None:
            p.data.addcdiv_(exp_avg, denom, value=-adamw_lr / bias1)
        else:
            p.data.add_((exp_avg / denom) * mult, alpha=-adamw_lr / bias1)

    # -- step ----------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure: Optional[Callable[[], Tensor]] = None) -> Optional[Tensor]:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        arena = self._arena
        if arena is not None and arena.flat_param.is_cuda and arena.still_valid():
            self._step_arena(arena)
        elif self._fused:
            self._step_fused()
        else:
            self._step_plain()
        return loss

    def _step_plain(self) -> None:
        for group in self.param_groups:
            lr, mu, nesterov = group["lr"], group["momentum"], group["nesterov"]
            wd = group["weight_decay"]
            beta1, beta2 = group["adamw_betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                grad, state = p.grad, self.state[p]
                if self._is_matrix_param(p):
                    if not self._owns(p):
                        continue
                    if "momentum_buffer" not in state:
                        state["momentum_buffer"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    buf = state["momentum_buffer"]
                    buf.mul_(mu).add_(grad)
                    direction = grad.add(buf, alpha=mu) if nesterov else buf
                    update = newton_schulz_orthogonalize(direction, steps=group["ns_steps"],
                                                         compute_dtype=self._compute_dtype)
                    self.ns_calls += 1
                    scale = max(1.0, p.shape[-2] / p.shape[-1]) ** 0.5
                    if wd > 0.0:
                        p.data.mul_(1.0 - lr * wd)
                    mult = self._plasticity_multiplier_for(p)
                    if mult is not None:
                        update = update * mult
                    p.data.add_(update.to(dtype=p.dtype), alpha=-lr * scale)
                else:
                    self._adamw_update_param(p=p, state=state, grad=grad, beta1=beta1, beta2=beta2,
                                             adamw_eps=group["adamw_eps"], adamw_lr=group["adamw_lr"],
                                             adamw_wd=group["adamw_weight_decay"])

    def _step_fused(self) -> None:
        """Stack matrix params by exact shape -> one batched NS per shape group; the
        rest goes through AdamW.  Per-parameter state entries are kept so
        ``state_dict()`` matches the plain path."""
        for group in self.param_groups:
            lr, mu, nesterov = group["lr"], group["momentum"], group["nesterov"]
            wd = group["weight_decay"]
            beta1, beta2 = group["adamw_betas"]
            by_shape: dict[tuple, list[Tensor]] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                if self._is_matrix_param(p):
                    if self._owns(p):
                        by_shape.setdefault((tuple(p.shape), p.dtype, p.device), []).append(p)
                else:
                    self._adamw_update_param(p=p, state=self.state[p], grad=p.grad, beta1=beta1,
                                             beta2=beta2, adamw_eps=group["adamw_eps"],
                                             adamw_lr=group["adamw_lr"],
                                             adamw_wd=group["adamw_weight_decay"])
            for (shape, _dt, _dev), ps in by_shape.items():
                dirs = []
                for p in ps:
                    st = self.state[p]
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(p, memory_format=torch.preserve_format)
                    buf = st["momentum_buffer"]
                    buf.mul_(mu).add_(p.grad)
                    dirs.append(p.grad.add(buf, alpha=mu) if nesterov else buf)
                upd = newton_schulz_orthogonalize(torch.stack(dirs, 0), steps=group["ns_steps"],
                                                  compute_dtype=self._compute_dtype)
                self.ns_calls += 1
                scale = max(1.0, shape[-2] / shape[-1]) ** 0.5
                for i, p in enumerate(ps):
                    if wd > 0.0:
                        p.data.mul_(1.0 - lr * wd)
                    u = upd[i]
                    mult = self._plasticity_multiplier_for(p)
                    if mult is not None:
                        u = u * mult
                    p.data.add_(u.to(dtype=p.dtype), alpha=-lr * scale)

    # -- flat-buffer kernel path ---------------------------------------------
    def _arena_buffers(self, arena):
        st = self._arena_state
        if not st:
            dev = arena.flat_param.device
            n = arena.flat_param.numel()
            st["momentum"] = torch.zeros(n, dtype=torch.float32, device=dev)
            st["exp_avg"] = torch.zeros(n, dtype=torch.float32, device=dev)
            st["exp_avg_sq"] = torch.zeros(n, dtype=torch.float32, device=dev)
            st["dir"] = torch.empty(n, dtype=torch.bfloat16, device=dev)
            st["sumsq"] = torch.zeros(max(g.count for g in arena.muon_groups), dtype=torch.float32,
                                      device=dev)
            st["step"] = 0
            # per-parameter views keep state_dict() layout compatible with the plain path
            for name, p in arena.params.items():
                off, _ = arena.slots[name]
                s = self.state[p]
                if self._is_matrix_param(p):
                    s["momentum_buffer"] = st["momentum"][off: off + p.numel()].view_as(p)
                else:
                    s["exp_avg"] = st["exp_avg"][off: off + p.numel()].view_as(p)
                    s["exp_avg_sq"] = st["exp_avg_sq"][off: off + p.numel()].view_as(p)
                    s["step"] = 0
        return st

    def _step_arena(self, arena) -> None:
        if self._plasticity_multiplier is not None or self._log_a_beta_coupling or len(self.param_groups) != 1:
            # research knobs are per-parameter features, and the flat path reads ONE set of
            # hyper-parameters: several param groups run on the general path too
            if not arena.grads_fresh:
                pass
            arena.materialize_grads()
            self._step_fused()
            return
        if not arena.grads_fresh:
            arena.pull_grads()
        st = self._arena_buffers(arena)
        group = self.param_groups[0]
        lr, mu, nesterov = group["lr"], group["momentum"], int(group["nesterov"])
        wd, steps = group["weight_decay"], group["ns_steps"]
        L = _lib.lib()
        stream = _lib.stream_ptr()
        p_bf16 = arena.flat_param.dtype == torch.bfloat16
        es = arena.flat_param.element_size()
        shard = getattr(self, "_arena_shard", None)
        for gi, g in enumerate(arena.muon_groups):
            r, c = g.shape
            per = r * c
            m0, m1 = (0, g.count) if shard is None else shard.get(gi, (0, 0))
            cnt = m1 - m0
            if cnt <= 0:
                continue
            off = g.offset + m0 * per          # first owned matrix of this group
            gptr = arena.flat_grad.data_ptr() + off * 4
            _lib.check(L.ccb_muon_momentum(gptr, st["momentum"].data_ptr() + off * 4,
                                           st["dir"].data_ptr() + off * 2, st["sumsq"].data_ptr(),
                                           cnt, per, mu, nesterov, stream), "muon_momentum")
            _lib.check(L.ccb_muon_normalize(st["dir"].data_ptr() + off * 2, st["sumsq"].data_ptr(),
                                            cnt, per, 1e-7, stream), "muon_normalize")
            X = st["dir"][off: off + cnt * per].view(cnt, r, c)
            O = _ns_kernels(X, steps)
            self.ns_calls += 1
            scale = max(1.0, r / c) ** 0.5
            # apply over maximal runs of non-skipped matrices (indices relative to m0)
            i = 0
            while i < cnt:
                if (m0 + i) in g.skip:
                    i += 1
                    continue
                j = i
                while j < cnt and (m0 + j) not in g.skip:
                    j += 1
                n = (j - i) * per
                if p_bf16:
                    _lib.check(L.ccb_muon_apply(arena.flat_param.data_ptr() + (off + i * per) * es,
                                                O.data_ptr() + i * per * 2, n, lr * scale,
                                                1.0 - lr * wd, stream), "muon_apply")
                else:
                    pv = arena.flat_param[off + i * per: off + j * per]
                    pv.mul_(1.0 - lr * wd).add_(O.reshape(-1)[i * per: j * per].float(), alpha=-lr * scale)
                i = j
        # AdamW ranges
        st["step"] += 1
        t = st["step"]
        beta1, beta2 = group["adamw_betas"]
        for (a0, a1) in arena.adamw_ranges:
            _lib.check(L.ccb_adamw(arena.flat_param.data_ptr() + a0 * es, int(p_bf16),
                                   arena.flat_grad.data_ptr() + a0 * 4,
                                   st["exp_avg"].data_ptr() + a0 * 4,
                                   st["exp_avg_sq"].data_ptr() + a0 * 4, a1 - a0, group["adamw_lr"],
                                   beta1, beta2, group["adamw_eps"], group["adamw_weight_decay"],
                                   1.0 - beta1 ** t, (1.0 - beta2 ** t) ** 0.5, None, stream), "adamw")
        for name, p in arena.params.items():
            if not self._is_matrix_param(p):
                self.state[p]["step"] = t
        arena.grads_fresh = False
