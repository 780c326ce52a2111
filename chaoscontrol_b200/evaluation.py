"""Windowed evaluation of the research models: bits per byte with optional
warm-up of the runtime memory and an optional metabolic-gate pass, warming
curves under the test-time-training reset protocol, and the buffer x causal-SLOT
2x2 factorial (public surface of src/chaoscontrol/evaluation.py:30-766).

Reset protocol: between segments every piece of runtime state (episodic slots,
single-slot outer state, prototypes, semantic bases, posterior corrections) is
cleared, so a measurement reflects how fast the model rebuilds context, never
residue of an earlier segment.

Warm-up that must not leak out of an evaluation runs against a snapshot of the
outer model (a deep copy of its state dict plus its trigger attributes) that is
restored in a ``finally`` block.  CE sums are accumulated on the device and read
once.
"""
from __future__ import annotations

import copy
import math
import random
from typing import Any, Optional

import torch
import torch.nn.functional as F

from .data import batch_from_starts, maybe_autocast
from .metabolic import StructuredProjections, metabolic_fork, metabolic_monte_carlo, micro_mcts  # noqa: F401
from .models.memory import MultiSlotOuterModel
from .scoring import compute_bpb

__all__ = ["compute_bpb", "evaluate_chaoscontrol_bpb", "evaluate_warming_curve", "causal_slot_eval",
           "WARMING_CURVE_STEPS"]

WARMING_CURVE_STEPS = [0, 100, 500, 1000, 5000]
_OM_ATTRS = ("_spike_seen", "_steps_since_spike", "_pre_spike_loss", "_retrieval_weights", "_retrieval_indices")


# ---------------------------------------------------------------------------
# outer-model snapshot
# ---------------------------------------------------------------------------
def _snapshot_outer(om) -> dict[str, Any]:
    snap = {"sd": copy.deepcopy(om.state_dict()), "attrs": {a: getattr(om, a) for a in _OM_ATTRS if hasattr(om, a)}}
    if hasattr(om, "_compress_rng"):
        snap["rng"] = om._compress_rng.getstate()
    if hasattr(om, "_compression_consequences"):
        snap["cc"] = list(om._compression_consequences)
    if hasattr(om, "_bucket_affinity"):
        snap["aff"] = None if om._bucket_affinity is None else om._bucket_affinity.clone()
    return snap


def _restore_outer(om, snap: dict[str, Any]) -> None:
    # buffers that consolidation replaces (rather than updates in place) must be re-seated first
    for name, val in snap["sd"].items():
        if torch.is_tensor(val) and "." not in name and hasattr(om, name) and getattr(om, name).shape != val.shape:
            setattr(om, name, val.clone())
    om.load_state_dict(snap["sd"])
    for a, v in snap["attrs"].items():
        setattr(om, a, v)
    if "rng" in snap:
        om._compress_rng.setstate(snap["rng"])
    if "cc" in snap:
        om._compression_consequences = snap["cc"]
    if "aff" in snap:
        om._bucket_affinity = snap["aff"]


def _clear_outer(om) -> None:
    if isinstance(om, MultiSlotOuterModel):
        om._slots = []
        om._survival = []
        om._slot_buckets = []
        om._slot_event_ids = []
        om._latent_traces = []
        om._retrieval_weights = None
        om._compression_consequences.clear()
    elif hasattr(om, "state"):
        om.state.zero_()


def _warm_outer(model, out, batch_loss: float, write_mode: str, latent: bool) -> None:
    om = model.outer_model
    if write_mode == "full_sequence" and hasattr(om, "write_sequence"):
        avg = om.loss_ema.item()
        sig = om.compute_consolidation_signal(batch_loss, avg)
        if avg > 0 and sig / avg > 0.01:
            om.write_sequence(out["hidden"].detach(), bucket_id=None)
        om.update_survival(batch_loss)
        om.loss_ema = om.ema_decay * om.loss_ema + (1 - om.ema_decay) * batch_loss
    else:
        om.consolidation_step(out["hidden"][:, -1, :].detach(), current_loss=batch_loss, bucket_id=None)
    if latent and hasattr(om, "try_reactivate"):
        ratio = batch_loss / max(om.loss_ema.item(), 1e-6)
        if ratio > 1.0:
            om.try_reactivate(bucket_id=None, surprise=ratio)


# ---------------------------------------------------------------------------
# bpb
# ---------------------------------------------------------------------------
def evaluate_chaoscontrol_bpb(model: Any, *, tokens: torch.Tensor, eval_starts: list[int], batch_size: int, seq_len: int,
                              device: torch.device, metabolic_gate: bool = False, metabolic_k: int = 4,
                              metabolic_score: str = "memory_consistency", metabolic_noise_std: float = 0.01,
                              metabolic_mode: str = "fork", generation_mode: str = "noise", structured_proj: Any = None,
                              warmup: bool = False, warmup_write_mode: str = "last", warmup_latent: bool = False,
                              warmup_cold_start: bool = False, total_raw_bytes: Optional[int] = None,
                              tokenizer: Any = None, prior_bias: Any = None) -> dict[str, float]:
    """``{"loss", "bpb", "tokens"[, "bpb_raw", "loss_gated", "bpb_gated"]}``.

    ``warmup`` lets the outer model consolidate during the evaluation (its state is put
    back afterwards; ``warmup_cold_start`` empties it first).  With ``metabolic_gate`` a
    second, gate-aware pass is scored next to the plain one.  With a learned
    ``tokenizer`` the byte count is the raw input bytes and the reconstruction loss is
    charged to the total."""
    was_training = model.training
    model.eval()
    V = model.vocab_size
    om = getattr(model, "outer_model", None)
    warm = warmup and om is not None
    snap = _snapshot_outer(om) if warm else None
    if warm and warmup_cold_start:
        _clear_outer(om)
    ce = torch.zeros((), dtype=torch.float64, device=device)
    ce_gated = torch.zeros((), dtype=torch.float64, device=device)
    n_tok = raw_seen = 0
    try:
        with torch.no_grad():
            for i in range(0, len(eval_starts), batch_size):
                inputs, targets = batch_from_starts(tokens, eval_starts[i:i + batch_size], seq_len, device)
                extra = 0.0
                if tokenizer is not None:
                    raw = int(inputs.numel())
                    tok = tokenizer(inputs)
                    extra = float(tok["recon_loss"]) * raw
                    inputs, targets = tok["token_ids"][:, :-1], tok["token_ids"][:, 1:]
                    raw_seen += raw
                dt = next(model.parameters()).dtype if device.type == "cuda" else torch.float32
                with maybe_autocast(device, dt):
                    out = model(inputs)
                    flat_t = targets.reshape(-1)
                    batch_sum = F.cross_entropy(out["logits"].float().reshape(-1, V), flat_t, reduction="sum")
                    if warm:
                        _warm_outer(model, out, float(batch_sum) / max(flat_t.numel(), 1), warmup_write_mode,
                                    warmup_latent)
                    if metabolic_gate:
                        if metabolic_mode == "mcts":
                            g = micro_mcts(model, inputs, n_rollouts=metabolic_k, horizon=8, prior_bias=prior_bias)
                        elif metabolic_mode == "monte_carlo":
                            g = metabolic_monte_carlo(model, inputs, k=metabolic_k, noise_std=metabolic_noise_std,
                                                      generation_mode=generation_mode, structured_proj=structured_proj)
                        else:
                            g = metabolic_fork(model, inputs, k=metabolic_k, noise_std=metabolic_noise_std,
                                               score_mode=metabolic_score, generation_mode=generation_mode,
                                               structured_proj=structured_proj, prior_bias=prior_bias)
                        ce_gated += F.cross_entropy(g["logits"].float().reshape(-1, V), flat_t, reduction="sum").double() + extra
                ce += batch_sum.double() + extra
                n_tok += int(flat_t.numel())
    finally:
        if snap is not None:
            _restore_outer(om, snap)
        if was_training:
            model.train()
    total = float(ce)
    mean = total / max(n_tok, 1)
    res = {"loss": mean, "bpb": compute_bpb(total, raw_seen) if tokenizer is not None and raw_seen > 0
           else mean / math.log(2.0), "tokens": float(n_tok)}
    if total_raw_bytes is not None:
        res["bpb_raw"] = compute_bpb(total, total_raw_bytes)
    if metabolic_gate:
        tg = float(ce_gated)
        res["loss_gated"] = tg / max(n_tok, 1)
        res["bpb_gated"] = compute_bpb(tg, raw_seen) if raw_seen > 0 else res["loss_gated"] / math.log(2.0)
    return res


# ---------------------------------------------------------------------------
# reset protocol
# ---------------------------------------------------------------------------
def _reset_model_state(model: Any) -> None:
    for layer in getattr(model, "layers", []):
        core = getattr(layer, "core", None)
        if core is not None and hasattr(core, "state"):
            core.state = None
    om = getattr(model, "outer_model", None)
    if om is not None:
        _clear_outer(om)
        if hasattr(om, "loss_ema"):
            om.loss_ema.fill_(2.0)
    bpm = getattr(model, "bucket_prototypes_module", None)
    if bpm is not None and hasattr(bpm, "prototypes"):
        bpm.prototypes.zero_()
    st = getattr(model, "semantic_tier", None)
    if st is not None and hasattr(st, "bases"):
        st.bases.zero_()
    post = getattr(model, "posterior", None)
    if post is not None and hasattr(post, "reset"):
        post.reset()


def _assert_state_clean(model: Any) -> None:
    om = getattr(model, "outer_model", None)
    if isinstance(om, MultiSlotOuterModel):
        assert len(om._slots) == 0, "state leak: buffer not empty after reset"
        assert len(om._survival) == 0, "state leak: survival scores not empty"
        assert len(om._slot_buckets) == 0, "state leak: bucket assignments not empty"
        assert len(om._latent_traces) == 0, "state leak: latent traces not empty"
    bpm = getattr(model, "bucket_prototypes_module", None)
    if bpm is not None and hasattr(bpm, "prototypes"):
        assert bpm.prototypes.abs().sum() == 0, "state leak: prototypes not zeroed"
    st = getattr(model, "semantic_tier", None)
    if st is not None and hasattr(st, "bases"):
        assert st.bases.abs().sum() == 0, "state leak: semantic tier bases not zeroed"
    post = getattr(model, "posterior", None)
    for attr in ("delta", "deltas"):
        if post is not None and hasattr(post, attr):
            assert getattr(post, attr).abs().sum() == 0, f"state leak: posterior {attr} not zeroed"


def _assert_no_grad_leak(model: Any) -> None:
    for n, p in model.named_parameters():
        assert p.grad is None or p.grad.abs().sum() == 0, f"gradient leak: {n} has non-zero .grad after eval"


def _assert_bpb_sane(bpb: float, label: str = "") -> None:
    assert math.isfinite(bpb), f"bpb is not finite: {bpb} {label}"
    assert 0 < bpb < 15, f"bpb out of sane range [0, 15]: {bpb} {label}"


def _segments(n_tokens: int, warmup_tokens, score_tokens, segment_len, segment_starts, max_segments) -> list[int]:
    if segment_starts is None:
        seg = segment_len if segment_len is not None else max(warmup_tokens) + score_tokens + 1
        segment_starts = list(range(0, n_tokens - seg + 1, seg)) or [0]
    if max_segments > 0 and len(segment_starts) > max_segments:
        segment_starts = sorted(random.Random(42).sample(segment_starts, max_segments))
    return segment_starts


def _window(tokens, a, b, device):
    return (tokens[a:b].unsqueeze(0).to(device=device, dtype=torch.long),
            tokens[a + 1:b + 1].unsqueeze(0).to(device=device, dtype=torch.long))


def evaluate_warming_curve(model: Any, tokens: torch.Tensor, *, warmup_tokens: Optional[list[int]] = None,
                           score_tokens: int = 1024, segment_len: Optional[int] = None,
                           segment_starts: Optional[list[int]] = None, max_segments: int = 10,
                           device: Optional[torch.device] = None) -> dict[int, float]:
    """``{N: mean bpb}``: reset, feed ``N`` tokens with append-only memory writes (unscored,
    256 at a time), score the next ``score_tokens`` with writes off, per segment."""
    warmup_tokens = list(WARMING_CURVE_STEPS) if warmup_tokens is None else warmup_tokens
    device = next(model.parameters()).device if device is None else device
    starts = _segments(int(tokens.numel()), warmup_tokens, score_tokens, segment_len, segment_starts, max_segments)
    was_training = model.training
    model.eval()
    V, n_all = model.vocab_size, int(tokens.numel())
    out_curve: dict[int, float] = {}
    try:
        with torch.no_grad():
            for N in warmup_tokens:
                ce = torch.zeros((), dtype=torch.float64, device=device)
                scored = 0
                for s in starts:
                    _reset_model_state(model)
                    _assert_state_clean(model)
                    for a in range(s, s + N, 256):
                        b = min(a + 256, s + N)
                        if b + 1 > n_all:
                            break
                        model(_window(tokens, a, b, device)[0], memory_write_mode="append_only")
                    a, b = s + N, s + N + score_tokens
                    if b + 1 > n_all:
                        continue
                    inp, tgt = _window(tokens, a, b, device)
                    logits = model(inp, memory_write_mode="none")["logits"]
                    ce += F.cross_entropy(logits.float().reshape(-1, V), tgt.reshape(-1), reduction="sum").double()
                    scored += tgt.numel()
                if scored:
                    bpb = float(ce) / scored / math.log(2.0)
                    _assert_bpb_sane(bpb, f"warming_curve N={N}")
                    out_curve[N] = bpb
                else:
                    out_curve[N] = float("nan")
    finally:
        if was_training:
            model.train()
    return out_curve


# ---------------------------------------------------------------------------
# buffer x causal SLOT
# ---------------------------------------------------------------------------
_CONDITIONS = {"cold": (False, False), "buffer_only": (True, False), "slot_only": (False, True),
               "buffer_plus_slot": (True, True)}


def causal_slot_eval(model, tokens: torch.Tensor, *, conditions: tuple[str, ...] = tuple(_CONDITIONS),
                     warmup_tokens: Optional[list[int]] = None, score_tokens: int = 1024, window_size: int = 256,
                     slot_lr: float = 1e-3, slot_steps: int = 24, segment_starts: Optional[list[int]] = None,
                     segment_len: Optional[int] = None, max_segments: int = 10, freeze_during_scoring: bool = True,
                     device: Optional[torch.device] = None) -> dict[str, dict[int, float]]:
    """``{condition: {N: bpb}}`` for the 2x2 of (episodic buffer on/off) x (causal SLOT on/off).
    SLOT = a hidden-space ``delta`` and a ``logit_bias`` optimised by Adam on each warm-up window;
    model parameters stay frozen.  ``freeze_during_scoring=False`` keeps adapting while scoring
    (each window is scored before it is trained on)."""
    warmup_tokens = list(WARMING_CURVE_STEPS) if warmup_tokens is None else warmup_tokens
    device = next(model.parameters()).device if device is None else device
    starts = _segments(int(tokens.numel()), warmup_tokens, score_tokens, segment_len, segment_starts, max_segments)
    was_training = model.training
    model.eval()
    saved_rg = {n: p.requires_grad for n, p in model.named_parameters()}
    for p in model.parameters():
        p.requires_grad_(False)
    D, V, n_all = model.dim, model.vocab_size, int(tokens.numel())
    dtype = next(model.parameters()).dtype

    def head(hidden, delta, bias):
        return model.lm_head(model.final_norm(hidden + delta)) + bias

    def hidden_of(inp, write: bool):
        with torch.no_grad():
            return model(inp, memory_write_mode="append_only" if write else "none")["hidden"].detach()

    def adapt(hidden, tgt_flat, delta, bias, opt):
        for _ in range(slot_steps):
            F.cross_entropy(head(hidden, delta, bias).float().reshape(-1, V), tgt_flat).backward()
            opt.step()
            opt.zero_grad()

    # determinism canary: two cold passes over the first segment must agree exactly
    if starts:
        sums = []
        for _ in range(2):
            _reset_model_state(model)
            inp, tgt = _window(tokens, starts[0], starts[0] + score_tokens, device)
            with torch.no_grad():
                lg = model.lm_head(model.final_norm(model(inp, memory_write_mode="none")["hidden"]))
                sums.append(float(F.cross_entropy(lg.float().reshape(-1, V), tgt.reshape(-1), reduction="sum")))
        assert sums[0] == sums[1], (f"Reproducibility canary failed: cold N=0 gave different results ({sums[0]} vs "
                                    f"{sums[1]}). State is leaking between resets.")
    results: dict[str, dict[int, float]] = {}
    try:
        for cond in conditions:
            buf_on, slot_on = _CONDITIONS[cond]
            per_n: dict[int, float] = {}
            for N in warmup_tokens:
                total, scored = 0.0, 0
                for s in starts:
                    _reset_model_state(model)
                    _assert_state_clean(model)
                    delta = torch.zeros(1, 1, D, device=device, dtype=dtype, requires_grad=True)
                    bias = torch.zeros(1, 1, V, device=device, dtype=dtype, requires_grad=True)
                    opt = torch.optim.Adam([delta, bias], lr=slot_lr)
                    if N > 0 and (buf_on or slot_on):
                        for a in range(s, s + N, window_size):
                            b = min(a + window_size, s + N)
                            if b + 1 > n_all:
                                break
                            inp, tgt = _window(tokens, a, b, device)
                            h = hidden_of(inp, buf_on)
                            if slot_on:
                                adapt(h, tgt.reshape(-1), delta, bias, opt)
                    a0, b0 = s + N, s + N + score_tokens
                    if b0 + 1 > n_all:
                        continue
                    wins = [(a0, b0)] if freeze_during_scoring else \
                        [(a, min(a + window_size, b0)) for a in range(a0, b0, window_size)]
                    for a, b in wins:
                        if b + 1 > n_all:
                            break
                        inp, tgt = _window(tokens, a, b, device)
                        h = hidden_of(inp, buf_on and not freeze_during_scoring)
                        with torch.no_grad():
                            lg = head(h, delta.detach(), bias.detach())
                            total += float(F.cross_entropy(lg.float().reshape(-1, V), tgt.reshape(-1), reduction="sum"))
                        scored += tgt.numel()
                        if slot_on and not freeze_during_scoring:
                            adapt(h, tgt.reshape(-1), delta, bias, opt)
                if scored:
                    bpb = total / scored / math.log(2.0)
                    _assert_bpb_sane(bpb, f"causal_slot {cond} N={N}")
                    per_n[N] = bpb
                else:
                    per_n[N] = float("nan")
            results[cond] = per_n
    finally:
        for n, p in model.named_parameters():
            p.requires_grad_(saved_rg.get(n, p.requires_grad))
        _assert_no_grad_leak(model)
        if was_training:
            model.train()
    return results
