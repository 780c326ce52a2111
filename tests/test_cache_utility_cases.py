"""Memory-utility oracle pieces, one property per test (CPU)."""
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from chaoscontrol_b200 import cache_utility as CU
from chaoscontrol_b200.cache_utility import (
    LOSS_REWEIGHT_DIAGNOSTIC_NAMES, CrctGradientConflictMonitor, ScarcityAwareMemoryOptimizer, alpha_ramp,
    assign_memory_credit, chunked_nll_from_hidden, plasticity_budget_from_hidden_delta,
    positive_only_lm_weight, rank3_score_batch_causal)
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.wake_cache import TransactionalWakeCache

W = dict(tau=0.1, strength=0.1, w_max=1.15)


# ---------------------------------------------------------------- loss weight
def test_uniform_positive_utility_normalises_to_one():
    w = positive_only_lm_weight(torch.full((2, 5), 0.3), torch.ones(2, 5, dtype=torch.bool), **W)
    assert torch.allclose(w, torch.ones(2, 5), atol=1e-6)


def test_large_negative_utility_is_not_downweighted():
    u = torch.tensor([[-50.0, -0.2, 0.0]])
    w = positive_only_lm_weight(u, torch.ones(1, 3, dtype=torch.bool), **W)
    assert torch.allclose(w, torch.ones(1, 3), atol=1e-6)


def test_weight_matches_relu_tanh_statement():
    torch.manual_seed(0)
    u = torch.randn(3, 7) * 0.2
    m = torch.rand(3, 7) > 0.2
    raw = (1 + 0.1 * F.relu(torch.tanh(u / 0.1))).clamp(1.0, 1.15)
    want = raw / raw[m].mean() * m
    assert torch.allclose(positive_only_lm_weight(u, m, **W), want, atol=1e-6)


def test_mixed_signs_upweight_positives_relative_to_negatives():
    w = positive_only_lm_weight(torch.tensor([[0.5, -0.5]]), torch.ones(1, 2, dtype=torch.bool), **W)
    assert w[0, 0] > 1.0 > w[0, 1] and float(w.mean()) == pytest.approx(1.0)


def test_w_max_clamps_the_raw_weight():
    u = torch.tensor([[10.0, 0.0]])
    w = positive_only_lm_weight(u, torch.ones(1, 2, dtype=torch.bool), tau=0.1, strength=5.0, w_max=1.5)
    assert float(w[0, 0] / w[0, 1]) == pytest.approx(1.5)


def test_invalid_positions_get_zero_and_mean_is_over_valid_only():
    u = torch.tensor([[0.4, 0.0, 0.4, 0.0]])
    m = torch.tensor([[True, True, False, False]])
    w = positive_only_lm_weight(u, m, **W)
    assert w[0, 2] == 0 and w[0, 3] == 0 and float(w[m].mean()) == pytest.approx(1.0)


def test_all_invalid_gives_zeros_not_nan():
    w = positive_only_lm_weight(torch.randn(2, 3), torch.zeros(2, 3, dtype=torch.bool), **W)
    assert torch.isfinite(w).all() and float(w.abs().sum()) == 0.0


def test_weight_shape_and_dtype_follow_input():
    w = positive_only_lm_weight(torch.randn(4, 9).half(), torch.ones(4, 9, dtype=torch.bool), **W)
    assert w.shape == (4, 9) and w.dtype == torch.float32


def test_reweight_diagnostics_measure_weighted_against_plain():
    nll = torch.tensor([[1.0, 3.0, 9.0]])
    w = torch.tensor([[0.5, 1.5, 0.0]])
    m = torch.tensor([[True, True, False]])
    d = dict(zip(LOSS_REWEIGHT_DIAGNOSTIC_NAMES, CU._loss_reweight_diagnostics(nll_off=nll, loss_weight=w, mask=m).tolist()))
    assert d["valid_tokens"] == 2 and d["plain_nll_mean"] == pytest.approx(2.0)
    assert d["weighted_nll_mean"] == pytest.approx((0.5 + 4.5) / 2.0) and d["weighted_minus_plain"] == pytest.approx(0.5)
    assert d["weighted_rel_delta"] == pytest.approx(0.25) and d["loss_weight_abs_dev_mean"] == pytest.approx(0.5)
    assert d["loss_weight_std"] == pytest.approx(0.5) and d["loss_weight_max"] == pytest.approx(1.5)
    z = CU._loss_reweight_diagnostics(nll_off=nll, loss_weight=w, mask=torch.zeros_like(m))
    assert float(z.abs().sum()) == 0.0


# ---------------------------------------------------------------- per-token NLL
class _LM(nn.Module):
    def __init__(self, D=8, V=13, dtype=torch.float32):
        super().__init__()
        torch.manual_seed(0)
        self.final_norm = nn.LayerNorm(D).to(dtype)
        self.lm_head = nn.Linear(D, V, bias=False).to(dtype)


def test_nll_shape_sign_and_reference():
    m = _LM()
    h, y = torch.randn(3, 10, 8), torch.randint(0, 13, (3, 10))
    out = chunked_nll_from_hidden(m, h, y)
    assert out.shape == (3, 10) and out.dtype == torch.float32 and bool((out >= 0).all())
    want = F.cross_entropy(m.lm_head(m.final_norm(h)).reshape(-1, 13), y.reshape(-1), reduction="none").view(3, 10)
    assert torch.allclose(out, want, atol=1e-5)


@pytest.mark.parametrize("chunk", [1, 3, 10, 1000])
def test_nll_chunk_size_does_not_change_result(chunk):
    m = _LM()
    h, y = torch.randn(2, 10, 8), torch.randint(0, 13, (2, 10))
    assert torch.allclose(chunked_nll_from_hidden(m, h, y, chunk_size=chunk), chunked_nll_from_hidden(m, h, y), atol=1e-6)


def test_nll_accepts_int32_targets_and_casts_hidden_to_head_dtype():
    m = _LM(dtype=torch.bfloat16)
    h, y = torch.randn(2, 6, 8), torch.randint(0, 13, (2, 6), dtype=torch.int32)
    out = chunked_nll_from_hidden(m, h, y)
    assert out.dtype == torch.float32 and torch.isfinite(out).all()


def test_nll_budget_clamps_the_chunk(monkeypatch):
    m = _LM()
    seen = []
    real = m.lm_head.forward
    monkeypatch.setattr(m.lm_head, "forward", lambda x: (seen.append(x.shape[1]), real(x))[1])
    h, y = torch.randn(2, 10, 8), torch.randint(0, 13, (2, 10))
    tight = chunked_nll_from_hidden(m, h, y, chunk_size=10, chunk_budget_bytes=2 * 13 * 4 * 3)    # three steps' worth
    assert max(seen) == 3 and len(seen) == 4
    assert torch.allclose(tight, chunked_nll_from_hidden(m, h, y, chunk_size=10), atol=1e-6)


@pytest.mark.parametrize("kw", [dict(chunk_size=0), dict(chunk_size=-2), dict(chunk_budget_bytes=0), dict(chunk_budget_bytes=-1)])
def test_nll_rejects_non_positive_sizes(kw):
    with pytest.raises(ValueError):
        chunked_nll_from_hidden(_LM(), torch.randn(1, 2, 8), torch.zeros(1, 2, dtype=torch.long), **kw)


def test_nll_has_no_host_side_scorer_argument():
    import inspect
    assert set(inspect.signature(chunked_nll_from_hidden).parameters) == {"model", "hidden_states", "targets", "chunk_size",
                                                                         "chunk_budget_bytes"}


# ---------------------------------------------------------------- alpha ramp
def test_alpha_ramp_landmarks():
    assert alpha_ramp(0, 100, alpha_max=1.0) < 0.1
    assert alpha_ramp(30, 100, alpha_max=1.0) == pytest.approx(0.5)
    assert alpha_ramp(100, 100, alpha_max=1.0) > 0.99
    assert alpha_ramp(30, 100, alpha_max=0.2) == pytest.approx(0.1)


def test_alpha_ramp_is_monotone_and_total_zero_counts_as_done():
    v = [alpha_ramp(s, 50, alpha_max=0.7) for s in range(51)]
    assert all(b > a for a, b in zip(v, v[1:]))
    assert alpha_ramp(0, 0, alpha_max=0.7) == pytest.approx(alpha_ramp(10, 10, alpha_max=0.7))


# ---------------------------------------------------------------- prices
def test_optimizer_initial_state():
    o = ScarcityAwareMemoryOptimizer()
    assert o.read_price == o.write_price == 0.0 and o.read_rate_ema == 0.25 and o.write_rate_ema == 0.10


def test_targets_are_detached_clamped_and_shaped():
    o = ScarcityAwareMemoryOptimizer()
    u = (torch.randn(3, 5) * 5).requires_grad_()
    for fn in (o.controller_target, o.write_target):
        t, c = fn(u)
        assert t.shape == c.shape == (3, 5) and not t.requires_grad and not c.requires_grad
        assert float(t.min()) >= 0.05 and float(t.max()) <= 0.95 and float(c.min()) >= 0 and float(c.max()) <= 1


def test_dual_step_moves_price_toward_balance():
    o = ScarcityAwareMemoryOptimizer(dual_lr=0.5, ema_beta=0.0)
    o.dual_step(actual_read_rate=0.75)
    assert o.read_price == pytest.approx(0.25) and o.write_price == 0.0            # write side untouched
    o.dual_step(actual_read_rate=0.05)
    assert o.read_price == pytest.approx(0.15)
    for _ in range(10):
        o.dual_step(actual_read_rate=0.0)
    assert o.read_price == 0.0
    for _ in range(20):
        o.dual_step(actual_read_rate=1.0, actual_write_rate=1.0)
    assert o.read_price == o.max_price == 0.5 and o.write_price == 0.5


def test_ema_smooths_the_rate():
    o = ScarcityAwareMemoryOptimizer(ema_beta=0.9)
    o.dual_step(actual_read_rate=1.0)
    assert o.read_rate_ema == pytest.approx(0.9 * 0.25 + 0.1)


def test_read_price_shifts_the_target_and_confidence_peaks_at_extremes():
    o = ScarcityAwareMemoryOptimizer(tau=0.1)
    u = torch.tensor([0.1])
    free, _ = o.controller_target(u)
    o.read_price = 0.1
    priced, conf0 = o.controller_target(u)
    assert float(free) > float(priced) == pytest.approx(0.5) and float(conf0) == pytest.approx(0.0)
    _, conf = o.controller_target(torch.tensor([-3.0, 0.1, 3.0]))
    assert conf[0] > 0.99 and conf[2] > 0.99 and conf[1] < 0.01


# ---------------------------------------------------------------- credit
def _ledger(n=6):
    return torch.zeros(n), torch.zeros(n)


def test_positive_utility_is_credit_negative_is_debit_zero_is_neither():
    ids = torch.tensor([[[2]]])
    w = torch.tensor([[[0.5]]])
    for u, want_c, want_d in ((0.4, 0.2, 0.0), (-0.4, 0.0, 0.2), (0.0, 0.0, 0.0)):
        c, d = _ledger()
        assign_memory_credit(c, d, ids, w, torch.tensor([[u]]))
        assert float(c[2]) == pytest.approx(want_c) and float(d[2]) == pytest.approx(want_d)
        assert float(c.sum() + d.sum()) == pytest.approx(want_c + want_d)


def test_credit_accumulates_over_calls_and_entries():
    c, d = _ledger()
    ids = torch.tensor([[[1, 3], [3, 3]]])
    w = torch.tensor([[[0.25, 0.75], [0.5, 0.5]]])
    u = torch.tensor([[1.0, -2.0]])
    assign_memory_credit(c, d, ids, w, u)
    assign_memory_credit(c, d, ids, w, u)
    assert c.tolist() == pytest.approx([0, 0.5, 0, 1.5, 0, 0]) and d.tolist() == pytest.approx([0, 0, 0, 4.0, 0, 0])


def test_credit_needs_no_grad_and_keeps_ledger_dtype():
    c, d = torch.zeros(4, dtype=torch.float64), torch.zeros(4, dtype=torch.float64)
    u = torch.tensor([[0.5]], requires_grad=True)
    assign_memory_credit(c, d, torch.tensor([[[0]]]), torch.tensor([[[1.0]]]), u)
    assert c.dtype == torch.float64 and not c.requires_grad and float(c[0]) == 0.5


# ---------------------------------------------------------------- plasticity
def test_plasticity_positive_when_residual_tracks_utility():
    torch.manual_seed(0)
    u = torch.rand(2, 40)
    h_off = torch.zeros(2, 40, 3)
    h_mem = torch.stack([u, torch.rand(2, 40), torch.full((2, 40), 0.3)], -1)
    out = plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem, utility=u, mask=torch.ones(2, 40, dtype=torch.bool), tau=0.1)
    cov = out["plasticity_coverage"]
    assert cov[0] > 0.99 and abs(float(cov[1])) < 0.4 and float(cov[2]) == pytest.approx(0.0, abs=1e-3)
    assert out["plasticity_budget"][0] > 0.9 and out["plasticity_budget"][2] == pytest.approx(0.0, abs=1e-3)


def test_plasticity_closed_without_positive_utility_or_valid_tokens():
    h_mem = torch.randn(2, 10, 4)
    h_off = torch.zeros_like(h_mem)
    neg = plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem, utility=-torch.rand(2, 10),
                                              mask=torch.ones(2, 10, dtype=torch.bool), tau=0.1)
    none = plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem, utility=torch.rand(2, 10),
                                               mask=torch.zeros(2, 10, dtype=torch.bool), tau=0.1)
    for out in (neg, none):
        assert float(out["plasticity_budget"].abs().sum()) == 0.0 and torch.isfinite(out["plasticity_coverage"]).all()


def test_plasticity_anticorrelated_channel_gets_no_budget_but_has_confidence():
    u = torch.rand(1, 50)
    h_mem = (1.0 - u).unsqueeze(-1)
    out = plasticity_budget_from_hidden_delta(h_off=torch.zeros_like(h_mem), h_mem=h_mem, utility=u,
                                              mask=torch.ones(1, 50, dtype=torch.bool), tau=0.1)
    assert out["plasticity_coverage"][0] < -0.99 and out["plasticity_budget"][0] == 0.0 and out["plasticity_confidence"][0] > 0.9


@pytest.mark.parametrize("bad", ["shape", "rank", "util", "mask"])
def test_plasticity_rejects_mismatched_inputs(bad):
    h = torch.zeros(2, 5, 3)
    kw = dict(h_off=h, h_mem=h.clone(), utility=torch.zeros(2, 5), mask=torch.ones(2, 5, dtype=torch.bool), tau=0.1)
    if bad == "shape":
        kw["h_mem"] = torch.zeros(2, 5, 4)
    elif bad == "rank":
        kw["h_off"] = kw["h_mem"] = torch.zeros(10, 3)
    elif bad == "util":
        kw["utility"] = torch.zeros(2, 4)
    else:
        kw["mask"] = torch.ones(5, 2, dtype=torch.bool)
    with pytest.raises(ValueError):
        plasticity_budget_from_hidden_delta(**kw)


def test_compact_residual_contract():
    assert CU._compact_residual(torch.zeros(3, 8), 3).shape == (3, 1, 8)
    assert CU._compact_residual(torch.zeros(3, 1, 8), 3).shape == (3, 1, 8)
    with pytest.raises(ValueError, match="compact"):
        CU._compact_residual(torch.zeros(3, 5, 8), 3)                      # a per-token packet is refused
    with pytest.raises(ValueError, match="batch"):
        CU._compact_residual(torch.zeros(2, 8), 3)


# ---------------------------------------------------------------- conflict monitor
class _TinyLM(nn.Module):
    def __init__(self):
        super().__init__()
        self.final_norm = nn.Identity()
        self.lm_head = nn.Linear(2, 2, bias=False)
        with torch.no_grad():
            self.lm_head.weight.copy_(torch.tensor([[1.0, 0.0], [-1.0, 0.0]]))


def _apply(mon, targets, util=(1.0, 0.5), max_tokens=2, mask=None, step=None):
    hidden = torch.zeros(1, 2, 2)
    u = torch.tensor([list(util)])
    m = torch.ones(1, 2, dtype=torch.bool) if mask is None else mask
    return mon.apply_to_write_scores(model=_TinyLM(), hidden=hidden, targets=torch.tensor([targets]), utility=u, mask=m,
                                     max_tokens=max_tokens, step=step)


def test_monitor_cold_start_only_observes():
    mon = CrctGradientConflictMonitor()
    score, limit = _apply(mon, [0, 0])
    d = mon.diagnostics()
    assert score.tolist() == [[1.0, 0.5]] and limit == 2 and d["cold_start_calls"] == 1 and d["has_reference"]
    assert d["guardrail_suppressed_candidates"] == 0 and d["candidates_compared"] == 0


def test_monitor_aligned_candidates_pass_untouched():
    mon = CrctGradientConflictMonitor()
    _apply(mon, [0, 0])
    score, limit = _apply(mon, [0, 0])
    d = mon.diagnostics()
    assert score.tolist() == [[1.0, 0.5]] and limit == 2 and d["max_conflict"] == pytest.approx(1.0)
    assert d["candidates_compared"] == 2 and d["admitted_candidates"] >= 2


def test_monitor_threshold_decides_suppression():
    for thr, suppressed in ((-0.5, True), (-1.5, False)):
        mon = CrctGradientConflictMonitor(catastrophic_threshold=thr)
        _apply(mon, [0, 0])
        score, limit = _apply(mon, [0, 1])
        assert bool(score[0, 1] == -math.inf) is suppressed and limit == (1 if suppressed else 2)


def test_monitor_soft_gate_floor():
    mon = CrctGradientConflictMonitor(catastrophic_threshold=-2.0, soft_gate_strength=5.0, soft_gate_floor=0.2)
    _apply(mon, [0, 0])
    score, _ = _apply(mon, [0, 1])
    assert float(score[0, 1]) == pytest.approx(0.5 * 0.2) and float(score[0, 0]) == pytest.approx(1.0)


def test_monitor_disabled_and_empty_mask():
    off = CrctGradientConflictMonitor(enabled=False)
    score, limit = _apply(off, [0, 1], max_tokens=1)
    assert score.tolist() == [[1.0, 0.5]] and limit == 1 and off.diagnostics()["calls"] == 0
    mon = CrctGradientConflictMonitor()
    _, limit = _apply(mon, [0, 0], mask=torch.zeros(1, 2, dtype=torch.bool))
    assert limit == 0


def test_monitor_trace_stride_and_cap(tmp_path):
    path = tmp_path / "c.jsonl"
    mon = CrctGradientConflictMonitor(trace_path=str(path), trace_stride=2, trace_max_rows=100, trace_flush_rows=1)
    for step in range(4):
        _apply(mon, [0, 0], step=step)
    mon.flush_trace()
    import json
    steps = sorted({json.loads(l)["step"] for l in path.read_text().splitlines()})
    assert steps == [0, 2] or steps == [1, 3]                      # every second call is traced
    assert mon.diagnostics()["trace_rows_written"] == len(path.read_text().splitlines())


# ---------------------------------------------------------------- the oracle on the real model
def _memory_model(seed=0):
    torch.manual_seed(seed)
    return CareStudentLM(vocab_size=48, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                         outer_max_slots=0, buffer_mode="append_only")


def _batch(B=3, T=9, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 48, (B, T), generator=g), torch.ones(B, T, dtype=torch.bool)


def test_oracle_returns_expected_keys_and_per_target_shapes():
    ids, valid = _batch()
    out = rank3_score_batch_causal(model=_memory_model(), cache=TransactionalWakeCache(), input_ids=ids, valid_mask=valid)
    assert {"utility", "controller_target", "confidence", "loss_weight", "loss_reweight_diagnostics",
            "plasticity_coverage", "plasticity_confidence", "plasticity_budget"} <= set(out)
    for k in ("utility", "controller_target", "confidence", "loss_weight"):
        assert out[k].shape == (3, 8)
    assert out["plasticity_budget"].shape == (16,) and "memory_write_records" not in out


def test_oracle_needs_no_grad_and_leaves_none():
    m = _memory_model()
    ids, valid = _batch()
    out = rank3_score_batch_causal(model=m, cache=TransactionalWakeCache(), input_ids=ids, valid_mask=valid)
    assert all(p.grad is None for p in m.parameters())
    assert not any(v.requires_grad for v in out.values() if isinstance(v, torch.Tensor))


def test_oracle_cache_lifecycle_is_begin_then_commit():
    calls = []

    class Cache(TransactionalWakeCache):
        def begin_batch(self):
            calls.append("begin")
            return super().begin_batch()

        def commit(self, txn):
            calls.append("commit")
            return super().commit(txn)
    ids, valid = _batch()
    rank3_score_batch_causal(model=_memory_model(), cache=Cache(), input_ids=ids, valid_mask=valid)
    assert calls == ["begin", "commit"]


def test_oracle_zeroes_invalid_positions_with_and_without_prices():
    ids, valid = _batch()
    valid[0, 4:] = False
    m = _memory_model()
    cache = TransactionalWakeCache()
    rank3_score_batch_causal(model=m, cache=cache, input_ids=ids, valid_mask=valid, update_model_memory_after=True,
                             memory_write_tokens=6)
    sc = ScarcityAwareMemoryOptimizer()
    sc.read_price = 0.2
    for opt in (None, sc):
        out = rank3_score_batch_causal(model=m, cache=cache, input_ids=ids, valid_mask=valid, scarcity_optimizer=opt)
        for k in ("utility", "controller_target", "confidence", "loss_weight"):
            assert float(out[k][0, 3:].abs().sum()) == 0.0, k
        mm = valid[:, 1:]
        assert float(out["loss_weight"][mm].mean()) == pytest.approx(1.0, rel=1e-5)


def test_oracle_price_lowers_controller_targets():
    ids, valid = _batch()
    m = _memory_model()
    cache = TransactionalWakeCache()
    rank3_score_batch_causal(model=m, cache=cache, input_ids=ids, valid_mask=valid, update_model_memory_after=True,
                             memory_write_tokens=6)
    free = rank3_score_batch_causal(model=m, cache=cache, input_ids=ids, valid_mask=valid,
                                    scarcity_optimizer=ScarcityAwareMemoryOptimizer())
    sc = ScarcityAwareMemoryOptimizer()
    sc.read_price = 0.3
    priced = rank3_score_batch_causal(model=m, cache=cache, input_ids=ids, valid_mask=valid, scarcity_optimizer=sc)
    assert torch.allclose(free["utility"], priced["utility"])
    assert float(priced["controller_target"].sum()) < float(free["controller_target"].sum())


def test_oracle_stage_seconds_are_optional_and_named():
    ids, valid = _batch()
    stages: dict = {}
    rank3_score_batch_causal(model=_memory_model(), cache=TransactionalWakeCache(), input_ids=ids, valid_mask=valid,
                             record_stage_seconds=stages)
    assert {"encode_off", "nll_off", "nll_mem", "plasticity"} <= set(stages) and all(v >= 0 for v in stages.values())
    assert stages["_batch"] == 3.0 and stages["_seq_len"] == 8.0 if "_batch" in stages else stages["_seq_len"] == 8.0


def test_oracle_writes_only_the_requested_number_of_tokens_with_fresh_event_ids():
    ids, valid = _batch()
    m = _memory_model()
    cache = TransactionalWakeCache()
    a = rank3_score_batch_causal(model=m, cache=cache, input_ids=ids, valid_mask=valid, update_model_memory_after=True,
                                 memory_write_tokens=3)
    b = rank3_score_batch_causal(model=m, cache=cache, input_ids=ids, valid_mask=valid, update_model_memory_after=True,
                                 memory_write_tokens=2)
    ea = [int(r["event_id"]) for r in a["memory_write_records"]]
    eb = [int(r["event_id"]) for r in b["memory_write_records"]]
    assert len(ea) == 3 and len(eb) == 2 and len(set(ea + eb)) == 5 and min(eb) > max(ea)
    assert m.outer_model.table.n_active == 5
