"""Memory-utility oracle (cf. tests/test_cache_utility.py of the reference)."""
import json
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from chaoscontrol_b200.cache_utility import (
    LOSS_REWEIGHT_DIAGNOSTIC_NAMES, CrctGradientConflictMonitor, ScarcityAwareMemoryOptimizer, alpha_ramp,
    assign_memory_credit, chunked_nll_from_hidden, plasticity_budget_from_hidden_delta,
    positive_only_lm_weight, rank3_score_batch_causal)
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.wake_cache import TransactionalWakeCache


# ---------------------------------------------------------------- weights / ramp / prices
def test_positive_only_weight():
    u = torch.tensor([[0.5, -3.0, 0.0, 0.2]])
    m = torch.tensor([[True, True, True, False]])
    w = positive_only_lm_weight(u, m, tau=0.1, strength=0.1, w_max=1.15)
    raw = (1.0 + 0.1 * torch.relu(torch.tanh(u / 0.1))).clamp(1.0, 1.15)
    assert torch.allclose(w[0, :3], raw[0, :3] / raw[0, :3].mean())
    assert w[0, 3] == 0 and w[0, 1] == w[0, 2]
    assert math.isclose(float(w[m].mean()), 1.0, rel_tol=1e-6)
    assert torch.equal(positive_only_lm_weight(u, torch.zeros_like(m), tau=0.1, strength=0.1, w_max=1.15),
                       torch.zeros_like(u))
    big = positive_only_lm_weight(torch.tensor([[100.0, 0.0]]), torch.ones(1, 2, dtype=torch.bool), tau=0.1,
                                  strength=5.0, w_max=1.5)
    assert math.isclose(float(big[0, 0] / big[0, 1]), 1.5, rel_tol=1e-6)


def test_alpha_ramp():
    assert math.isclose(alpha_ramp(30, 100, alpha_max=0.4), 0.2, rel_tol=1e-9)
    assert alpha_ramp(0, 100, alpha_max=1.0) < 0.1 and alpha_ramp(100, 100, alpha_max=1.0) > 0.99
    vals = [alpha_ramp(s, 50, alpha_max=1.0) for s in range(51)]
    assert vals == sorted(vals)
    assert alpha_ramp(3, 0, alpha_max=1.0) > 0.99


def test_scarcity_optimizer_prices():
    opt = ScarcityAwareMemoryOptimizer(dual_lr=0.1, ema_beta=0.0, max_price=0.2)
    assert opt.read_price == 0.0 and opt.read_rate_ema == 0.25
    t, c = opt.controller_target(torch.tensor([-5.0, 0.0, 5.0]))
    assert t.tolist() == pytest.approx([0.05, 0.5, 0.95]) and c[1] == 0 and c[2] > 0.99
    opt.dual_step(actual_read_rate=1.0)
    assert math.isclose(opt.read_price, 0.075) and opt.write_price == 0.0
    for _ in range(10):
        opt.dual_step(actual_read_rate=1.0, actual_write_rate=1.0)
    assert opt.read_price == 0.2 and opt.write_price == 0.2
    t2, _ = opt.controller_target(torch.tensor([0.2]))
    assert math.isclose(float(t2), 0.5)
    for _ in range(10):
        opt.dual_step(actual_read_rate=0.0)
    assert opt.read_price == 0.0
    smooth = ScarcityAwareMemoryOptimizer(ema_beta=0.9)
    smooth.dual_step(actual_read_rate=1.0)
    assert math.isclose(smooth.read_rate_ema, 0.9 * 0.25 + 0.1)


def test_assign_memory_credit():
    credit, debit = torch.zeros(4), torch.zeros(4)
    ids = torch.tensor([[[0, 1], [1, 2]]])
    w = torch.tensor([[[0.75, 0.25], [0.5, 0.5]]])
    assign_memory_credit(credit, debit, ids, w, torch.tensor([[2.0, -4.0]]))
    assert credit.tolist() == [1.5, 0.5, 0.0, 0.0] and debit.tolist() == [0.0, 2.0, 2.0, 0.0]


# ---------------------------------------------------------------- NLL
class _Head(nn.Module):
    def __init__(self, dim=8, vocab=32):
        super().__init__()
        self.final_norm = nn.LayerNorm(dim)
        self.lm_head = nn.Linear(dim, vocab, bias=False)


def test_chunked_nll_matches_cross_entropy_for_any_chunking():
    torch.manual_seed(0)
    m = _Head()
    h, y = torch.randn(3, 11, 8), torch.randint(0, 32, (3, 11), dtype=torch.int32)
    ref = F.cross_entropy(m.lm_head(m.final_norm(h)).reshape(-1, 32), y.reshape(-1).long(),
                          reduction="none").view(3, 11)
    for kw in ({}, {"chunk_size": 2}, {"chunk_size": 1000, "chunk_budget_bytes": 3 * 32 * 4 * 3}):
        assert torch.allclose(chunked_nll_from_hidden(m, h, y, **kw), ref, atol=1e-6)
    with pytest.raises(ValueError):
        chunked_nll_from_hidden(m, h, y, chunk_size=0)
    with pytest.raises(ValueError):
        chunked_nll_from_hidden(m, h, y, chunk_budget_bytes=0)
    m16 = _Head().to(torch.bfloat16)
    assert chunked_nll_from_hidden(m16, h, y).dtype == torch.float32


# ---------------------------------------------------------------- plasticity
def test_plasticity_matches_centered_statement():
    torch.manual_seed(1)
    B, T, D = 3, 9, 5
    h_off, h_mem = torch.randn(B, T, D), torch.randn(B, T, D)
    u, mask = torch.randn(B, T), torch.rand(B, T) > 0.3
    got = plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem, utility=u, mask=mask, tau=0.1)
    x = (h_mem - h_off).abs()[mask]
    y = torch.relu(u)[mask]
    xc, yc = x - x.mean(0), y - y.mean()
    cov = (xc * yc[:, None]).mean(0)
    ref = cov / torch.sqrt((xc.square().mean(0) * yc.square().mean()).clamp_min(1e-6))
    assert torch.allclose(got["plasticity_coverage"], ref.clamp(-1, 1), atol=1e-5)
    conf = ref.abs() * torch.tanh(torch.sqrt(y.square().mean()) / 0.1)
    assert torch.allclose(got["plasticity_confidence"], conf.clamp(0, 1), atol=1e-5)
    assert torch.allclose(got["plasticity_budget"], torch.relu(ref) * conf, atol=1e-5)


def test_plasticity_tracks_and_ignores():
    B, T, D = 2, 16, 3
    u = torch.linspace(0, 1, B * T).view(B, T)
    h_off = torch.zeros(B, T, D)
    h_mem = torch.zeros(B, T, D)
    h_mem[..., 0] = u
    h_mem[..., 1] = 1.0 - u
    mask = torch.ones(B, T, dtype=torch.bool)
    got = plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem, utility=u, mask=mask, tau=0.1)
    assert got["plasticity_coverage"][0] > 0.99 and got["plasticity_coverage"][1] < -0.99
    assert got["plasticity_budget"][0] > 0.9 and got["plasticity_budget"][1] == 0 and got["plasticity_budget"][2] == 0
    none = plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem, utility=-u, mask=mask, tau=0.1)
    assert float(none["plasticity_budget"].abs().sum()) == 0.0
    with pytest.raises(ValueError):
        plasticity_budget_from_hidden_delta(h_off=h_off, h_mem=h_mem[:, :3], utility=u, mask=mask, tau=0.1)


# ---------------------------------------------------------------- conflict sensor
class _TinyLM(nn.Module):
    def __init__(self):
        super().__init__()
        self.final_norm = nn.Identity()
        self.lm_head = nn.Linear(2, 2, bias=False)
        with torch.no_grad():
            self.lm_head.weight.copy_(torch.tensor([[1.0, 0.0], [-1.0, 0.0]]))


def test_conflict_monitor_cold_start_guardrail_and_trace(tmp_path):
    model = _TinyLM()
    path = tmp_path / "trace" / "conflict.jsonl"
    mon = CrctGradientConflictMonitor(catastrophic_threshold=-0.5, trace_path=str(path), trace_max_rows=3)
    hidden = torch.tensor([[[0.0, 0.0], [0.0, 0.0]]])
    util = torch.tensor([[1.0, 0.5]])
    mask = torch.ones(1, 2, dtype=torch.bool)
    # both tokens target class 0: gradient w.r.t. the head input points along -e0
    score, limit = mon.apply_to_write_scores(model=model, hidden=hidden, targets=torch.tensor([[0, 0]]),
                                             utility=util, mask=mask, max_tokens=2, step=7)
    assert torch.equal(score, util) and limit == 2 and mon.diagnostics()["cold_start_calls"] == 1
    # second token now targets class 1: gradient along +e0, cosine -1 with the EMA
    score, limit = mon.apply_to_write_scores(model=model, hidden=hidden, targets=torch.tensor([[0, 1]]),
                                             utility=util, mask=mask, max_tokens=2, step=8)
    assert score[0, 0] == 1.0 and score[0, 1] == -math.inf and limit == 1
    d = mon.diagnostics()
    assert d["guardrail_suppressed_candidates"] == 1 and d["last_reason"] == "guardrail_suppressed"
    assert d["min_conflict"] == pytest.approx(-1.0) and d["has_reference"]
    rows = [json.loads(l) for l in path.read_text().splitlines()]
    assert len(rows) == 3 and d["trace_rows_dropped"] == 1
    assert rows[0]["step"] == 7 and rows[0]["has_reference"] is False and rows[2]["has_reference"] is True
    # soft gate
    soft = CrctGradientConflictMonitor(catastrophic_threshold=-2.0, soft_gate_strength=0.5)
    soft.apply_to_write_scores(model=model, hidden=hidden, targets=torch.tensor([[0, 0]]), utility=util,
                               mask=mask, max_tokens=None)
    score, limit = soft.apply_to_write_scores(model=model, hidden=hidden, targets=torch.tensor([[0, 1]]),
                                              utility=util, mask=mask, max_tokens=None)
    assert score[0, 1] == pytest.approx(0.25) and limit == 2 and soft.diagnostics()["last_reason"] == "soft_gated"
    off = CrctGradientConflictMonitor(enabled=False)
    assert off.apply_to_write_scores(model=model, hidden=hidden, targets=torch.tensor([[0, 0]]), utility=util,
                                     mask=mask, max_tokens=1) == (util, 1)
    _, lim0 = mon.apply_to_write_scores(model=model, hidden=hidden, targets=torch.tensor([[0, 0]]), utility=util,
                                        mask=torch.zeros_like(mask), max_tokens=2)
    assert lim0 == 0


# ---------------------------------------------------------------- oracle on the real model
def _memory_model():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=48, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                         outer_max_slots=0, buffer_mode="append_only")


def test_oracle_end_to_end_with_append_and_event_cutoff():
    model = _memory_model()
    cache = TransactionalWakeCache()
    ids = torch.randint(0, 48, (3, 9))
    valid = torch.ones(3, 9, dtype=torch.bool)
    valid[1, 5:] = False
    stages: dict = {}
    out = rank3_score_batch_causal(model=model, cache=cache, input_ids=ids, valid_mask=valid,
                                   update_model_memory_after=True, memory_write_tokens=4,
                                   record_stage_seconds=stages)
    for k in ("utility", "controller_target", "confidence", "loss_weight"):
        assert out[k].shape == (3, 8)
        assert float(out[k][1, 4:].abs().sum()) == 0.0
    # empty store: memory changes nothing
    assert float(out["utility"].abs().max()) < 1e-5
    m = valid[:, 1:]
    assert math.isclose(float(out["loss_weight"][m].mean()), 1.0, rel_tol=1e-5)
    diag = dict(zip(LOSS_REWEIGHT_DIAGNOSTIC_NAMES, out["loss_reweight_diagnostics"].tolist()))
    assert diag["valid_tokens"] == int(m.sum()) and diag["plain_nll_mean"] > 0
    recs = out["memory_write_records"]
    assert len(recs) == 4
    cutoff_first = min(int(r["event_id"]) for r in recs)
    assert set(stages) >= {"encode_off", "nll_off", "nll_mem", "plasticity", "append_memory", "_paired_encode"}
    assert stages["_paired_encode"] == 1.0 and stages["_seq_len"] == 8.0
    # second batch sees the slots written by the first; its own writes carry later ids
    sc = ScarcityAwareMemoryOptimizer()
    out2 = rank3_score_batch_causal(model=model, cache=cache, input_ids=ids, valid_mask=valid,
                                    scarcity_optimizer=sc, update_model_memory_after=True, memory_write_tokens=2)
    assert float(out2["utility"].abs().max()) > 0
    assert out2["controller_target"][m].min() >= 0.05 and out2["controller_target"][m].max() <= 0.95
    assert 0 <= float(out2["confidence"].min()) and float(out2["confidence"].max()) <= 1
    assert min(int(r["event_id"]) for r in out2["memory_write_records"]) > max(int(r["event_id"]) for r in recs)
    assert cutoff_first > 0
    if "memory_residual" in out2:
        assert out2["memory_residual"].shape == (3, 1, 16) and out2["memory_gate"].shape == (3, 8)


def test_oracle_unpaired_path_and_guardrail_skip():
    model = _memory_model()
    calls = []

    class Wrapper:
        """Hides the paired encoder so the two-pass path runs."""
        lm_head, final_norm, dim = model.lm_head, model.final_norm, model.dim

        def encode(self, x, **kw):
            calls.append((kw["memory_mode"], kw["cache_read_cutoff"]))
            return model.encode(x, **kw)

        append_memory_from_hidden = staticmethod(model.append_memory_from_hidden)

    cache = TransactionalWakeCache()
    ids = torch.randint(0, 48, (2, 7))
    valid = torch.ones(2, 7, dtype=torch.bool)

    class Block(CrctGradientConflictMonitor):
        def apply_to_write_scores(self, **kw):
            return kw["utility"], 0

    out = rank3_score_batch_causal(model=Wrapper(), cache=cache, input_ids=ids, valid_mask=valid,
                                   update_model_memory_after=True, memory_write_tokens=3,
                                   gradient_conflict_monitor=Block())
    assert [c[0] for c in calls] == ["off", "force_on"] and calls[0][1] == calls[1][1]
    assert "memory_write_records" not in out and "gradient_conflict" in out and "write_score" in out
    with pytest.raises(ValueError):
        class NoAppend:
            lm_head, final_norm, dim = model.lm_head, model.final_norm, model.dim
            encode = staticmethod(model.encode)
        rank3_score_batch_causal(model=NoAppend(), cache=cache, input_ids=ids, valid_mask=valid,
                                 update_model_memory_after=True)
