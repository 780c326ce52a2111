"""Semantic optimizer, ScOpt, criticality distillation and the ScOpt gates (CPU)."""
import copy

import pytest
import torch

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim.criticality import CriticalityDistillation, compute_event_mask, compute_future_energy
from chaoscontrol_b200.optim.muon import Muon
from chaoscontrol_b200.optim.scopt import (FrequencyBucketBaseline, ScarcityAwareOptimizer, scarcity_pressure_from_ce,
                                           scopt_allreduce_config, scopt_optimizer_config)
from chaoscontrol_b200.optim.semantic import SemanticOptimizer, default_beta_from_log_a, semantic_optimizer_config
from chaoscontrol_b200.scopt_probes import evaluate_tier0_gates, summarize_gates


def _model(seed=0):
    torch.manual_seed(seed)
    return CareStudentLM(vocab_size=32, dim=16, num_layers=2)


def _grads(model, seed):
    g = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        p.grad = torch.randn(p.shape, generator=g)


# --------------------------------------------------------------------------- semantic
def test_semantic_reduces_to_muon_without_a_param():
    a, b = _model(), _model()
    oa = SemanticOptimizer(a.parameters(), lr=0.02, weight_decay=0.01)
    oa.bind_param_names(a.named_parameters())
    ob = Muon(b.parameters(), lr=0.02, weight_decay=0.01, fused=True,
              is_matrix=lambda p, n: p.ndim == 2)
    ob.bind_param_names(b.named_parameters())
    for s in range(3):
        _grads(a, s)
        _grads(b, s)
        oa.step()
        ob.step()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert torch.allclose(p, q, atol=1e-5), n


def test_semantic_per_channel_beta_shapes_momentum():
    m = _model()
    cfg = semantic_optimizer_config(m, 0)
    assert cfg["a_param_name"] == "layers.0.core.log_a" and cfg["channel_map"]["layers.0.core.out_proj.weight"] == 1
    with torch.no_grad():
        m.layers[0].core.log_a.copy_(torch.linspace(-6, 6, 16))
    opt = SemanticOptimizer(m.parameters(), lr=0.02, momentum=0.95, momentum_min=0.5, **cfg)
    opt.bind_param_names(m.named_parameters())
    beta = opt.current_beta_vec()
    assert torch.allclose(beta, default_beta_from_log_a(m.layers[0].core.log_a, beta_min=0.5, beta_max=0.95))
    tr = opt.beta_trace()
    assert tr["beta_min"] < 0.51 and tr["beta_max"] > 0.94 and tr["tau_steps"][-1] > tr["tau_steps"][0]
    W = m.layers[0].core.in_proj.weight
    Wo = m.layers[0].core.out_proj.weight
    for _ in range(2):
        W.grad = torch.ones_like(W)
        Wo.grad = torch.ones_like(Wo)
        for n, p in m.named_parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        opt.step()
    buf = opt.state[W]["momentum_buffer"]
    assert buf.dtype == torch.float32
    assert torch.allclose(buf[:, 0], 1.0 + beta)                     # axis 0 = state channels
    assert torch.allclose(opt.state[Wo]["momentum_buffer"][0], 1.0 + beta)   # axis 1 for out_proj
    with pytest.raises(ValueError):
        SemanticOptimizer(m.parameters(), a_param_name="x", channel_map={"x": 0})
    bad = SemanticOptimizer(m.parameters(), a_param_name="nope")
    with pytest.raises(ValueError):
        bad.bind_param_names(m.named_parameters())
    with pytest.raises(RuntimeError):
        bad2 = SemanticOptimizer(m.parameters(), a_param_name="layers.0.core.log_a")
        _grads(m, 0)
        bad2.step()


# --------------------------------------------------------------------------- scopt
def test_scopt_without_state_is_muon():
    a, b = _model(), _model()
    oa = ScarcityAwareOptimizer(a.parameters(), lr=0.02, weight_decay=0.01, warmup_steps=0)
    oa.bind_param_names(a.named_parameters())
    ob = Muon(b.parameters(), lr=0.02, weight_decay=0.01, fused=True, is_matrix=lambda p, n: p.ndim == 2)
    ob.bind_param_names(b.named_parameters())
    for s in range(3):
        _grads(a, s)
        _grads(b, s)
        oa.step()
        ob.step()
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert torch.allclose(p, q, atol=1e-5), n


def test_scopt_rare_direction_is_orthogonal_and_capped():
    m = _model()
    opt = ScarcityAwareOptimizer(m.parameters(), lr=0.02, warmup_steps=0, rare_macro_c=0.5, momentum=0.0)
    opt.bind_param_names(m.named_parameters())
    W = m.layers[0].ff.fc.weight
    common = torch.randn_like(W)
    rare = torch.randn_like(W) * 10
    opt._step_count = 1
    opt.set_rare_grad_ema({"layers.0.ff.fc.weight": rare})
    d = opt._rare_adjusted_direction(p=W, common=common)
    extra = d - common
    assert abs(float((extra * common).sum())) < 1e-3 * float(common.norm() * extra.norm())
    assert float(extra.norm()) == pytest.approx(0.5 * float(common.norm()), rel=1e-4)     # cap fired
    tr = opt.scarcity_trace()
    assert tr["rare_macro_cap_fired"]["max"] == 1.0 and "cos_rare_common" in tr
    assert "cos_rare_common" not in opt.scarcity_trace()                                  # window was reset


def test_scopt_warmup_gates_and_scarcity_geometry():
    m = _model()
    cfg = scopt_optimizer_config(m, 0)
    name = "layers.0.core.in_proj.weight"
    assert cfg["matrix_scarcity_map"][name] == ("layers.0.core.in_proj.__out__", "layers.0.core.in_proj.__in__")
    assert cfg["recurrence_scarcity_map"] == {"layers.0.core.log_a": "layers.0.core.in_proj.__out__"}
    opt = ScarcityAwareOptimizer(m.parameters(), lr=0.02, warmup_steps=2, **cfg)
    opt.bind_param_names(m.named_parameters())
    opt.update_rare_grad_ema({name: torch.ones(16, 16)})
    assert "rare_grad_ema" not in opt.state[m.layers[0].core.in_proj.weight]     # writes closed in warm-up
    assert opt.update_row_pressure_ema(torch.tensor([1, 1, 3]), torch.tensor([2.0, 4.0, 6.0]), vocab_size=32) is None
    for s in range(2):
        _grads(m, s)
        opt.step()
    row = opt.update_row_pressure_ema(torch.tensor([1, 1, 3]), torch.tensor([2.0, 4.0, 6.0]), vocab_size=32, decay=0.5)
    assert row[1] == pytest.approx(1.5) and row[3] == pytest.approx(3.0) and row[0] == 0
    pres = torch.zeros(16)
    pres[:4] = 5.0
    opt.set_channel_pressure({"layers.0.core.in_proj.__out__": pres})
    _grads(m, 9)
    opt.step()
    assert opt._scarcity_enabled()
    d, out_f, in_f = opt._apply_matrix_scarcity(name, torch.ones(16, 16))
    assert in_f is None and out_f[:4].min() > 1.9 and torch.allclose(out_f[4:], torch.ones(12))
    assert torch.allclose(d[:4], out_f[:4].sqrt()[:, None].expand(4, 16))
    d2, rf = opt._apply_row_scarcity("embed.weight", torch.ones(32, 16))
    assert rf[3] > rf[1] > rf[0] == 1.0
    la = opt._apply_recurrence_scarcity("layers.0.core.log_a", torch.ones(16))
    assert la[0] > 1.9 and la[10] == 1.0
    tr = opt.scarcity_trace()
    assert tr["scarcity_enabled"] and "out_scarcity_max" in tr and tr["row_pressure"]["max"] == pytest.approx(3.0)


def test_pressure_baseline_and_allreduce_config():
    freq = torch.tensor([1000.0, 10.0, 1.0, 0.0])
    ce = torch.tensor([[2.0, 2.0, 2.0, 0.5]])
    tg = torch.tensor([[0, 1, 2, 1]])
    p = scarcity_pressure_from_ce(ce, tg, token_frequencies=freq, baseline=1.0)
    assert p[0, 3] == 0 and p[0, 2] > p[0, 1] > p[0, 0] > 0
    assert p[0, 0] == pytest.approx(1.0 / torch.log1p(torch.tensor(1000.0)).item())
    big = torch.cat([torch.ones(99), torch.tensor([1000.0])]).unsqueeze(0)
    clamped = scarcity_pressure_from_ce(big, torch.zeros(1, 100, dtype=torch.long), token_frequencies=torch.ones(1),
                                        upper_c=3.0, upper_floor=2.0)
    assert float(clamped.max()) == pytest.approx(2.0)
    with pytest.raises(ValueError):
        scarcity_pressure_from_ce(ce, tg[:, :2], token_frequencies=freq)
    fb = FrequencyBucketBaseline(torch.tensor([1.0, 1.0, 1e6, 1e6]), num_buckets=2, decay=0.5)
    fb.update(torch.tensor([4.0, 2.0, 1.0]), torch.tensor([0, 1, 2]))
    assert fb.baseline(torch.tensor([0, 3])).tolist() == [3.0, 1.0]
    fb.update(torch.tensor([1.0]), torch.tensor([1]))
    assert fb.baseline(torch.tensor([0])).item() == 2.0 and fb.state_dict()["num_buckets"] == 2
    assert scopt_allreduce_config(world_size=1, all_group=None).train_grad_scale == 1.0
    c = scopt_allreduce_config(world_size=4, all_group=object())
    assert c.train_rank_count == 3 and c.materialize_zeros and c.train_grad_scale == pytest.approx(1 / 3)
    assert scopt_allreduce_config(world_size=4, all_group=None).train_grad_scale == 0.25


def test_tier0_gates():
    def tr(step, out_med, cos, fp):
        return {"step": step, "scarcity_enabled": True, "out_scarcity": {"median": out_med},
                "cos_rare_common": {"median": cos}, "pressure_stats": {"fraction_positive": fp}}
    good = evaluate_tier0_gates([tr(100, 1.0, 0.0, 0.9), tr(250, 1.1, 0.4, 0.1), tr(300, 1.4, -0.5, 0.2)])
    assert [good[k]["status"] for k in good] == ["pass", "skip", "pass", "pass"]
    bad = evaluate_tier0_gates([tr(250, 1.1, 0.95, 0.5), tr(300, 1.1, 0.99, 0.6)])
    assert [bad[k]["status"] for k in bad] == ["fail", "skip", "fail", "fail"]
    assert "inert" in bad["0.3_rare_common_alignment"]["reason"] and "too dense" in bad["0.4_pressure_sparsity"]["reason"]
    assert evaluate_tier0_gates([])["0.4_pressure_sparsity"]["status"] == "skip"
    assert "0.1_signal_distribution: FAIL" in summarize_gates(bad)


# --------------------------------------------------------------------------- criticality
def test_future_energy_and_event_mask():
    s = torch.arange(1.0, 6.0).reshape(1, 5, 1)
    fe = compute_future_energy(s, 2)
    assert fe.reshape(-1).tolist() == [(4 + 9) / 2, (9 + 16) / 2, (16 + 25) / 2, 25.0, 0.0]
    assert torch.equal(compute_future_energy(s.expand(3, 2, 5, 1), 2)[1, 1], fe[0])       # leading dims broadcast
    with pytest.raises(ValueError):
        compute_future_energy(s, 0)
    p = torch.tensor([[0.1, -1.0, 3.0, 2.0, 0.0, 0.0]])
    assert compute_event_mask(p, 0.5).tolist() == [[True, False, True, True, False, False]]
    assert compute_event_mask(-p.abs(), 0.5).sum() == 0 and compute_event_mask(p, 0.0).sum() == 0


def test_criticality_accumulators_match_exact_bank_scoring():
    torch.manual_seed(0)
    cd = CriticalityDistillation(num_layers=2, dim=8, trace_ttl_steps=4, trace_half_life_steps=3.0,
                                 min_weighted_events_per_layer=0.5, criticality_budget_frac=0.25)
    for step in range(7):                                  # wraps the 4-slot ring
        states = [torch.randn(2, 12, 8) * (1 + l) for l in range(2)]
        cd.ingest_step(step=step, pressure=torch.rand(2, 12), states_per_layer=states, horizon_H=3, event_frac=0.25)
    assert (cd.bank_step >= 3).all() and bool(cd.baseline_initialized.all())
    exact = cd.score(current_step=6)
    fast = cd.score_from_accumulators()
    assert torch.allclose(exact, fast, atol=1e-5)
    w = torch.exp2(-(6 - cd.bank_step).float() / 3.0) * cd.bank_event_count
    assert torch.allclose(cd.event_mass, w.sum(1), atol=1e-4)
    cd.allocate_seats(current_step=6)
    a = cd.seat_mask.clone()
    cd.allocate_seats_from_accumulators(current_step=6)
    assert torch.equal(a, cd.seat_mask) and cd.seat_mask.sum(1).tolist() == [2, 2]
    assert torch.equal(cd.seat_mask[0].nonzero().reshape(-1).sort().values, exact[0].topk(2).indices.sort().values)
    # loss touches seated channels only
    las = [torch.zeros(8, requires_grad=True) for _ in range(2)]
    loss = cd.criticality_loss(las)
    loss.backward()
    assert float(loss.detach()) == pytest.approx(2 * (0.5 - 0.95) ** 2 * 1e-3, rel=1e-5)
    assert torch.equal(las[0].grad != 0, cd.seat_mask[0])
    snap = cd.diagnostics_snapshot(log_a_per_layer=[l.detach() for l in las], current_step=6)
    assert snap["seat_churn_per_layer"] == [0.0, 0.0] and snap["seat_mask_fraction_per_layer"] == [0.25, 0.25]
    assert len(snap["seat_indices_per_layer"][0]) == 2
    cd.seat_mask.zero_()
    assert cd.diagnostics_snapshot(log_a_per_layer=[l.detach() for l in las], current_step=7)["seat_churn_per_layer"] \
        == [1.0, 1.0]
    assert float(cd.criticality_loss(las)) == 0.0
    sd = copy.deepcopy(cd.state_dict())
    cd2 = CriticalityDistillation(num_layers=2, dim=8, trace_ttl_steps=4)
    cd2.load_state_dict(sd)
    assert torch.equal(cd2.bank_step, cd.bank_step)


def test_criticality_gates_and_fixed_seats():
    cd = CriticalityDistillation(num_layers=1, dim=8, min_weighted_events_per_layer=1e6)
    cd.ingest_step(step=0, pressure=torch.rand(1, 10), states_per_layer=[torch.randn(1, 10, 8)], horizon_H=2,
                   event_frac=0.3)
    cd.allocate_seats_from_accumulators(current_step=0)
    assert cd.seat_mask.sum() == 0                         # not enough evidence
    fx = CriticalityDistillation(num_layers=2, dim=20, fixed_random_seats=True, criticality_budget_frac=0.2)
    before = fx.seat_mask.clone()
    fx.allocate_seats(current_step=5)
    assert torch.equal(before, fx.seat_mask) and fx.seat_mask.sum(1).tolist() == [4, 4]
    with pytest.raises(ValueError):
        CriticalityDistillation(num_layers=1, dim=4, criticality_budget_frac=1.0)
    with pytest.raises(ValueError):
        cd.ingest_gpu(pressure=torch.rand(1, 4), states_per_layer=[], horizon_H=1, event_frac=0.5)
    cd.add_step_evidence(layer=0, step=3, evidence=torch.ones(8), event_count=2.0)
    with pytest.raises(IndexError):
        cd.add_step_evidence(layer=4, step=3, evidence=torch.ones(8), event_count=2.0)
