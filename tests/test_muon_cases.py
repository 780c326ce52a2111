"""Muon: Newton-Schulz bounds, matrix / AdamW routing, research knobs, state, toy training (CPU)."""
import copy

import pytest
import torch
import torch.nn as nn

from chaoscontrol_b200.optim.muon import Muon, newton_schulz_orthogonalize


def _sv(x):
    return torch.linalg.svdvals(x.float())


# ---------------------------------------------------------------- Newton-Schulz
@pytest.mark.parametrize("shape", [(16, 16), (8, 32), (32, 8)])
def test_ns_singular_values_land_in_the_quintic_band(shape):
    torch.manual_seed(0)
    s = _sv(newton_schulz_orthogonalize(torch.randn(*shape), steps=5))
    assert float(s.max()) < 1.3 and float(s.min()) > 0.3 and s.numel() == min(shape)


def test_ns_keeps_shape_dtype_policy_and_batches_like_singles():
    torch.manual_seed(0)
    g = torch.randn(3, 8, 12)
    out = newton_schulz_orthogonalize(g, steps=5)
    assert out.shape == g.shape and out.dtype == torch.float32
    for i in range(3):
        assert torch.allclose(out[i], newton_schulz_orthogonalize(g[i], steps=5), atol=1e-5)
    assert newton_schulz_orthogonalize(g[0].double(), compute_dtype=torch.float64).dtype == torch.float64


def test_ns_is_scale_invariant_and_sign_equivariant():
    torch.manual_seed(0)
    g = torch.randn(8, 8)
    a = newton_schulz_orthogonalize(g)
    assert torch.allclose(a, newton_schulz_orthogonalize(g * 1000.0), atol=1e-4)
    assert torch.allclose(-a, newton_schulz_orthogonalize(-g), atol=1e-6)


def test_ns_zero_input_stays_finite():
    assert torch.isfinite(newton_schulz_orthogonalize(torch.zeros(4, 6))).all()


def test_ns_tall_equals_transposed_wide():
    torch.manual_seed(0)
    g = torch.randn(24, 6)
    assert torch.allclose(newton_schulz_orthogonalize(g), newton_schulz_orthogonalize(g.T).T, atol=1e-5)


# ---------------------------------------------------------------- matrix path
def test_first_matrix_step_is_lr_times_orthogonalised_nesterov_direction():
    torch.manual_seed(0)
    p = nn.Parameter(torch.randn(8, 8))
    g = torch.randn(8, 8)
    p0 = p.detach().clone()
    opt = Muon([p], lr=0.1, momentum=0.9)
    p.grad = g.clone()
    opt.step()
    want = newton_schulz_orthogonalize(g + 0.9 * g, steps=5)             # buf = g, direction = g + mu * buf
    assert torch.allclose(p0 - p.detach(), 0.1 * want, atol=1e-6)


def test_non_nesterov_uses_the_buffer_itself():
    torch.manual_seed(0)
    p = nn.Parameter(torch.randn(6, 6))
    g1, g2 = torch.randn(6, 6), torch.randn(6, 6)
    opt = Muon([p], lr=0.1, momentum=0.5, nesterov=False)
    p.grad = g1.clone()
    opt.step()
    before = p.detach().clone()
    p.grad = g2.clone()
    opt.step()
    assert torch.allclose(before - p.detach(), 0.1 * newton_schulz_orthogonalize(0.5 * g1 + g2), atol=1e-6)


@pytest.mark.parametrize("shape,scale", [((32, 8), 2.0), ((8, 32), 1.0), ((8, 8), 1.0)])
def test_rectangular_scale_is_sqrt_of_rows_over_cols_floored_at_one(shape, scale):
    torch.manual_seed(0)
    p = nn.Parameter(torch.zeros(*shape))
    g = torch.randn(*shape)
    opt = Muon([p], lr=1.0, momentum=0.0)
    p.grad = g.clone()
    opt.step()
    assert torch.allclose(-p.detach(), scale * newton_schulz_orthogonalize(g), atol=1e-5)


def test_weight_decay_is_decoupled():
    p = nn.Parameter(torch.ones(4, 4))
    opt = Muon([p], lr=0.1, momentum=0.0, weight_decay=0.5)
    p.grad = torch.zeros(4, 4)
    opt.step()
    assert torch.allclose(p.detach(), torch.full((4, 4), 0.95), atol=1e-6)


def test_params_without_grad_are_skipped():
    a, b = nn.Parameter(torch.ones(4, 4)), nn.Parameter(torch.ones(4))
    opt = Muon([a, b], lr=0.1)
    opt.step()
    assert torch.equal(a.detach(), torch.ones(4, 4)) and len(opt.state) == 0


# ---------------------------------------------------------------- AdamW side
@pytest.mark.parametrize("wd", [0.0, 0.1])
def test_vector_params_match_torch_adamw_over_several_steps(wd):
    torch.manual_seed(0)
    a = nn.Parameter(torch.randn(10))
    b = nn.Parameter(a.detach().clone())
    mu = Muon([a], lr=0.01, adamw_lr=0.01, adamw_betas=(0.9, 0.95), adamw_eps=1e-8, adamw_weight_decay=wd)
    ref = torch.optim.AdamW([b], lr=0.01, betas=(0.9, 0.95), eps=1e-8, weight_decay=wd)
    for _ in range(5):
        g = torch.randn(10)
        a.grad, b.grad = g.clone(), g.clone()
        mu.step()
        ref.step()
    assert torch.allclose(a, b, atol=1e-6)


def test_adamw_lr_and_decay_default_to_the_matrix_values():
    opt = Muon([nn.Parameter(torch.zeros(3))], lr=0.03, weight_decay=0.2)
    g = opt.param_groups[0]
    assert g["adamw_lr"] == 0.03 and g["adamw_weight_decay"] == 0.2
    opt2 = Muon([nn.Parameter(torch.zeros(3))], lr=0.03, weight_decay=0.2, adamw_lr=0.001, adamw_weight_decay=0.0)
    assert opt2.param_groups[0]["adamw_lr"] == 0.001 and opt2.param_groups[0]["adamw_weight_decay"] == 0.0


# ---------------------------------------------------------------- routing
def _named(model):
    return list(model.named_parameters())


def test_default_rule_two_d_is_matrix_except_delta_projections():
    m = nn.ModuleDict({"lin": nn.Linear(4, 4, bias=True),
                       "core": nn.ModuleDict({"delta_proj": nn.Linear(4, 4, bias=False)})})
    opt = Muon(m.parameters(), lr=0.1)
    opt.bind_param_names(_named(m))
    for p in m.parameters():
        p.grad = torch.ones_like(p)
    opt.step()
    st = {n: set(opt.state[p]) for n, p in m.named_parameters()}
    assert "momentum_buffer" in st["lin.weight"] and "exp_avg" in st["lin.bias"] and "exp_avg" in st["core.delta_proj.weight"]


def test_name_set_overrides_the_rule_and_empty_set_means_no_matrices():
    m = nn.Linear(4, 4)
    for names, key in (({"bias"}, "exp_avg"), (set(), "exp_avg"), ({"weight"}, "momentum_buffer")):
        opt = Muon(m.parameters(), lr=0.1, matrix_param_names=names)
        opt.bind_param_names(_named(m))
        m.weight.grad, m.bias.grad = torch.ones(4, 4), torch.ones(4)
        if names == {"bias"}:
            continue                                                # a vector cannot take the matrix path; routing only
        opt.step()
        assert key in opt.state[m.weight]


def test_custom_predicate_routes_parameters():
    m = nn.Linear(4, 4)
    opt = Muon(m.parameters(), lr=0.1, is_matrix=lambda p, name: False)
    m.weight.grad, m.bias.grad = torch.ones(4, 4), torch.ones(4)
    opt.step()
    assert "exp_avg" in opt.state[m.weight] and opt.ns_calls == 0


@pytest.mark.parametrize("kw", [dict(lr=0.0), dict(lr=-1.0), dict(ns_steps=0), dict(momentum=1.0), dict(momentum=-0.1),
                                dict(log_a_beta_min=1.0), dict(log_a_beta_ema=1.0)])
def test_bad_hyperparameters_are_refused(kw):
    with pytest.raises(ValueError):
        Muon([nn.Parameter(torch.zeros(2, 2))], **kw)


# ---------------------------------------------------------------- fused path
class _Toy(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.a, self.b, self.c = nn.Linear(8, 8), nn.Linear(8, 8), nn.Linear(8, 4)
        self.scale = nn.Parameter(torch.ones(4))

    def forward(self, x):
        return self.c(torch.tanh(self.b(torch.tanh(self.a(x))))) * self.scale


def _train(opt_kw, steps=4, seed=1):
    m = _Toy()
    opt = Muon(m.parameters(), lr=0.05, **opt_kw)
    opt.bind_param_names(_named(m))
    g = torch.Generator().manual_seed(seed)
    losses = []
    for _ in range(steps):
        x, y = torch.randn(16, 8, generator=g), torch.randn(16, 4, generator=g)
        loss = (m(x) - y).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return m, opt, losses


def test_fused_matches_plain_and_runs_one_ns_per_shape_group():
    m1, o1, _ = _train(dict(fused=False))
    m2, o2, _ = _train(dict(fused=True))
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(a, b, atol=1e-5)
    assert o1.ns_calls == 3 * 4 and o2.ns_calls == 2 * 4            # shapes (8, 8) x 2 and (4, 8)


def test_fused_state_dict_has_the_plain_layout():
    _, o1, _ = _train(dict(fused=False), steps=1)
    _, o2, _ = _train(dict(fused=True), steps=1)
    s1, s2 = o1.state_dict()["state"], o2.state_dict()["state"]
    assert {k: sorted(v) for k, v in s1.items()} == {k: sorted(v) for k, v in s2.items()}


def test_training_is_deterministic_and_reduces_the_loss():
    _, _, l1 = _train(dict(), steps=12)
    _, _, l2 = _train(dict(), steps=12)
    assert l1 == l2
    m = _Toy()
    opt = Muon(m.parameters(), lr=0.05)
    x, y = torch.randn(32, 8), torch.randn(32, 4)
    first = last = None
    for _ in range(30):
        loss = (m(x) - y).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        first, last = (float(loss.detach()) if first is None else first), float(loss.detach())
    assert last < 0.7 * first


def test_state_dict_round_trip_continues_identically():
    m1, o1, _ = _train(dict(), steps=3)
    m2 = copy.deepcopy(m1)
    o2 = Muon(m2.parameters(), lr=0.05)
    o2.bind_param_names(_named(m2))
    o2.load_state_dict(copy.deepcopy(o1.state_dict()))
    x, y = torch.randn(8, 8), torch.randn(8, 4)
    for m, o in ((m1, o1), (m2, o2)):
        o.zero_grad()
        (m(x) - y).pow(2).mean().backward()
        o.step()
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(a, b)


# ---------------------------------------------------------------- plasticity budget
class _Core(nn.Module):
    def __init__(self, d=4):
        super().__init__()
        self.in_proj, self.out_proj = nn.Linear(d, d, bias=False), nn.Linear(d, d, bias=False)
        self.log_a = nn.Parameter(torch.zeros(d))


class _Layered(nn.Module):
    def __init__(self, d=4):
        super().__init__()
        self.layers = nn.ModuleList([nn.ModuleDict({"core": _Core(d), "ff": nn.Linear(d, d, bias=False)})])


def test_budget_maps_to_rows_columns_and_vectors_of_core_parameters_only():
    m = _Layered()
    opt = Muon(m.parameters(), lr=0.1)
    opt.bind_param_names(_named(m))
    opt.set_plasticity_budget(torch.tensor([0.0, 1.0, 0.5, 0.0]), strength=1.0, step=3)
    core = m.layers[0]["core"]
    assert opt._plasticity_multiplier_for(core.in_proj.weight).shape == (4, 1)
    assert opt._plasticity_multiplier_for(core.out_proj.weight).shape == (1, 4)
    assert opt._plasticity_multiplier_for(core.log_a).tolist() == [1.0, 2.0, 1.5, 1.0]
    assert opt._plasticity_multiplier_for(m.layers[0]["ff"].weight) is None
    tr = opt.plasticity_budget_trace()
    assert tr["enabled"] and tr["step"] == 3 and tr["dim"] == 4 and tr["lr_multiplier_max"] == 2.0
    assert tr["top_channels"][0] == 1 and tr["budget_nonzero_fraction"] == 0.5


def test_budget_scales_the_log_a_update_per_channel():
    def run(budget):
        m = _Layered()
        with torch.no_grad():
            for p in m.parameters():
                p.zero_()
        opt = Muon(m.parameters(), lr=0.1, adamw_lr=0.1)
        opt.bind_param_names(_named(m))
        if budget is not None:
            opt.set_plasticity_budget(budget, strength=1.0)
        m.layers[0]["core"].log_a.grad = torch.ones(4)
        opt.step()
        return m.layers[0]["core"].log_a.detach().clone()
    base, scaled = run(None), run(torch.tensor([0.0, 1.0, 0.5, 0.0]))
    assert torch.allclose(scaled / base, torch.tensor([1.0, 2.0, 1.5, 1.0]), atol=1e-5)


def test_budget_views_are_cached_per_device_and_dtype_and_cleared_on_update():
    m = _Layered()
    opt = Muon(m.parameters(), lr=0.1)
    opt.bind_param_names(_named(m))
    opt.set_plasticity_budget(torch.ones(4))
    core = m.layers[0]["core"]
    a = opt._plasticity_multiplier_for(core.log_a)
    b = opt._plasticity_multiplier_for(core.log_a)
    assert a.data_ptr() == b.data_ptr() and len(opt._plasticity_multiplier_views) == 1
    opt.set_plasticity_budget(torch.zeros(4))
    assert len(opt._plasticity_multiplier_views) == 0
    with pytest.raises(ValueError, match="confidence"):
        opt.set_plasticity_budget(torch.ones(4), confidence=torch.ones(3))
    assert Muon([nn.Parameter(torch.zeros(2))], lr=0.1).plasticity_budget_trace()["enabled"] is False


# ---------------------------------------------------------------- log_a beta coupling
def test_log_a_beta_follows_a_slow_ema_of_the_parameter():
    m = _Layered()
    core = m.layers[0]["core"]
    with torch.no_grad():
        core.log_a.copy_(torch.tensor([-4.0, 0.0, 4.0, 0.0]))
    opt = Muon(m.parameters(), lr=0.1, adamw_betas=(0.9, 0.95), log_a_beta_coupling=True, log_a_beta_min=0.5,
               log_a_beta_ema=0.5)
    opt.bind_param_names(_named(m))
    core.log_a.grad = torch.zeros(4)
    opt.step()
    want = 0.5 + 0.4 * torch.sigmoid(torch.tensor([-4.0, 0.0, 4.0, 0.0]))
    tr = opt.ssm_role_trace()
    assert tr["log_a_beta_updates"] == 1 and tr["log_a_beta_min"] == pytest.approx(float(want.min()), abs=1e-6)
    assert tr["log_a_beta_max"] == pytest.approx(float(want.max()), abs=1e-6)
    st = opt.state[core.log_a]
    assert torch.allclose(st["log_a_slow_ema"], torch.tensor([-4.0, 0.0, 4.0, 0.0]))
    with torch.no_grad():
        core.log_a.fill_(2.0)
    core.log_a.grad = torch.zeros(4)
    opt.step()
    assert torch.allclose(st["log_a_slow_ema"], 0.5 * torch.tensor([-4.0, 0.0, 4.0, 0.0]) + 1.0)   # EMA moves first


def test_log_a_beta_coupling_off_is_plain_adamw_and_only_touches_log_a():
    m = _Layered()
    opt = Muon(m.parameters(), lr=0.1, log_a_beta_coupling=True)
    opt.bind_param_names(_named(m))
    for p in m.parameters():
        p.grad = torch.ones_like(p)
    opt.step()
    assert "log_a_slow_ema" in opt.state[m.layers[0]["core"].log_a]
    assert all("log_a_slow_ema" not in opt.state[p] for n, p in m.named_parameters() if not n.endswith("log_a"))
    off = Muon([nn.Parameter(torch.zeros(3))], lr=0.1)
    assert off.ssm_role_trace()["log_a_beta_coupling"] is False and off.ssm_role_trace()["log_a_beta_updates"] == 0
