"""Per-channel-momentum Muon, one property per test (CPU)."""
import copy

import pytest
import torch
import torch.nn as nn

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim import SemanticOptimizer as ExportedSemantic
from chaoscontrol_b200.optim.muon import Muon, newton_schulz_orthogonalize
from chaoscontrol_b200.optim.semantic import SemanticOptimizer, default_beta_from_log_a, semantic_optimizer_config


class _Core(nn.Module):
    def __init__(self, d=6, dtype=torch.float32):
        super().__init__()
        torch.manual_seed(0)
        self.in_proj = nn.Linear(4, d, bias=True).to(dtype)          # [d, 4]: channels on axis 0
        self.out_proj = nn.Linear(d, 4, bias=False).to(dtype)        # [4, d]: channels on axis 1
        self.log_a = nn.Parameter(torch.linspace(-3, 3, d))


def _opt(m, **kw):
    base = dict(lr=0.1, momentum=0.9, momentum_min=0.5, a_param_name="log_a",
                channel_map={"in_proj.weight": 0, "out_proj.weight": 1})
    base.update(kw)
    o = SemanticOptimizer(m.parameters(), **base)
    o.bind_param_names(m.named_parameters())
    return o


def _ones(m):
    """Unit gradients everywhere except on ``log_a`` (which would move the betas between steps)."""
    for n, p in m.named_parameters():
        p.grad = None if n == "log_a" else torch.ones_like(p)


def test_package_exports_the_optimizer():
    assert ExportedSemantic is SemanticOptimizer


def test_beta_is_monotone_bounded_detached_and_fp32():
    la = torch.linspace(-20, 20, 9, dtype=torch.bfloat16, requires_grad=True)
    b = default_beta_from_log_a(la, beta_min=0.5, beta_max=0.95)
    assert b.dtype == torch.float32 and not b.requires_grad
    assert bool((b[1:] >= b[:-1]).all()) and float(b.min()) >= 0.5 and float(b.max()) <= 0.95
    assert float(b[0]) == pytest.approx(0.5, abs=1e-3) and float(b[-1]) == pytest.approx(0.95, abs=1e-3)


def test_uncoupled_optimizer_matches_muon_on_a_single_matrix():
    torch.manual_seed(0)
    a, b = nn.Parameter(torch.randn(6, 4)), None
    b = nn.Parameter(a.detach().clone())
    oa = SemanticOptimizer([a], lr=0.05, momentum=0.9)
    ob = Muon([b], lr=0.05, momentum=0.9)
    for s in range(3):
        g = torch.randn(6, 4, generator=torch.Generator().manual_seed(s))
        a.grad, b.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    assert torch.allclose(a, b, atol=1e-6)


def test_row_axis_decay_follows_beta_per_channel():
    m = _Core()
    o = _opt(m)
    beta = o.current_beta_vec()
    for _ in range(3):
        _ones(m)
        o.step()
    want = 1.0 + beta + beta * beta                                        # buf after three unit gradients
    assert torch.allclose(o.state[m.in_proj.weight]["momentum_buffer"], want.view(-1, 1).expand(6, 4), atol=1e-6)
    assert torch.allclose(o.state[m.out_proj.weight]["momentum_buffer"], want.view(1, -1).expand(4, 6), atol=1e-6)


def test_negative_axis_resolves_like_the_positive_one():
    m1, m2 = _Core(), _Core()
    o1 = _opt(m1, channel_map={"out_proj.weight": 1})
    o2 = _opt(m2, channel_map={"out_proj.weight": -1})
    for o, m in ((o1, m1), (o2, m2)):
        _ones(m)
        o.step()
    assert torch.equal(m1.out_proj.weight, m2.out_proj.weight)


def test_nesterov_uses_the_tensor_beta_in_the_lookahead():
    m = _Core()
    o = _opt(m, nesterov=True, lr=1.0)
    w0 = m.in_proj.weight.detach().clone()
    g = torch.randn(6, 4, generator=torch.Generator().manual_seed(1))
    for p in m.parameters():
        p.grad = torch.zeros_like(p)
    m.in_proj.weight.grad = g.clone()
    o.step()
    beta = o.current_beta_vec().view(-1, 1)
    want = newton_schulz_orthogonalize(g + beta * g)                       # buf = g after the first step
    scale = max(1.0, 6 / 4) ** 0.5
    assert torch.allclose(w0 - m.in_proj.weight.detach(), scale * want, atol=1e-5)


def test_channel_count_mismatch_raises_at_step():
    m = _Core()
    o = _opt(m, channel_map={"in_proj.weight": 1})                         # axis 1 has 4 entries, beta has 6
    _ones(m)
    with pytest.raises(ValueError, match="channels"):
        o.step()
    with pytest.raises(ValueError, match="out of range"):
        SemanticOptimizer._broadcast_beta(torch.ones(3), torch.Size([3, 3]), 5)


def test_binding_checks_names():
    m = _Core()
    with pytest.raises(ValueError, match="not found"):
        _opt(m, a_param_name="missing")
    with pytest.raises(ValueError, match="channel_map names"):
        _opt(m, channel_map={"nope.weight": 0})
    o = SemanticOptimizer([m.in_proj.weight], a_param_name="log_a")        # log_a exists but is not optimised here
    with pytest.raises(ValueError, match="not in any param_group"):
        o.bind_param_names(m.named_parameters())


def test_step_without_binding_raises_and_a_in_channel_map_is_refused():
    m = _Core()
    o = SemanticOptimizer(m.parameters(), a_param_name="log_a")
    _ones(m)
    with pytest.raises(RuntimeError, match="bind_param_names"):
        o.step()
    with pytest.raises(ValueError, match="cannot be in channel_map"):
        SemanticOptimizer(m.parameters(), a_param_name="log_a", channel_map={"log_a": 0})


@pytest.mark.parametrize("kw", [dict(lr=0.0), dict(ns_steps=0), dict(momentum=1.0), dict(momentum=0.4, momentum_min=0.5),
                                dict(momentum_min=-0.1)])
def test_bad_hyperparameters_are_refused(kw):
    with pytest.raises(ValueError):
        SemanticOptimizer([nn.Parameter(torch.zeros(2, 2))], **kw)


def test_vectors_take_the_adamw_branch_like_muon():
    torch.manual_seed(0)
    a = nn.Parameter(torch.randn(5))
    b = nn.Parameter(a.detach().clone())
    oa = SemanticOptimizer([a], lr=0.01, weight_decay=0.1)
    ob = torch.optim.AdamW([b], lr=0.01, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for s in range(4):
        g = torch.randn(5, generator=torch.Generator().manual_seed(s))
        a.grad, b.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    assert torch.allclose(a, b, atol=1e-6)


def test_a_parameter_without_gradient_leaves_its_buffers_alone():
    m = _Core()
    o = _opt(m)
    _ones(m)
    o.step()
    buf = o.state[m.in_proj.weight]["momentum_buffer"].clone()
    w = m.in_proj.weight.detach().clone()
    for p in m.parameters():
        p.grad = None
    m.out_proj.weight.grad = torch.ones_like(m.out_proj.weight)
    o.step()
    assert torch.equal(o.state[m.in_proj.weight]["momentum_buffer"], buf) and torch.equal(m.in_proj.weight, w)


def test_bf16_matrices_get_fp32_buffers_only_when_coupled():
    m = _Core(dtype=torch.bfloat16)
    o = _opt(m)
    _ones(m)
    o.step()
    assert o.state[m.in_proj.weight]["momentum_buffer"].dtype == torch.float32
    assert m.in_proj.weight.dtype == torch.bfloat16
    p = nn.Parameter(torch.randn(4, 4).bfloat16())
    plain = SemanticOptimizer([p], lr=0.1)
    p.grad = torch.ones_like(p)
    plain.step()
    assert plain.state[p]["momentum_buffer"].dtype == torch.bfloat16


def test_resume_from_state_dict_gives_identical_updates():
    m1 = _Core()
    o1 = _opt(m1)
    for s in range(2):
        for p in m1.parameters():
            p.grad = torch.randn(p.shape, generator=torch.Generator().manual_seed(s))
        o1.step()
    m2 = copy.deepcopy(m1)
    o2 = _opt(m2)
    o2.load_state_dict(copy.deepcopy(o1.state_dict()))
    for m, o in ((m1, o1), (m2, o2)):
        for p in m.parameters():
            p.grad = torch.randn(p.shape, generator=torch.Generator().manual_seed(9))
        o.step()
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(a, b)


def test_param_groups_keep_their_own_learning_rates():
    m = _Core()
    groups = [{"params": [m.in_proj.weight], "lr": 1.0}, {"params": [m.out_proj.weight], "lr": 0.0001},
              {"params": [m.in_proj.bias, m.log_a]}]
    o = SemanticOptimizer(groups, lr=0.1, a_param_name="log_a", channel_map={"in_proj.weight": 0, "out_proj.weight": 1})
    o.bind_param_names(m.named_parameters())
    w_in, w_out = m.in_proj.weight.detach().clone(), m.out_proj.weight.detach().clone()
    _ones(m)
    o.step()
    assert float((m.in_proj.weight.detach() - w_in).norm()) > 1000 * float((m.out_proj.weight.detach() - w_out).norm())


def test_trace_follows_log_a_and_is_absent_without_it():
    m = _Core()
    o = _opt(m)
    t0 = o.beta_trace()
    assert t0["beta_vec"].shape == (6,) and t0["tau_steps"].shape == (6,) and t0["beta_min"] < t0["beta_mean"] < t0["beta_max"]
    with torch.no_grad():
        m.log_a.fill_(10.0)
    t1 = o.beta_trace()
    assert t1["beta_min"] == pytest.approx(0.9, abs=1e-3) and float(t1["tau_steps"][0]) == pytest.approx(-1 / torch.log(torch.tensor(0.9)).item(), rel=1e-3)
    plain = SemanticOptimizer([nn.Parameter(torch.zeros(2, 2))])
    assert plain.beta_trace() is None and plain.current_beta_vec() is None


def test_config_helper_lists_the_coupled_matrices_of_a_block():
    model = CareStudentLM(vocab_size=32, dim=16, num_layers=2)
    cfg = semantic_optimizer_config(model, 1)
    assert cfg["a_param_name"] == "layers.1.core.log_a"
    assert all(k.startswith("layers.1.core.") for k in cfg["channel_map"]) and cfg["channel_map"]["layers.1.core.in_proj.weight"] == 0
    with pytest.raises(ValueError):
        semantic_optimizer_config(model, 7)


def test_toy_regression_loss_goes_down():
    torch.manual_seed(0)
    m = _Core()
    o = _opt(m, lr=0.02)
    x, y = torch.randn(64, 4), torch.randn(64, 4)
    first = last = None
    for _ in range(40):
        h = torch.tanh(m.in_proj(x)) * torch.sigmoid(m.log_a)
        loss = (m.out_proj(h) - y).pow(2).mean()
        o.zero_grad()
        loss.backward()
        o.step()
        first, last = (float(loss.detach()) if first is None else first), float(loss.detach())
    assert last < first
