"""Optimizers on CPU: Muon NS isometry and AdamW-fallback parity, fused vs plain
step parity, one NS call per shape group, LAMB == Adam at trust ratio 1, param
grouping, momentum warm-up, weight EMA."""
import copy

import pytest
import torch

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim import (LAMB, Muon, WeightEMA, apply_momentum_warmup,
                                     build_optimizer_params, classify_param, eval_with_ema,
                                     newton_schulz_orthogonalize, wrap_optimizer_step)


@pytest.mark.parametrize("shape", [(32, 32), (48, 16), (16, 48), (3, 24, 24)])
def test_newton_schulz_near_isometry(shape):
    torch.manual_seed(0)
    g = torch.randn(*shape)
    o = newton_schulz_orthogonalize(g, steps=5)
    assert o.shape == g.shape
    sv = torch.linalg.svdvals(o.reshape(-1, *shape[-2:])[0])
    assert sv.max() < 1.3 and sv.median() > 0.5


def test_muon_adamw_fallback_matches_torch_adamw():
    torch.manual_seed(0)
    p1 = torch.nn.Parameter(torch.randn(10))
    p2 = torch.nn.Parameter(p1.detach().clone())
    o1 = Muon([p1], lr=0.01, weight_decay=0.1, adamw_betas=(0.9, 0.95), adamw_eps=1e-8)
    o2 = torch.optim.AdamW([p2], lr=0.01, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8)
    for _ in range(5):
        g = torch.randn(10)
        p1.grad, p2.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    assert torch.allclose(p1, p2, atol=1e-6)


def test_muon_fused_equals_plain_and_one_ns_per_shape():
    torch.manual_seed(1)
    m1 = CareStudentLM(vocab_size=32, dim=16, num_layers=2)
    m2 = copy.deepcopy(m1)
    o1 = Muon(m1.parameters(), lr=0.02, weight_decay=0.01)
    o2 = Muon(m2.parameters(), lr=0.02, weight_decay=0.01, fused=True)
    o1.bind_param_names(m1.named_parameters())
    o2.bind_param_names(m2.named_parameters())
    for _ in range(3):
        for p, q in zip(m1.parameters(), m2.parameters()):
            g = torch.randn_like(p)
            p.grad, q.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    for (n, p), (_, q) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(p, q, atol=1e-5), n
    shapes = {tuple(p.shape) for n, p in m2.named_parameters() if p.ndim == 2 and "delta_proj" not in n}
    assert o2.ns_calls == 3 * len(shapes)
    # delta_proj is excluded from the matrix path; state layout matches between the paths
    for n, p in m2.named_parameters():
        st = o2.state[p]
        assert ("momentum_buffer" in st) == (p.ndim == 2 and "delta_proj" not in n), n
    assert set(o1.state_dict()["state"][0]) == set(o2.state_dict()["state"][0])


def test_muon_empty_matrix_name_set_routes_everything_to_adamw():
    p = torch.nn.Parameter(torch.randn(8, 8))
    o = Muon([p], lr=0.01, matrix_param_names=set())
    o.bind_param_names([("w", p)])
    p.grad = torch.randn(8, 8)
    o.step()
    assert "exp_avg" in o.state[p] and "momentum_buffer" not in o.state[p]
    with pytest.raises(ValueError):
        Muon([p], lr=-1)


def test_lamb_trust_ratio_one_equals_adam():
    torch.manual_seed(2)
    p1 = torch.nn.Parameter(torch.randn(6, 5))
    p2 = torch.nn.Parameter(p1.detach().clone())
    o1 = LAMB([p1], lr=0.01, betas=(0.9, 0.999), eps=1e-8, trust_ratio_override=1.0)
    o2 = torch.optim.Adam([p2], lr=0.01, betas=(0.9, 0.999), eps=1e-8)
    for _ in range(4):
        g = torch.randn(6, 5)
        p1.grad, p2.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    assert torch.allclose(p1, p2, atol=1e-5)
    # trust ratio clips and skips 1-D tensors
    assert float(LAMB._trust_ratio(torch.tensor(100.0), torch.tensor(1.0), trust_clip=10.0)) == 10.0
    assert float(LAMB._trust_ratio(torch.tensor(0.0), torch.tensor(1.0), trust_clip=10.0)) == 1.0


def test_param_groups():
    m = CareStudentLM(vocab_size=16, dim=8, num_layers=1)
    names = dict(m.named_parameters())
    assert classify_param("layers.0.core.log_a", names["layers.0.core.log_a"]) == "dynamics"
    assert classify_param("final_norm.weight", names["final_norm.weight"]) == "no_decay"
    assert classify_param("lm_head.weight", names["lm_head.weight"]) == "main"
    groups = build_optimizer_params(m.named_parameters(), grouping="ssm_three_group", base_lr=0.1,
                                    weight_decay=0.01)
    by = {g["name"]: g for g in groups}
    assert by["dynamics"]["lr"] == pytest.approx(0.01) and by["dynamics"]["weight_decay"] == 0.0
    assert by["main"]["adamw_weight_decay"] == 0.01 and by["no_decay"]["weight_decay"] == 0.0
    flat = build_optimizer_params(m.named_parameters(), grouping="flat", base_lr=0.1, weight_decay=0.0)
    assert len(flat) == len(list(m.parameters()))
    with pytest.raises(ValueError):
        build_optimizer_params(m.named_parameters(), grouping="typo", base_lr=0.1, weight_decay=0.0)


def test_momentum_warmup_ema_and_wrapper():
    m = CareStudentLM(vocab_size=16, dim=8, num_layers=1)
    o = Muon(m.parameters(), lr=0.01)
    assert apply_momentum_warmup(o, step=0, target=0.99, start=0.9, steps=10) == pytest.approx(0.9)
    assert apply_momentum_warmup(o, step=5, target=0.99, start=0.9, steps=10) == pytest.approx(0.945)
    assert apply_momentum_warmup(o, step=50, target=0.99, start=0.9, steps=0) == pytest.approx(0.99)
    wrap_optimizer_step(o, model=m, target_momentum=0.95, warmup_start=0.85, warmup_steps=2,
                        weight_ema_decay=0.5, is_rank_zero=True)
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    for _ in range(3):
        for p in m.parameters():
            p.grad = torch.ones_like(p) * 0.1
        o.step()
    assert o._momentum_warmup_step == 3 and o.param_groups[0]["momentum"] == pytest.approx(0.95)
    ema: WeightEMA = o._weight_ema
    cur = m.lm_head.weight.detach().clone()
    with ema.applied(m):
        inside = m.lm_head.weight.detach().clone()
        assert not torch.equal(inside, cur)
    assert torch.equal(m.lm_head.weight, cur)            # restored
    # shadow lies between the initial and current weights
    assert (inside - before["lm_head.weight"]).abs().max() <= (cur - before["lm_head.weight"]).abs().max() + 1e-6
    assert eval_with_ema(m, None, lambda: 7) == 7
    with pytest.raises(ValueError):
        WeightEMA(m, decay=1.0)
