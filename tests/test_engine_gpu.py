"""Kernel training engine on the GPU vs autograd through the fp32 module, and
the arena Muon path vs the plain per-parameter path."""
import copy

import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200.engine import TrainEngine
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.ops import _lib
from chaoscontrol_b200.optim.muon import Muon, newton_schulz_orthogonalize
from chaoscontrol_b200.train_ssm import train_ssm_step
from chaoscontrol_b200.utils.arena import ParamArena

pytestmark = pytest.mark.gpu


def _model(vocab=512, layers=2, seed=0, dim=256, ff_mult=2):
    torch.manual_seed(seed)
    m = CareStudentLM(vocab_size=vocab, dim=dim, num_layers=layers, ff_mult=ff_mult)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("norm.weight"):
                p.uniform_(0.7, 1.3)
            if n.endswith("log_a"):
                p.normal_()
    return m


@pytest.mark.parametrize("dim,ff_mult", [(256, 2), (512, 4), (128, 2)])
def test_engine_step_vs_fp32_autograd(dim, ff_mult):
    ref = _model(dim=dim, ff_mult=ff_mult).cuda()
    m = copy.deepcopy(ref).to(torch.bfloat16)
    # the fp32 oracle uses the bf16-rounded weights
    with torch.no_grad():
        for p, q in zip(ref.parameters(), m.parameters()):
            p.copy_(q.float())
    tok = torch.randint(0, 512, (4, 129), device="cuda")
    inp, tgt = tok[:, :-1], tok[:, 1:]
    out = ref(inp)
    loss_ref = F.cross_entropy(out["logits"].reshape(-1, 512), tgt.reshape(-1))
    loss_ref.backward()
    arena = ParamArena.install(m)
    assert TrainEngine.supported(m)
    eng = TrainEngine(m, arena)
    loss = eng.step(inp, tgt)
    _lib.assert_ok()
    assert abs(float(loss) - float(loss_ref.detach())) < 0.03
    for n, p in ref.named_parameters():
        g, r = arena.grad_view(n), p.grad
        scale = r.abs().max().item()
        err = (g - r).abs().max().item()
        assert err <= 0.06 * scale + 2e-5, (n, err, scale)


def test_kernel_trunk_encode_matches_module_path():
    m = _model(seed=1).cuda().to(torch.bfloat16)
    tok = torch.randint(0, 512, (3, 64), device="cuda")
    assert m.kernel_trunk_supported()
    h0 = [torch.randn(3, 256, device="cuda") for _ in m.layers]
    hid, fin = m.encode(tok, initial_states=h0, return_final_states=True)
    ref = _model(seed=1).cuda()
    with torch.no_grad():
        for p, q in zip(ref.parameters(), m.parameters()):
            p.copy_(q.float())
    rh, rf = ref.encode(tok, initial_states=h0, return_final_states=True)
    assert (hid.float() - rh).abs().max().item() < 0.06 * rh.abs().max().item()
    for a, b in zip(fin, rf):
        assert torch.allclose(a.float(), b, rtol=5e-2, atol=5e-2)
    _lib.assert_ok()


def test_train_ssm_step_engine_and_autograd_paths_agree():
    m1 = _model(seed=2).cuda().to(torch.bfloat16)
    m2 = copy.deepcopy(m1)
    ParamArena.install(m1)
    tok = torch.randint(0, 512, (4, 65), device="cuda")
    l1 = train_ssm_step(m1, tok[:, :-1], tok[:, 1:], 16, lm_head_backward_mode="fused")
    l2 = train_ssm_step(m2, tok[:, :-1], tok[:, 1:], 16, lm_head_backward_mode="fused")
    _lib.assert_ok()
    assert abs(float(l1) - float(l2)) < 0.02
    for (n, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        a, b = p1.grad.float(), p2.grad.float()
        s = b.abs().max().item()
        assert (a - b).abs().max().item() <= 0.08 * s + 2e-5, n


@pytest.mark.parametrize("shape", [(256, 256), (512, 256), (256, 512), (2048, 256)])
def test_newton_schulz_kernel_vs_torch(shape):
    torch.manual_seed(0)
    g = torch.randn(3, *shape, device="cuda")
    got = newton_schulz_orthogonalize(g).float()
    ref = newton_schulz_orthogonalize(g.cpu(), compute_dtype=torch.float32).cuda()
    _lib.assert_ok()
    assert (got - ref).abs().max().item() < 0.05
    # singular values pushed toward 1 (the smallest few of a random matrix stay small)
    sv = torch.linalg.svdvals(got[0])
    assert sv.max() < 1.3 and 0.6 < sv.median() < 1.25


def test_muon_arena_vs_plain():
    m1 = _model(seed=3).cuda().to(torch.bfloat16)
    m2 = copy.deepcopy(m1)
    arena = ParamArena.install(m1)
    o1 = Muon(m1.parameters(), lr=0.02, weight_decay=0.01, fused=True)
    o1.bind_arena(arena)
    o2 = Muon(m2.parameters(), lr=0.02, weight_decay=0.01)
    o2.bind_param_names(m2.named_parameters())
    torch.manual_seed(1)
    for n, p in m2.named_parameters():
        g = (torch.randn_like(p.float()) * 0.01)
        p.grad = g.to(p.dtype)
        arena.grad_view(n).copy_(p.grad.float())
    arena.grads_fresh = True
    o1.step()
    o2.step()
    _lib.assert_ok()
    for (n, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        d = (p1.float() - p2.float()).abs().max().item()
        assert d < 1e-2, (n, d)   # one bf16 ulp at |w| ~ 1
    assert o1.ns_calls == len(arena.muon_groups)
