"""CPU check of the hand-scheduled trunk (ops/trunk.py): forward and the
hand-derived backward, built from the GEMM-epilogue contracts, against
autograd through the plain PyTorch modules."""
import torch

from chaoscontrol_b200.models.model import CareSSMBlock, CareStudentLM, _TrunkFn
from chaoscontrol_b200.ops import trunk as T


def _weights(blk):
    c = blk.core
    Wp = torch.cat((c.select_proj.weight, c.in_proj.weight, c.gate_proj.weight,
                    c.delta_proj.weight), 0).detach()
    return T.LayerWeights(Wp=Wp, Wo=c.out_proj.weight.detach(), Wfc=blk.ff.fc.weight.detach(),
                          Wproj=blk.ff.proj.weight.detach(), wn1=blk.input_norm.weight.detach(),
                          wn2=blk.ff_norm.weight.detach(), log_a=c.log_a.detach()).prepare()


def test_layer_forward_backward_matches_autograd():
    torch.manual_seed(0)
    B, Tn, D = 3, 11, 16
    blk = CareSSMBlock(D, 2)
    with torch.no_grad():
        blk.input_norm.weight.uniform_(0.5, 1.5)
        blk.ff_norm.weight.uniform_(0.5, 1.5)
        blk.core.log_a.normal_()
    x = torch.randn(B, Tn, D, requires_grad=True)
    h0 = torch.randn(B, D, requires_grad=True)
    ref, hT_ref = blk(x, initial_state=h0, return_final_state=True)
    dout = torch.randn_like(ref)
    dhT = torch.randn(B, D)
    ((ref * dout).sum() + (hT_ref * dhT).sum()).backward()

    w = _weights(blk)
    xf = x.detach().reshape(B * Tn, D)
    ss = (xf ** 2).sum(-1)
    x3, ss3, hT, ctx = T.layer_forward(xf, ss, w, B, Tn, h0.detach())
    assert torch.allclose(x3.view(B, Tn, D), ref, atol=1e-5)
    assert torch.allclose(hT, hT_ref, atol=1e-5)
    assert torch.allclose(ss3, (x3 ** 2).sum(-1), atol=1e-4)
    dx, g = T.layer_backward(dout.reshape(B * Tn, D), ctx, w, B, Tn, dhT, want_dh0=True)
    assert torch.allclose(dx.view(B, Tn, D), x.grad, atol=2e-5)
    c = blk.core
    ref_dWp = torch.cat((c.select_proj.weight.grad, c.in_proj.weight.grad, c.gate_proj.weight.grad,
                         c.delta_proj.weight.grad), 0)
    assert torch.allclose(g.dWp, ref_dWp, atol=2e-5)
    assert torch.allclose(g.dWo, c.out_proj.weight.grad, atol=2e-5)
    assert torch.allclose(g.dWfc, blk.ff.fc.weight.grad, atol=2e-5)
    assert torch.allclose(g.dWproj, blk.ff.proj.weight.grad, atol=2e-5)
    assert torch.allclose(g.dwn1, blk.input_norm.weight.grad, atol=2e-5)
    assert torch.allclose(g.dwn2, blk.ff_norm.weight.grad, atol=2e-5)
    assert torch.allclose(g.dlog_a, c.log_a.grad, atol=2e-5)
    assert torch.allclose(g.dh0, h0.grad, atol=2e-5)


def test_trunk_fn_matches_module_path():
    torch.manual_seed(1)
    model = CareStudentLM(vocab_size=50, dim=16, num_layers=2)
    tok = torch.randint(0, 50, (2, 9))
    ref = model.encode(tok)
    (ref ** 2).sum().backward()
    ref_grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    hidden, ss, hT = _TrunkFn.apply(tok, None, True, model.embed.weight, *model._trunk_params())
    assert torch.allclose(hidden, ref, atol=1e-5)
    assert torch.allclose(ss, (hidden.reshape(-1, 16) ** 2).sum(-1), atol=1e-4)
    (hidden ** 2).sum().backward()
    for n, p in model.named_parameters():
        if n in ref_grads:
            assert torch.allclose(p.grad, ref_grads[n], atol=5e-5), n
