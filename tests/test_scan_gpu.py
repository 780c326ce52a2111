"""Fused scan kernels vs the fp32 PyTorch statement (and autograd through it)."""
import pytest
import torch

from chaoscontrol_b200.ops import _lib
from chaoscontrol_b200.ops import scan as S

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1, 2], ids=["scalar", "scalar_fma_exp", "packed_f32x2"])
def poly(request):
    """Every arithmetic mode of the fused scan: scalar fp32, scalar with FMA-pipe exponentials, packed fp32x2."""
    old = _lib.lib().ccb_scan_poly_exp(request.param)
    yield request.param
    _lib.lib().ccb_scan_poly_exp(old)


@pytest.mark.parametrize("per_row_log_a", [False, True], ids=["shared_log_a", "log_a_per_row"])
@pytest.mark.parametrize("B,T,D,with_h0", [(4, 64, 256, False), (3, 37, 512, True), (2, 9, 64, True)])
def test_scan_fused_fwd_bwd(B, T, D, with_h0, per_row_log_a, poly):
    torch.manual_seed(0)
    dev = "cuda"
    P = (torch.randn(B * T, 4 * D, device=dev) * 1.5).bfloat16()
    log_a = torch.randn(B, D, device=dev) if per_row_log_a else torch.randn(D, device=dev)
    h0 = torch.randn(B, D, device=dev) if with_h0 else None
    y, h, hT = S.scan_fused_fwd(P, log_a, h0, B, T, D)
    Pr = P.float().requires_grad_(True)
    la = log_a.clone().requires_grad_(True)
    h0r = h0.clone().requires_grad_(True) if with_h0 else None
    y_ref, h_ref, hT_ref = S.scan_fused_reference(Pr, la, h0r, B, T, D)
    assert torch.allclose(y.float(), y_ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(h.float(), h_ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(hT, hT_ref, rtol=1e-3, atol=1e-3)

    dy = (torch.randn(B * T, D, device=dev)).bfloat16()
    dhT = torch.randn(B, D, device=dev)
    (y_ref * dy.float()).sum().add((hT_ref * dhT).sum()).backward()
    dP, dloga, dh0 = S.scan_fused_bwd(P, log_a, h0, h, dy, dhT, None, 0.0, 0.0, B, T, D,
                                      want_dh0=with_h0)
    _lib.assert_ok()
    scale = Pr.grad.abs().max().item()
    assert (dP.float() - Pr.grad).abs().max().item() <= 0.03 * scale + 1e-3
    ga = la.grad
    assert dloga.shape == ga.shape
    assert (dloga - ga).abs().max().item() <= 0.03 * ga.abs().max().item() + 1e-2
    if with_h0:
        assert torch.allclose(dh0, h0r.grad, rtol=2e-2, atol=2e-2)


def test_scan_arithmetic_modes_track_each_other():
    """The modes differ by a few fp32 ulps per step: outputs agree far inside bf16 rounding."""
    torch.manual_seed(3)
    B, T, D = 4, 512, 256
    P = (torch.randn(B * T, 4 * D, device="cuda") * 2.0).bfloat16()
    P[:, 3 * D:] -= 4.0                       # small steps: long memory, where a decay error would compound
    log_a = torch.randn(D, device="cuda")
    outs = []
    for mode in (0, 1, 2):
        old = _lib.lib().ccb_scan_poly_exp(mode)
        try:
            outs.append(S.scan_fused_fwd(P, log_a, None, B, T, D))
        finally:
            _lib.lib().ccb_scan_poly_exp(old)
    y0, _, hT0 = outs[0]
    for y1, _, hT1 in outs[1:]:
        assert (hT0 - hT1).abs().max().item() <= 2e-4 * hT0.abs().max().item()
        assert (y0.float() - y1.float()).abs().max().item() <= 2.0 ** -7 * y0.float().abs().max().item()


def test_scan_bwd_rowscale():
    torch.manual_seed(1)
    B, T, D = 2, 16, 256
    P = torch.randn(B * T, 4 * D, device="cuda").bfloat16()
    log_a = torch.zeros(D, device="cuda")
    y, h, _ = S.scan_fused_fwd(P, log_a, None, B, T, D)
    dy = torch.randn(B * T, D, device="cuda").bfloat16()
    ss = torch.rand(B * T, device="cuda") * D + 1.0
    dP0, _, _ = S.scan_fused_bwd(P, log_a, None, h, dy, None, None, 0.0, 0.0, B, T, D)
    dP1, _, _ = S.scan_fused_bwd(P, log_a, None, h, dy, None, ss, 1.0 / D, 1e-6, B, T, D)
    rs = torch.rsqrt(ss / D + 1e-6)[:, None]
    assert torch.allclose(dP1.float(), dP0.float() * rs, rtol=2e-2, atol=1e-3)


def test_ssm_scan_public_op():
    torch.manual_seed(2)
    B, T, D = 3, 50, 96
    decay = torch.rand(B, T, D, device="cuda").requires_grad_(True)
    update = torch.randn(B, T, D, device="cuda").requires_grad_(True)
    out = S.ssm_scan(decay, update)
    ref = S.diag_recurrence_reference(decay, update)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
    g = torch.randn_like(out)
    gd, gu = torch.autograd.grad(out, (decay, update), g)
    rd, ru = torch.autograd.grad(ref, (decay, update), g)
    assert torch.allclose(gd, rd, rtol=1e-4, atol=1e-4)
    assert torch.allclose(gu, ru, rtol=1e-4, atol=1e-4)
    # t=0 decay gradient is exactly zero with a zero initial state
    assert torch.count_nonzero(gd[:, 0]) == 0
    with pytest.raises(ValueError):
        S.ssm_scan(decay.transpose(0, 1), update.transpose(0, 1))


_COMBOS = [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float16), (torch.float16, torch.float16),
           (torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.float32, torch.float16)]


@pytest.mark.parametrize("ddt,udt", _COMBOS, ids=lambda d: str(d).replace("torch.", ""))
@pytest.mark.parametrize("with_h0", [False, True])
def test_ssm_scan_dtype_matrix(ddt, udt, with_h0):
    """The six (decay, update) dtype pairs of the reference op run natively (no cast of the operands):
    values and both gradients against the fp32 serial loop on the same rounded inputs, gradient
    dtypes follow the operand dtypes."""
    torch.manual_seed(3)
    B, T, D = 2, 70, 160
    decay = (torch.rand(B, T, D, device="cuda") * 0.9 + 0.05).to(ddt).requires_grad_(True)
    update = torch.randn(B, T, D, device="cuda").to(udt).requires_grad_(True)
    h0 = torch.randn(B, D, device="cuda").requires_grad_(True) if with_h0 else None
    out = S.ssm_scan(decay, update, h0)
    assert out.dtype == udt
    dref = decay.detach().float().requires_grad_(True)
    uref = update.detach().float().requires_grad_(True)
    href = h0.detach().clone().requires_grad_(True) if with_h0 else None
    ref = S.diag_recurrence_reference(dref, uref, href)
    lowp = udt != torch.float32
    tol = dict(rtol=2e-2, atol=2e-2) if lowp else dict(rtol=1e-5, atol=1e-5)
    assert torch.allclose(out.float(), ref, **tol)
    g = torch.randn(B, T, D, device="cuda").to(udt)
    ins = (decay, update) + ((h0,) if with_h0 else ())
    refs = (dref, uref) + ((href,) if with_h0 else ())
    got = torch.autograd.grad(out, ins, g)
    want = torch.autograd.grad(ref, refs, g.float())
    assert got[0].dtype == ddt and got[1].dtype == udt
    gt = dict(rtol=5e-2, atol=1e-1) if (lowp or ddt != torch.float32) else dict(rtol=1e-4, atol=1e-4)
    for a, b in zip(got, want):
        assert torch.allclose(a.float(), b, **gt), (a.float() - b).abs().max()


def test_ssm_scan_rejects_unlisted_dtype_pairs():
    d = torch.rand(1, 4, 8, device="cuda", dtype=torch.float16)
    u = torch.randn(1, 4, 8, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        S.ssm_scan(d, u)
    with pytest.raises(TypeError):
        S.ssm_scan(d.double(), u.double())
