"""fp8 linear: scaling-state contract on CPU, kernel numerics on the GPU."""
import pytest
import torch
import torch.nn as nn

from chaoscontrol_b200.ops import fp8_linear as F8
from chaoscontrol_b200.ops.fp8_linear import FusedFP8Linear, fused_fp8_flush_all
from chaoscontrol_b200.precision import maybe_promote_linears_to_fused_fp8


def test_state_buffers_and_cold_start_scales():
    m = FusedFP8Linear(32, 48, bias=True, dtype=torch.float32)
    sd = m.state_dict()
    for t in ("x", "w", "gy", "gx"):
        assert sd[f"{t}_amax_history"].shape == (16,) and sd[f"{t}_amax_pending"].shape == (1,)
    assert all(float(sd[f"{t}_scale"]) == 1.0 for t in ("x", "w", "gy"))
    assert "gx_scale" not in sd


def test_forward_backward_close_to_fp32_after_flush_cpu():
    torch.manual_seed(0)
    lin = nn.Linear(64, 32, bias=True)
    m = FusedFP8Linear.from_nn_linear(lin)
    x = torch.randn(20, 64, requires_grad=True)
    y0 = m(x)                                   # cold start: scale 1, observes amax
    gy = torch.randn_like(y0)
    y0.backward(gy)
    assert float(m.x_amax_pending) == pytest.approx(float(x.detach().abs().max()))
    assert float(m.gy_amax_pending) == pytest.approx(float(gy.abs().max()))
    assert fused_fp8_flush_all(nn.Sequential(m)) == 1
    assert float(m.x_scale) == pytest.approx(float(x.detach().abs().max()) / 448.0)
    assert float(m.gy_scale) == pytest.approx(float(gy.abs().max()) / 57344.0)
    assert float(m.x_amax_pending) == 0.0 and float(m.x_amax_history[-1]) > 0
    x.grad = None
    m.weight.grad = None
    m.bias.grad = None
    y = m(x)
    ref = lin(x)
    assert (y - ref).abs().max() < 0.08 * ref.abs().max()
    y.backward(gy)
    ref.backward(gy)
    assert (m.weight.grad - lin.weight.grad).norm() < 0.1 * lin.weight.grad.norm()   # e5m2: 2 mantissa bits
    assert torch.allclose(m.bias.grad, lin.bias.grad, atol=1e-4)
    # oracle of the forward quantisation
    want = F8.fp8_linear_reference(x, m.weight, m.bias, m.x_scale, m.w_scale)
    assert torch.allclose(m(x), want, atol=1e-4)


def test_history_rolls_and_old_peaks_expire():
    m = FusedFP8Linear(8, 8, bias=False, dtype=torch.float32, amax_history_len=3)
    for peak in (8.0, 2.0, 2.0, 2.0):
        m.x_amax_pending.fill_(peak)
        m.flush_amax_history()
    assert m.x_amax_history.tolist() == [2.0, 2.0, 2.0]
    assert float(m.x_scale) == pytest.approx(2.0 / 448.0)


def test_promotion_skips_ineligible_linears():
    net = nn.Sequential(nn.Linear(64, 64), nn.Linear(64, 10), nn.Linear(6, 64))
    n = maybe_promote_linears_to_fused_fp8(net, True)
    assert n >= 1 and isinstance(net[0], FusedFP8Linear)
    assert maybe_promote_linears_to_fused_fp8(nn.Sequential(nn.Linear(64, 64)), False) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N,bias", [(256, 256, 512, False), (300, 272, 200, True), (1024, 512, 256, True)])
def test_fp8_linear_gpu_matches_quantised_fp32_reference(M, K, N, bias):
    torch.manual_seed(0)
    dev = "cuda"
    m = FusedFP8Linear(K, N, bias=bias, device=dev)
    if bias:
        with torch.no_grad():
            m.bias.normal_()
    x = torch.randn(M, K, device=dev, dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    m(x).backward(gy)                            # observe amax at unit scale
    m.flush_amax_history()
    x.grad = None
    m.weight.grad = None
    if bias:
        m.bias.grad = None
    y = m(x)
    y.backward(gy)
    torch.cuda.synchronize()

    def q(t, scale, dt, mx):
        return (t.float() / scale).clamp(-mx, mx).to(dt).float() * scale
    xs, ws, gs = float(m.x_scale), float(m.w_scale), float(m.gy_scale)
    xq, wq = q(x.detach(), xs, torch.float8_e4m3fn, 448.0), q(m.weight.detach(), ws, torch.float8_e4m3fn, 448.0)
    gq = q(gy, gs, torch.float8_e5m2, 57344.0)
    y_ref = xq @ wq.T + (m.bias.float() if bias else 0.0)
    assert torch.allclose(y.float(), y_ref, atol=2e-2 * float(y_ref.detach().abs().max()), rtol=0)
    gx_ref, gw_ref = gq @ wq, gq.T @ xq
    assert torch.allclose(x.grad.float(), gx_ref, atol=2e-2 * float(gx_ref.abs().max()), rtol=0)
    assert torch.allclose(m.weight.grad.float(), gw_ref, atol=2e-2 * float(gw_ref.abs().max()), rtol=0)
    if bias:
        assert torch.allclose(m.bias.grad.float(), gy.float().sum(0), atol=0.5, rtol=2e-2)
    # and the quantised result is close to the unquantised one
    full = x.detach().float() @ m.weight.detach().float().T
    rel = (y.float() - (full + (m.bias.float() if bias else 0.0))).norm() / full.norm()
    assert rel < 0.06
    assert float(m.x_amax_pending) == pytest.approx(float(x.detach().abs().max()), rel=1e-3)
    from chaoscontrol_b200.ops import _lib
    _lib.assert_ok()


@pytest.mark.gpu
def test_fp8_cast_kernels_match_torch():
    torch.manual_seed(1)
    x = torch.randn(333, 200, device="cuda", dtype=torch.bfloat16) * 3
    scale = torch.tensor([0.02], device="cuda")
    pend = torch.zeros(1, device="cuda")
    for dt, mx in ((torch.float8_e4m3fn, 448.0), (torch.float8_e5m2, 57344.0)):
        pend.zero_()
        got = F8.fp8_cast(x, scale, pend, dt)
        want = (x.float() / 0.02).clamp(-mx, mx).to(dt)
        assert torch.equal(got.view(torch.uint8), want.view(torch.uint8))
        assert float(pend) == float(x.abs().max())
        cs = torch.zeros(200, device="cuda")
        pend.zero_()
        gt = F8.fp8_cast_transpose(x, scale, pend, dt, colsum=cs)
        assert gt.shape == (200, 333) and gt.stride(0) % 16 == 0
        assert torch.equal(gt.contiguous().view(torch.uint8), want.T.contiguous().view(torch.uint8))
        assert torch.allclose(cs, x.float().sum(0), atol=1e-2, rtol=1e-3)
        assert float(pend) == float(x.abs().max())
    hist = torch.tensor([5.0, 1.0, 2.0], device="cuda")
    p = torch.tensor([0.5], device="cuda")
    s = torch.ones(1, device="cuda")
    F8.fp8_flush_amax(hist, p, s, 448.0)
    assert hist.tolist() == [1.0, 2.0, 0.5] and float(p) == 0.0 and float(s) == pytest.approx(2.0 / 448.0)
