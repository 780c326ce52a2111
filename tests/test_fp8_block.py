"""Block-scaled e4m3 linear: quantisers, GEMM and the autograd layer against fp32 statements."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from chaoscontrol_b200.ops import fp8_block as FB
from chaoscontrol_b200.precision import maybe_promote_linears_to_fused_fp8


def _rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def test_quantisers_round_trip_cpu():
    torch.manual_seed(0)
    x = (torch.randn(37, 256) * torch.logspace(-2, 2, 37)[:, None]).bfloat16()
    qr, inv, y = FB.quant_rows(x)
    assert qr.q.shape == (37, 256) and qr.s_t.shape == (2, 37) and inv is None and y is None
    assert _rel(qr.dequant(), x) < 0.04           # e4m3: 3 mantissa bits, per-row-block scale
    w = torch.randn(200, 256).bfloat16()
    q, qt, s = FB.quant_blocks(w)
    assert q.shape == (200, 256) and qt.shape == (256, 200) and s.shape == (2, 2)
    assert torch.equal(q.t().contiguous().view(torch.uint8), qt.view(torch.uint8))
    assert _rel(FB._dequant_t(qt, s, 200, 256).t(), w) < 0.04
    # fused RMSNorm variant
    wn = torch.rand(256) + 0.5
    qn, inv, yn = FB.quant_rows(x, norm_weight=wn, want_normed=True)
    ref = F.rms_norm(x.float(), (256,), eps=1e-6) * wn.bfloat16().float()
    assert _rel(yn, ref) < 1e-2 and _rel(qn.dequant(), ref) < 0.04
    with pytest.raises(ValueError):
        FB.quant_rows(torch.randn(4, 100).bfloat16())


def test_block_gemm_emulation_matches_dequantised_matmul():
    torch.manual_seed(1)
    x, w = torch.randn(50, 384).bfloat16(), (torch.randn(200, 384) * 0.1).bfloat16()
    qa = FB.quant_rows(x)[0]
    q, qt, s = FB.quant_blocks(w)
    out = FB.block_gemm(qa, q, s, sb_strides=(s.shape[1], 1), out_dtype=torch.float32)
    ref = FB.block_linear_reference(x, w)
    assert _rel(out, ref) < 1e-5
    assert _rel(out, x.float() @ w.float().t()) < 0.05


def test_layer_forward_backward_cpu():
    torch.manual_seed(2)
    lin = nn.Linear(256, 128, bias=True)
    layer = FB.BlockFP8Linear.from_nn_linear(lin)
    x = torch.randn(3, 9, 256, requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    out = layer(x)
    ref = lin(xr)
    assert out.shape == ref.shape and _rel(out, ref) < 0.06
    g = torch.randn_like(ref)
    out.backward(g)
    gw, gb = lin.weight.grad.clone(), lin.bias.grad.clone()
    lin.weight.grad = lin.bias.grad = None
    ref.backward(g)
    assert _rel(x.grad, xr.grad) < 0.08
    assert _rel(gw, lin.weight.grad) < 0.02 and _rel(gb, lin.bias.grad) < 0.02


def test_promotion_block_mode():
    m = nn.Sequential(nn.Linear(128, 64), nn.Linear(64, 128), nn.Linear(256, 256))
    n = maybe_promote_linears_to_fused_fp8(m, True, scaling="block")
    assert n == 2 and isinstance(m[0], FB.BlockFP8Linear) and isinstance(m[1], nn.Linear)
    with pytest.raises(ValueError):
        maybe_promote_linears_to_fused_fp8(m, True, scaling="nope")


# ---------------------------------------------------------------- GPU
@pytest.mark.gpu
@pytest.mark.parametrize("R,K,N", [(128, 128, 128), (1000, 256, 384), (4096, 512, 256), (777, 2048, 512)])
def test_block_gemm_gpu(R, K, N):
    from chaoscontrol_b200.ops import _lib
    torch.manual_seed(3)
    x = (torch.randn(R, K, device="cuda") * torch.logspace(-1, 1, R, device="cuda")[:, None]).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    qa, _, _ = FB.quant_rows(x)
    qc, _, _ = FB.quant_rows(x.cpu())
    # the kernel multiplies by a reciprocal, the emulation divides: a code may differ by one step, rarely
    assert (qa.q.cpu().view(torch.uint8) != qc.q.view(torch.uint8)).float().mean() < 2e-3
    assert torch.allclose(qa.s_t.cpu(), qc.s_t, rtol=1e-6)
    q, qt, s = FB.quant_blocks(w)
    q_c, qt_c, s_c = FB.quant_blocks(w.cpu())
    assert (q.cpu().view(torch.uint8) != q_c.view(torch.uint8)).float().mean() < 2e-3
    assert torch.equal(q.t().contiguous().view(torch.uint8), qt.view(torch.uint8))
    assert torch.allclose(s.cpu(), s_c, rtol=1e-6)
    out = FB.block_gemm(qa, q, s, sb_strides=(s.shape[1], 1), out_dtype=torch.float32)
    _lib.assert_ok()
    # exact statement on the kernel's own quantised operands
    ref = FB.QuantRows(qa.q.cpu(), qa.s_t.cpu()).dequant() @ FB._dequant_t(qt.cpu(), s.cpu(), N, K)
    assert _rel(out.cpu(), ref) < 1e-4, _rel(out.cpu(), ref)
    assert _rel(out.cpu(), x.float().cpu() @ w.float().cpu().t()) < 0.05
    bias = torch.randn(N, device="cuda").bfloat16()
    outb = FB.block_gemm(qa, q, s, sb_strides=(s.shape[1], 1), bias=bias)
    assert _rel(outb.cpu(), ref + bias.cpu().float()) < 1e-2
    assert torch.equal(outb, FB.block_gemm(qa, q, s, sb_strides=(s.shape[1], 1), bias=bias))


@pytest.mark.gpu
def test_layer_and_fused_norm_gpu():
    from chaoscontrol_b200.models.core import RMSNorm
    from chaoscontrol_b200.ops import _lib
    torch.manual_seed(4)
    norm = RMSNorm(256).cuda().to(torch.bfloat16)
    with torch.no_grad():
        norm.weight.uniform_(0.5, 1.5)
    lin = nn.Linear(256, 512, bias=False).cuda().to(torch.bfloat16)
    layer = FB.BlockFP8Linear.from_nn_linear(lin)
    x = torch.randn(6, 100, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    xr = x.detach().clone().float().requires_grad_(True)
    norm.emit_fp8_blocks = True
    h = norm(x)
    assert hasattr(h, "_ccb_quant")
    out = layer(h)
    ref = F.linear(F.rms_norm(xr, (256,), eps=norm.eps) * norm.weight.float(), lin.weight.float())
    _lib.assert_ok()
    assert _rel(out, ref) < 0.06
    g = torch.randn_like(ref)
    out.backward(g.to(out.dtype))
    gw, gn = lin.weight.grad.clone().float(), norm.weight.grad.clone().float()
    lin.weight.grad = norm.weight.grad = None
    ref.backward(g)
    _lib.assert_ok()
    assert _rel(x.grad, xr.grad) < 0.08
    assert _rel(gw, lin.weight.grad.float()) < 0.03 and _rel(gn, norm.weight.grad.float()) < 0.05
    # without the producer tag the layer quantises on its own and agrees
    out2 = layer(h.detach().clone())
    assert _rel(out2, out) < 3e-2   # re-quantising the bf16-rounded row moves a few codes
