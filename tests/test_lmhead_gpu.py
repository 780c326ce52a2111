"""Fused LM-head kernels (lse / train / dW) vs the fp32 PyTorch statement."""
import pytest
import torch

from chaoscontrol_b200.ops import _lib
from chaoscontrol_b200.ops import lm_head as LH

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[(4, 0), (2, 0), (2, 1), (4, 1)], ids=["epi16warps", "epi8warps", "epi8warps-deep", "epi16warps-deep"])
def epilogue_parts(request):
    """Run a test with both widths of the fused head's epilogue (sixteen or eight warps) and with
    both ring layouts of the one-sweep training kernel (two stages with X in shared memory, three
    stages with X in tensor memory)."""
    L = _lib.lib()
    parts, deep = request.param
    old = L.ccb_lmhead_epilogue_parts(parts)
    old_deep = L.ccb_lmhead_deep_ring(deep)
    yield request.param
    L.ccb_lmhead_epilogue_parts(old)
    L.ccb_lmhead_deep_ring(old_deep)


def _mk(R, V, seed=0, wscale=0.08):
    torch.manual_seed(seed)
    x = torch.randn(R, 256, device="cuda").bfloat16()
    W = (torch.randn(V, 256, device="cuda") * wscale).bfloat16()
    t = torch.randint(0, V, (R,), device="cuda")
    ss = (x.float() ** 2).sum(-1)
    return x, W, t, ss


@pytest.mark.parametrize("R,V", [(128, 128), (256, 512), (1000, 1024), (4096, 16384)])
def test_lmhead_lse(R, V, epilogue_parts):
    x, W, t, ss = _mk(R, V)
    loss, lse = LH.lm_head_lse(x, ss, W, t)
    _lib.assert_ok()
    rl, rlse, _, _ = LH.lm_head_reference(x, ss, W, t, want_grads=False)
    assert torch.allclose(lse, rlse, rtol=1e-3, atol=2e-2), (lse - rlse).abs().max()
    assert torch.allclose(loss, rl, rtol=1e-3, atol=3e-2), (loss - rl).abs().max()


@pytest.mark.parametrize("R,V,chunks,norm", [(128, 128, 1, True), (384, 512, 3, True),
                                             (1000, 1024, 2, False), (2048, 16384, 4, True)])
def test_lmhead_train(R, V, chunks, norm, epilogue_parts):
    x, W, t, ss = _mk(R, V, seed=1)
    w = torch.rand(R, device="cuda")
    gscale = 1.0 / R
    rowss = ss if norm else None
    loss, lse, dX, part = LH.lm_head_train(x, rowss, W, t, gscale=gscale, rowweight=w,
                                           row_chunks=chunks)
    _lib.assert_ok()
    rl, rlse, rdX, rdW = LH.lm_head_reference(x, rowss, W, t, gscale=gscale, rowweight=w)
    assert torch.allclose(lse, rlse, rtol=1e-3, atol=2e-2)
    assert torch.allclose(loss, rl, rtol=1e-3, atol=3e-2), (loss - rl).abs().max()
    sx = rdX.abs().max().item()
    assert (dX.float() - rdX).abs().max().item() <= 0.03 * sx + 1e-7, \
        ((dX.float() - rdX).abs().max().item(), sx)
    dW = part.sum(0)
    sw = rdW.abs().max().item()
    assert (dW - rdW).abs().max().item() <= 0.03 * sw + 1e-7, ((dW - rdW).abs().max().item(), sw)


def test_lmhead_train_deterministic(epilogue_parts):
    x, W, t, ss = _mk(1024, 2048, seed=2)
    a = LH.lm_head_train(x, ss, W, t, gscale=1e-3)
    b = LH.lm_head_train(x, ss, W, t, gscale=1e-3)
    _lib.assert_ok()
    for u, v in zip(a, b):
        assert torch.equal(u, v)


def _mk_d(R, V, D, seed=0, wscale=0.08):
    torch.manual_seed(seed)
    x = torch.randn(R, D, device="cuda").bfloat16()
    W = (torch.randn(V, D, device="cuda") * wscale).bfloat16()
    t = torch.randint(0, V, (R,), device="cuda")
    return x, W, t, (x.float() ** 2).sum(-1)


@pytest.mark.parametrize("R,V,D,norm", [(300, 1000, 512, True), (1024, 16384, 512, True),
                                        (515, 520, 128, False), (20000, 2048, 384, True)])
def test_lmhead_general_dims(R, V, D, norm):
    """Model dims other than 256 go through the GEMM-epilogue LM head."""
    x, W, t, ss = _mk_d(R, V, D, seed=3)
    assert not LH.fused_supported(x, W) and LH.general_supported(x, W)
    rowss = ss if norm else None
    loss, lse = LH.lm_head_lse(x, rowss, W, t)
    rl, rlse, _, _ = LH.lm_head_reference(x, rowss, W, t, want_grads=False)
    _lib.assert_ok()
    assert torch.allclose(lse, rlse, rtol=1e-3, atol=2e-2), (lse - rlse).abs().max()
    assert torch.allclose(loss, rl, rtol=1e-3, atol=3e-2), (loss - rl).abs().max()
    w = torch.rand(R, device="cuda")
    gscale = 1.0 / R
    loss2, lse2, dX, part = LH.lm_head_train(x, rowss, W, t, gscale=gscale, rowweight=w)
    _lib.assert_ok()
    _, _, rdX, rdW = LH.lm_head_reference(x, rowss, W, t, gscale=gscale, rowweight=w)
    assert torch.allclose(loss2, rl, rtol=1e-3, atol=3e-2), (loss2 - rl).abs().max()
    assert torch.equal(lse2, lse)
    sx = rdX.abs().max().item()
    assert (dX.float() - rdX).abs().max().item() <= 0.03 * sx + 1e-7, ((dX.float() - rdX).abs().max().item(), sx)
    dW = part.sum(0)
    sw = rdW.abs().max().item()
    assert (dW - rdW).abs().max().item() <= 0.03 * sw + 1e-7, ((dW - rdW).abs().max().item(), sw)
    again = LH.lm_head_train(x, rowss, W, t, gscale=gscale, rowweight=w)
    for u, v in zip((loss2, lse2, dX, part), again):
        assert torch.equal(u, v)


@pytest.mark.parametrize("wscale,peak", [(0.08, 0.0), (1.5, 0.0), (0.3, 40.0)])
def test_lmhead_one_sweep_matches_two_sweeps_and_the_reference(wscale, peak, epilogue_parts):
    """The single-sweep training kernel (fixed per-row reference instead of the true row maximum)
    against the two-sweep kernel and the fp32 statement: ordinary logits, logits spread over tens of
    nats, and a target column that towers over the row's first 32 logits."""
    R, V = 1024, 4096
    x, W, t, ss = _mk(R, V, seed=3, wscale=wscale)
    if peak:
        # make each row's target logit ~`peak` nats larger than the rest: align W[t] with x
        xn = torch.nn.functional.normalize(x.float(), dim=-1)
        Wf = W.float()
        Wf[t] = Wf[t] + xn * (peak / 16.0)
        W = Wf.bfloat16()
    w = torch.rand(R, device="cuda") + 0.5
    kw = dict(gscale=1.0 / R, rowweight=w, row_chunks=2)
    l1, lse1, dX1, p1 = LH.lm_head_train(x, ss, W, t, one_sweep=True, **kw)
    l2, lse2, dX2, p2 = LH.lm_head_train(x, ss, W, t, one_sweep=False, **kw)
    _lib.assert_ok()
    rl, rlse, rdX, rdW = LH.lm_head_reference(x, ss, W, t, gscale=1.0 / R, rowweight=w)
    assert torch.isfinite(dX1.float()).all() and torch.isfinite(lse1).all()
    assert torch.allclose(lse1, rlse, rtol=1e-3, atol=3e-2), (lse1 - rlse).abs().max()
    assert torch.allclose(l1, rl, rtol=2e-3, atol=5e-2), (l1 - rl).abs().max()

    def rel(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))
    assert rel(dX1, rdX) < 2e-2 and rel(dX1, dX2) < 2e-2, (rel(dX1, rdX), rel(dX1, dX2))
    assert rel(p1.sum(0), rdW) < 2e-2 and rel(p1.sum(0), p2.sum(0)) < 1e-2
