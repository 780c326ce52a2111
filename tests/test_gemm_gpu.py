"""tcgen05 GEMM vs an fp32 PyTorch reference: every operand layout, epilogue,
ragged shapes, batching and split-K."""
import pytest
import torch

from chaoscontrol_b200.ops import _lib
from chaoscontrol_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def _close(got, ref, rtol=2e-2, atol=2e-2):
    got = got.float()
    err = (got - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err <= atol + rtol * den, f"max err {err} vs scale {den}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 256), (1000, 768, 256), (384, 512, 320),
                                   (130, 72, 40), (4096, 1024, 256)])
def test_gemm_tn(M, N, K):
    torch.manual_seed(0)
    a, b = _rand(M, K), _rand(N, K)
    out = G.gemm(a, b)
    _lib.assert_ok()
    _close(out, G.gemm_reference(a, b), atol=0.05 * (K ** 0.5) / 16)


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 304, 128), (128, 1024, 192)])
def test_gemm_b_mn(M, N, K):
    torch.manual_seed(1)
    a, b = _rand(M, K), _rand(K, N)
    out = G.gemm(a, b, b_mn=True)
    _lib.assert_ok()
    _close(out, G.gemm_reference(a, b, b_mn=True), atol=0.05 * (K ** 0.5) / 16)


@pytest.mark.parametrize("M,N,K,S", [(256, 256, 4096, 1), (1024, 256, 8192, 4), (512, 512, 5000, 3),
                                     (256, 256, 16384, 16)])
def test_gemm_mn_mn_splitk(M, N, K, S):
    torch.manual_seed(2)
    a, b = _rand(K, M), _rand(K, N)
    S = min(S, G.pick_splits(M, N, K) if S > 4 else S)
    out = G.gemm(a, b, a_mn=True, b_mn=True, splits=S, out_dtype=torch.float32)
    _lib.assert_ok()
    got = out.sum(0) if S > 1 else out
    _close(got, G.gemm_reference(a, b, a_mn=True, b_mn=True), rtol=1e-2, atol=0.02 * (K ** 0.5) / 16)


def test_gemm_batched_axpby():
    torch.manual_seed(3)
    a, b, c = _rand(5, 256, 256, scale=0.1), _rand(5, 256, 256, scale=0.1), _rand(5, 256, 256)
    out = G.gemm(a, b, alpha=2.0, beta=-0.5, cin=c)
    _lib.assert_ok()
    _close(out, G.gemm_reference(a, b, alpha=2.0, beta=-0.5, cin=c))
    # batched with MN-major B (the Newton-Schulz "poly @ X" form)
    x = _rand(3, 256, 512, scale=0.1)
    out2 = G.gemm(a[:3], x, b_mn=True, alpha=1.0, beta=3.0, cin=x)
    _lib.assert_ok()
    _close(out2, G.gemm_reference(a[:3], x, b_mn=True, alpha=1.0, beta=3.0, cin=x))


def test_gemm_epilogues():
    torch.manual_seed(4)
    M, D, F = 640, 256, 512
    x = _rand(M, D)
    ss = (x.float() ** 2).sum(-1)
    w = _rand(4 * D, D, scale=0.06)
    # row scale
    out = G.gemm(x, w, epi=G.EPI_ROWSCALE, rowss=ss, inv_dim=1.0 / D, eps=1e-6)
    _close(out, G.gemm_reference(x, w, epi=G.EPI_ROWSCALE, rowss=ss, inv_dim=1.0 / D))
    # row scale + silu
    wf = _rand(F, D, scale=0.06)
    f = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    u = G.gemm(x, wf, epi=G.EPI_ROWSCALE_SILU, rowss=ss, inv_dim=1.0 / D, c2=f)
    u_ref, f_ref = G.gemm_reference(x, wf, epi=G.EPI_ROWSCALE_SILU, rowss=ss, inv_dim=1.0 / D)
    _close(u, u_ref)
    _close(f, f_ref)
    # residual + sum of squares
    y = _rand(M, D)
    wo = _rand(D, D, scale=0.06)
    ss2 = torch.empty(M, dtype=torch.float32, device="cuda")
    x2 = G.gemm(y, wo, epi=G.EPI_RESID_SS, r1=x, ss_out=ss2)
    x2_ref, ss2_ref = G.gemm_reference(y, wo, epi=G.EPI_RESID_SS, r1=x)
    _close(x2, x2_ref)
    assert torch.allclose(ss2, (x2.float() ** 2).sum(-1), rtol=1e-3, atol=1e-3)
    _close(ss2, ss2_ref, rtol=3e-2, atol=1.0)
    # dsilu
    dx3 = _rand(M, D)
    wproj = _rand(D, F, scale=0.06)
    du = G.gemm(dx3, wproj, b_mn=True, epi=G.EPI_DSILU, r1=u, rowss=ss, inv_dim=1.0 / D)
    _close(du, G.gemm_reference(dx3, wproj, b_mn=True, epi=G.EPI_DSILU, r1=u, rowss=ss, inv_dim=1.0 / D))
    # rmsnorm backward + residual
    dres = _rand(M, D)
    dxo = G.gemm(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss, inv_dim=1.0 / D)
    _close(dxo, G.gemm_reference(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss,
                                 inv_dim=1.0 / D))
    _lib.assert_ok()


def test_gemm_ss_atomic_two_tiles():
    torch.manual_seed(5)
    M, D = 256, 512
    y, x = _rand(M, D), _rand(M, D)
    wo = _rand(D, D, scale=0.05)
    ss = torch.zeros(M, dtype=torch.float32, device="cuda")
    x2 = G.gemm(y, wo, epi=G.EPI_RESID_SS, r1=x, ss_out=ss, ss_atomic=True)
    _lib.assert_ok()
    assert torch.allclose(ss, (x2.float() ** 2).sum(-1), rtol=1e-3, atol=1e-3)


def test_gemm_deterministic():
    torch.manual_seed(6)
    a, b = _rand(2048, 256), _rand(1024, 256)
    o1 = G.gemm(a, b)
    o2 = G.gemm(a, b)
    _lib.assert_ok()
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("M,D,F", [(640, 512, 1024), (300, 384, 768), (4096, 512, 2048)])
def test_gemm_wide_rows(M, D, F):
    """Rows wider than one 256-column tile: RMSNorm backward over the paired
    accumulators and the residual epilogue's per-tile sum of squares."""
    torch.manual_seed(7)
    x, du, dres = _rand(M, D), _rand(M, F), _rand(M, D)
    ss = (x.float() ** 2).sum(-1)
    wf = _rand(F, D, scale=0.05)
    dxo = G.gemm(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss, inv_dim=1.0 / D)
    _close(dxo, G.gemm_reference(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss,
                                 inv_dim=1.0 / D))
    dx1 = G.gemm(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, rowss=ss, inv_dim=1.0 / D)
    _close(dx1, G.gemm_reference(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, rowss=ss, inv_dim=1.0 / D))
    y = _rand(M, F)
    wp = _rand(D, F, scale=0.05)
    ss2 = torch.full((M,), 123.0, dtype=torch.float32, device="cuda")   # stale contents must not leak
    x2 = G.gemm(y, wp, epi=G.EPI_RESID_SS, r1=x, ss_out=ss2)
    x2b = G.gemm(y, wp, epi=G.EPI_RESID_SS, r1=x, ss_out=torch.empty_like(ss2))
    _lib.assert_ok()
    _close(x2, G.gemm_reference(y, wp, epi=G.EPI_RESID_SS, r1=x)[0])
    assert torch.allclose(ss2, (x2.float() ** 2).sum(-1), rtol=1e-3, atol=1e-3)
    assert torch.equal(x2, x2b)
    assert torch.equal(dxo, G.gemm(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss,
                                   inv_dim=1.0 / D))
