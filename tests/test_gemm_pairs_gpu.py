"""The two alternative layouts of the tcgen05 GEMM -- CTA pairs (2-CTA clusters, ``cta_group::2``)
and the resident weight tile (B loaded once per CTA, only A streams) -- vs the fp32 PyTorch statement
and vs the default kernel: plain and MN-major B, ragged shapes (a pair tile whose second CTA is
partly or wholly past the last row, N that leaves half tiles empty, a last row tile that is partly
empty), every fused trunk epilogue."""
import pytest
import torch

from chaoscontrol_b200.ops import _lib
from chaoscontrol_b200.ops import gemm as G

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["pairs", "resident", "pair_resident"])
def pairs(request):
    L = _lib.lib()
    if request.param == "pairs":
        old = L.ccb_gemm_cta_group(2)
        yield
        L.ccb_gemm_cta_group(old)
    elif request.param == "pair_resident":
        # CTA pairs with the weight tile resident (half per CTA): K <= 256 and K in (256, 512]; shapes the
        # layout does not take fall through to the default kernel
        old = L.ccb_gemm_pair_resident(3)
        yield
        L.ccb_gemm_pair_resident(old)
    else:
        old = L.ccb_gemm_resident_b(1)
        yield
        L.ccb_gemm_resident_b(old)


def _default_layout(fn):
    L = _lib.lib()
    cg, rb, pr = L.ccb_gemm_cta_group(1), L.ccb_gemm_resident_b(0), L.ccb_gemm_pair_resident(0)
    try:
        return fn()
    finally:
        L.ccb_gemm_cta_group(cg)
        L.ccb_gemm_resident_b(rb)
        L.ccb_gemm_pair_resident(pr)


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def _close(got, ref, rtol=2e-2, atol=2e-2):
    got = got.float()
    err = (got - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err <= atol + rtol * den, f"max err {err} vs scale {den}"


@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (512, 256, 256), (1000, 768, 256), (640, 512, 320),
                                   (4096, 1024, 256), (513, 200, 128), (5000, 256, 1024),
                                   (40000, 256, 256), (20001, 1024, 192), (19000, 512, 256), (37999, 200, 64),
                                   (40000, 256, 512), (38001, 512, 448)])
def test_pair_gemm_tn(pairs, M, N, K):
    torch.manual_seed(0)
    a, b = _rand(M, K), _rand(N, K)
    out = G.gemm(a, b)
    _lib.assert_ok()
    _close(out, G.gemm_reference(a, b), atol=0.05 * (K ** 0.5) / 16)
    single = _default_layout(lambda: G.gemm(a, b))
    assert torch.equal(out, single)           # same k order, same accumulators: same bits


@pytest.mark.parametrize("M,N,K", [(512, 256, 256), (1024, 304, 128), (4096, 512, 256), (777, 256, 512),
                                   (38000, 256, 256), (19001, 512, 128), (38000, 256, 512), (40001, 512, 384)])
def test_pair_gemm_b_mn(pairs, M, N, K):
    torch.manual_seed(1)
    a, b = _rand(M, K), _rand(K, N)
    out = G.gemm(a, b, b_mn=True)
    _lib.assert_ok()
    _close(out, G.gemm_reference(a, b, b_mn=True), atol=0.05 * (K ** 0.5) / 16)


@pytest.mark.parametrize("M", [640, 4096, 9000, 40100, 76001])
def test_pair_gemm_epilogues(pairs, M):
    torch.manual_seed(4)
    D, F = 256, 512
    x = _rand(M, D)
    ss = (x.float() ** 2).sum(-1)
    w = _rand(4 * D, D, scale=0.06)
    out = G.gemm(x, w, epi=G.EPI_ROWSCALE, rowss=ss, inv_dim=1.0 / D, eps=1e-6)
    _close(out, G.gemm_reference(x, w, epi=G.EPI_ROWSCALE, rowss=ss, inv_dim=1.0 / D))
    wf = _rand(F, D, scale=0.06)
    f = torch.empty(M, F, dtype=torch.bfloat16, device="cuda")
    u = G.gemm(x, wf, epi=G.EPI_ROWSCALE_SILU, rowss=ss, inv_dim=1.0 / D, c2=f)
    u_ref, f_ref = G.gemm_reference(x, wf, epi=G.EPI_ROWSCALE_SILU, rowss=ss, inv_dim=1.0 / D)
    _close(u, u_ref)
    _close(f, f_ref)
    y = _rand(M, D)
    wo = _rand(D, D, scale=0.06)
    ss2 = torch.empty(M, dtype=torch.float32, device="cuda")
    x2 = G.gemm(y, wo, epi=G.EPI_RESID_SS, r1=x, ss_out=ss2)
    x2_ref, ss2_ref = G.gemm_reference(y, wo, epi=G.EPI_RESID_SS, r1=x)
    _close(x2, x2_ref)
    assert torch.allclose(ss2, (x2.float() ** 2).sum(-1), rtol=1e-3, atol=1e-3)
    dx3 = _rand(M, D)
    wproj = _rand(D, F, scale=0.06)
    du = G.gemm(dx3, wproj, b_mn=True, epi=G.EPI_DSILU, r1=u, rowss=ss, inv_dim=1.0 / D)
    _close(du, G.gemm_reference(dx3, wproj, b_mn=True, epi=G.EPI_DSILU, r1=u, rowss=ss, inv_dim=1.0 / D))
    dres = _rand(M, D)
    dxo = G.gemm(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss, inv_dim=1.0 / D)
    _close(dxo, G.gemm_reference(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss,
                                 inv_dim=1.0 / D))
    _lib.assert_ok()
    again = G.gemm(du, wf, b_mn=True, epi=G.EPI_RMSBWD, r1=x, r2=dres, rowss=ss, inv_dim=1.0 / D)
    assert torch.equal(dxo, again)
