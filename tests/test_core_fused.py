"""FusedCareSSMBlock / post_scan_fused against the plain block."""
import copy

import pytest
import torch

from chaoscontrol_b200.models.core_fused import FusedCareSSMBlock, post_scan_fused, post_scan_reference
from chaoscontrol_b200.models.model import CareSSMBlock


def _rel(a, b):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def test_from_unfused_round_trip_and_cpu_equivalence():
    torch.manual_seed(0)
    blk = CareSSMBlock(16, 2)
    fused = FusedCareSSMBlock.from_unfused(blk)
    assert set(fused.state_dict()) == set(blk.state_dict())
    x = torch.randn(2, 7, 16)
    assert torch.allclose(fused(x), blk(x), atol=1e-6)
    y1, h1 = fused(x, return_final_state=True, initial_state=torch.randn(2, 16).mul(0))
    y2, h2 = blk(x, return_final_state=True)
    assert torch.allclose(y1, y2, atol=1e-6) and torch.allclose(h1, h2, atol=1e-6)
    out, stats = fused(x, return_jacobian_stats=True)
    assert isinstance(stats, dict)
    s = torch.zeros(2, 16)
    a, sa = fused.step(x[:, 0], s)
    b, sb = blk.step(x[:, 0], s)
    assert torch.allclose(a, b, atol=1e-6) and torch.allclose(sa, sb, atol=1e-6)
    with pytest.raises(ValueError):
        FusedCareSSMBlock.from_unfused(CareSSMBlock(16, 2, a_mode="full"))
    with pytest.raises(ValueError):
        FusedCareSSMBlock.from_unfused(CareSSMBlock(16, 2, rich_b_mode="nn"))
    args = (torch.randn(2, 3, 16), torch.randn(2, 3, 16), torch.rand(16) + 0.5, 1e-6, torch.randn(32, 16), torch.randn(16, 32))
    assert torch.equal(post_scan_fused(*args), post_scan_reference(*args))


@pytest.mark.gpu
@pytest.mark.parametrize("dim,ff", [(256, 2), (512, 4)])
def test_fused_block_gpu_forward_backward(dim, ff):
    from chaoscontrol_b200.ops import _lib
    torch.manual_seed(1)
    ref = CareSSMBlock(dim, ff).cuda()
    with torch.no_grad():
        ref.input_norm.weight.uniform_(0.7, 1.3)
        ref.ff_norm.weight.uniform_(0.7, 1.3)
        ref.core.log_a.normal_()
    blk16 = copy.deepcopy(ref).to(torch.bfloat16)
    with torch.no_grad():
        for p, q in zip(ref.parameters(), blk16.parameters()):
            p.copy_(q.float())
    fused = FusedCareSSMBlock.from_unfused(blk16)
    x = torch.randn(3, 128, dim, device="cuda")
    h0 = torch.randn(3, dim, device="cuda") * 0.1
    xr = x.clone().requires_grad_(True)
    xf = x.bfloat16().requires_grad_(True)
    yr, hr = ref(xr, initial_state=h0, return_final_state=True)
    yf, hf = fused(xf, initial_state=h0, return_final_state=True)
    _lib.assert_ok()
    assert _rel(yf, yr) < 2e-2 and _rel(hf, hr) < 2e-2
    g = torch.randn_like(yr)
    yr.backward(g)
    yf.backward(g.bfloat16())
    _lib.assert_ok()
    assert _rel(xf.grad, xr.grad) < 4e-2
    for (n, p), q in zip(ref.named_parameters(), fused.parameters()):
        assert _rel(q.grad, p.grad) < 6e-2, n
    # post-scan tail on its own
    a = torch.randn(2, 64, dim, device="cuda").bfloat16().requires_grad_(True)
    b = torch.randn(2, 64, dim, device="cuda").bfloat16().requires_grad_(True)
    args = (fused.ff_norm.weight, 1e-6, fused.ff.fc.weight, fused.ff.proj.weight)
    out = post_scan_fused(a, b, *args)
    want = post_scan_reference(a.float(), b.float(), *(t.float() if torch.is_tensor(t) else t for t in args))
    assert _rel(out, want) < 2e-2
    out.float().sum().backward()
    assert a.grad is not None and torch.equal(a.grad, b.grad)
