import json

import pytest
import torch

from chaoscontrol_b200.utils import canary, profiling as P


def test_section_timer_and_kernel_timer_cpu():
    t = P.SectionTimer()
    x = torch.randn(64, 64)
    for _ in range(3):
        with t.section("mm"):
            x @ x
        with t.section("add"):
            x + x
    s = t.summary()
    assert set(s) == {"mm", "add"} and s["mm"]["calls"] == 3 and s["mm"]["total_ms"] >= 0
    t.reset()
    assert t.summary() == {}
    with P.nvtx_range("noop"):
        P.nvtx_mark("m")
    r = P.time_kernel(lambda: x @ x, warmup=1, iters=5)
    assert r["ms_min"] <= r["ms_median"]


def test_profile_steps_writes_tables(tmp_path):
    lin = torch.nn.Linear(8, 8)
    s = P.profile_steps(lambda i: lin(torch.randn(4, 8)).sum().backward(), out_dir=tmp_path / "prof", wait=0, warmup=1,
                        active=2)
    assert s["steps_profiled"] == 2 and (tmp_path / "prof" / "cpu_table.txt").read_text()
    assert json.loads((tmp_path / "prof" / "summary.json").read_text())["events"] > 0
    assert (tmp_path / "prof" / "trace.json").exists()
    assert isinstance(P.topology_snapshot(), dict)
    assert P.enable_stack_dump_signal() in (True, False)


def test_canary_detects_overrun():
    t = canary.guarded_empty((3, 5), dtype=torch.float32, device="cpu", name="ok")
    t.fill_(1.0)
    canary.check_canaries()
    t2 = canary.guarded_empty((16,), dtype=torch.bfloat16, device="cpu", name="victim")
    assert t2.data_ptr() % 2 == 0
    flat = t2.untyped_storage()
    raw = torch.tensor([], dtype=torch.uint8).set_(flat)
    raw[canary.MARGIN_BYTES + 32] = 0          # first byte after the 16 bf16 elements
    with pytest.raises(AssertionError, match="victim"):
        canary.check_canaries()
    canary.check_canaries()


@pytest.mark.gpu
def test_kernels_do_not_write_outside_their_outputs():
    """Ragged shapes through the GEMM / scan / LM-head kernels with canary margins around every output."""
    from chaoscontrol_b200.ops import _lib
    from chaoscontrol_b200.ops import gemm as G
    from chaoscontrol_b200.ops import lm_head as LH
    torch.manual_seed(0)
    dev = "cuda"
    for M, N, K in [(130, 72, 64), (257, 256, 320), (1000, 520, 256)]:
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        out = canary.guarded_empty((M, N), dtype=torch.bfloat16, device=dev, name=f"gemm{M}x{N}")
        G.gemm(a, b, out=out)
        o32 = canary.guarded_empty((M, N), dtype=torch.float32, device=dev, name=f"gemm32_{M}x{N}")
        G.gemm(a, b, out=o32)
        x = torch.randn(M, N, device=dev).bfloat16()
        ss = canary.guarded_empty((M,), dtype=torch.float32, device=dev, name="ss")
        res = canary.guarded_empty((M, N), dtype=torch.bfloat16, device=dev, name="resid")
        G.gemm(a, b, epi=G.EPI_RESID_SS, r1=x, ss_out=ss, out=res)
    x = torch.randn(300, 512, device=dev).bfloat16()
    W = (torch.randn(1000, 512, device=dev) * 0.05).bfloat16()
    t = torch.randint(0, 1000, (300,), device=dev)
    LH.lm_head_train(x, (x.float() ** 2).sum(-1), W, t, gscale=1.0 / 300)
    torch.cuda.synchronize()
    _lib.assert_ok()
    canary.check_canaries()
