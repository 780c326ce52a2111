"""Scan-backend and fused-block comparison benches: they run, time every mode, and agree on what they compare."""
import json

import pytest
import torch

from chaoscontrol_b200.utils import backend_bench as KB


def test_scan_bench_times_every_backend_and_mode_on_cpu(tmp_path, capsys):
    out = tmp_path / "s.json"
    assert KB.main(["scan", "--B", "2", "--T", "16", "--D", "8", "--dtype", "fp32", "--warmup", "1", "--iters", "2",
                    "--device", "cpu", "--output-json", str(out)]) == 0
    rep = json.loads(out.read_text())
    assert [r["backend"] for r in rep["results"]] == ["python", "chunked"]
    assert all(r[m]["ms"] > 0 and r[m]["tokens_per_sec"] > 0 for r in rep["results"] for m in ("fwd", "bwd", "fwd+bwd"))
    assert "fwd+bwd" in capsys.readouterr().out
    rep = KB.bench_scan(B=1, T=32, D=4, dtype="fp32", warmup=0, iters=1, device="cpu", python_max_T=8)
    assert rep["results"][0] == {"backend": "python", "skipped": "T = 32 > 8"}


def test_block_bench_compares_the_same_weights_on_cpu(capsys):
    assert KB.main(["block", "--batch-sizes", "2", "3", "--seq-len", "8", "--dim", "16", "--warmup", "1", "--iters", "2",
                    "--device", "cpu"]) == 0
    txt = capsys.readouterr().out
    assert "post-scan backend" in txt and "speedup" in txt
    rep = KB.bench_block(batch_sizes=[2], seq_len=8, dim=16, warmup=0, iters=1, device="cpu")
    assert rep["results"][0]["speedup"] > 0 and rep["dtype"] == "float32"


@pytest.mark.gpu
def test_cuda_scan_kernel_beats_the_tensor_op_scan():
    rep = KB.bench_scan(B=64, T=512, D=256, warmup=3, iters=5)
    by = {r["backend"]: r for r in rep["results"]}
    assert "skipped" in by["python"] and by["ssm_scan"]["fwd+bwd"]["ms"] < by["chunked"]["fwd+bwd"]["ms"]


@pytest.mark.gpu
def test_fused_block_is_not_slower_than_the_unfused_block():
    rep = KB.bench_block(batch_sizes=[64], warmup=3, iters=5)
    assert rep["results"][0]["speedup"] > 0.9
