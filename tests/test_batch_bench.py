"""Batch-size sweep tool: recommendation rule, memory estimate, out-of-memory handling, CPU run of the script."""
import json

import pytest
import torch

from chaoscontrol_b200.utils import batch_bench as BB


def _row(bs, tps, oom=False):
    return {"batch_size": bs, "tokens_per_sec": tps, "mean_ms": None if tps is None else 1.0, "std_ms": 0.0, "oom": oom, "skipped": None}


def test_recommendation_is_the_last_size_before_throughput_falls():
    assert BB.recommend([_row(32, 100), _row(64, 190), _row(128, 185), _row(256, 150), _row(512, 400)]) == 128
    assert BB.recommend([_row(32, 100)]) == 32 and BB.recommend([]) is None
    assert BB.recommend([_row(32, 100), _row(64, None, oom=True)]) == 32
    assert BB.recommend([_row(32, 100), _row(64, 96)], tolerance=0.05) == 64
    assert BB.recommend([_row(32, 100), _row(64, 94)], tolerance=0.05) == 32


def test_memory_estimate_grows_with_batch_and_covers_the_flagship_step():
    kw = dict(seq_len=512, dim=256, num_layers=4, vocab=16384)
    a, b = BB.estimate_step_bytes(batch=512, **kw), BB.estimate_step_bytes(batch=1024, **kw)
    assert a < b < 2 * a + 1 and 4 * 2**30 < b < 40 * 2**30


def test_out_of_memory_is_recorded_and_other_errors_propagate():
    dev = torch.device("cpu")

    def boom():
        raise RuntimeError("CUDA out of memory. Tried to allocate")
    r = BB.bench_one(boom, batch=8, seq_len=4, warmup=1, steps=2, device=dev)
    assert r["oom"] and r["tokens_per_sec"] is None

    def other():
        raise RuntimeError("shape mismatch")
    with pytest.raises(RuntimeError, match="shape mismatch"):
        BB.bench_one(other, batch=8, seq_len=4, warmup=1, steps=2, device=dev)


def test_sweep_runs_on_cpu_and_writes_the_report(tmp_path, capsys):
    out = tmp_path / "b.json"
    assert BB.main(["--dim", "16", "--num-layers", "1", "--seq-len", "8", "--vocab-size", "64", "--batch-sizes", "4,2",
                    "--warmup-steps", "1", "--measure-steps", "2", "--device", "cpu", "--output-json", str(out)]) == 0
    rep = json.loads(out.read_text())
    assert [r["batch_size"] for r in rep["results"]] == [2, 4] and all(r["tokens_per_sec"] > 0 for r in rep["results"])
    assert rep["recommended_batch_size"] in (2, 4)
    txt = capsys.readouterr().out
    assert "recommended batch size" in txt and "tok/sec" in txt


@pytest.mark.gpu
def test_sweep_on_the_gpu_uses_the_kernel_engine_and_skips_what_cannot_fit():
    rep = BB.sweep(batch_sizes=[64, 128], warmup=2, steps=3, memory_fraction=0.8)
    assert all(r["tokens_per_sec"] > 1e6 for r in rep["results"]) and rep["recommended_batch_size"] in (64, 128)
    rep = BB.sweep(batch_sizes=[64], warmup=1, steps=1, memory_fraction=1e-6)
    assert rep["results"][0]["skipped"] and rep["recommended_batch_size"] is None
