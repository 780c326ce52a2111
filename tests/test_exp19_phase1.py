"""Phase-1 lever ablation: matrix contract, summariser gates, micro-benchmark bookkeeping."""
import json

import pytest

from chaoscontrol_b200 import exp19_phase1 as P


def _res(tps, loss=3.5, bpb=1.5, vram=30000.0):
    return {"config": {}, "train": {"aggregate_tokens_per_sec": tps, "final_loss": loss, "peak_vram_mb": vram, "steps": 10},
            "eval": {"bpb": bpb}}


def _fill(runs, matrix, fn):
    runs.mkdir(parents=True, exist_ok=True)
    for e in matrix:
        (runs / f"{e['name']}_s{e['seed']}.json").write_text(json.dumps(fn(e)))


def test_matrix_is_leave_one_out_with_runner_key_names():
    m = P.build_matrix_phase1([1, 2, 3])
    assert len(m) == 15 and len(P.build_matrix_phase1([1, 2, 3], include_fp8=True)) == 30
    names = sorted({e["name"] for e in m})
    assert names == ["bf16_all", "bf16_no_compile", "bf16_no_fused_clip", "bf16_no_fused_muon", "bf16_stock"]
    for e in m:
        assert {"fused_grad_clip", "fused_muon", "compile_full_path", "precision", "seed", "world_size"} <= set(e)
        on = sum(bool(e[k]) for k in P.LEVERS)
        assert on == {"bf16_stock": 0, "bf16_all": 3}.get(e["name"], 2)
    assert m[0]["base_lr"] == 0.128 and m[0]["world_size"] == 4
    base = dict(P.DEFAULT_BASE_CONFIG, world_size=2)
    assert all(e["world_size"] == 2 for e in P.build_matrix_phase1([1], base_config=base))


def test_verdict_ladder():
    on = [{"tokens_per_sec": 110.0 + i, "final_loss": 3.5, "bpb": 1.5, "peak_vram_mb": 100.0} for i in range(4)]
    off = [{"tokens_per_sec": 100.0 + 0.5 * i, "final_loss": 3.5, "bpb": 1.5, "peak_vram_mb": 100.0} for i in range(4)]
    assert P.compute_lever_verdict(on, off)["verdict"] == "SHIP"
    assert P.compute_lever_verdict(off, on)["verdict"] == "PARK"
    noisy = [dict(o, tokens_per_sec=o["tokens_per_sec"] + d) for o, d in zip(off, (30, -28, 25, -24))]
    assert P.compute_lever_verdict(noisy, off)["verdict"] == "INCONCLUSIVE"
    drift = [dict(o, final_loss=3.6) for o in on]
    v = P.compute_lever_verdict(drift, off)
    assert v["verdict"] == "PARK" and "final_loss" in v["reason"]
    fat = [dict(o, peak_vram_mb=110.0) for o in on]
    assert "peak_vram" in P.compute_lever_verdict(fat, off)["reason"]
    assert P.compute_lever_verdict(on[:1], off[:1])["verdict"] == "INCONCLUSIVE"     # one pair: no test


def test_summarize_gates(tmp_path):
    m = P.build_matrix_phase1([1, 2, 3])
    runs = tmp_path / "runs"
    speed = {"bf16_all": 120.0, "bf16_no_compile": 90.0, "bf16_no_fused_clip": 118.0, "bf16_no_fused_muon": 121.0,
             "bf16_stock": 80.0}
    _fill(runs, m, lambda e: _res(speed[e["name"]] + 0.1 * e["seed"] * (1 if "all" in e["name"] else 0.5)))
    out = P.summarize(m, runs)
    v = out["verdicts"]
    assert v[("bf16", "compile_full_path")]["verdict"] == "SHIP"
    assert v[("bf16", "fused_muon")]["verdict"] == "PARK"                   # all-on is slower than leaving it out
    assert "| bf16 | compile_full_path |" in out["markdown"]
    # a missing file: strict mode refuses, lenient mode reports it
    (runs / "bf16_stock_s1.json").unlink()
    with pytest.raises((P.CoverageError, P.QualityError)):
        P.summarize(m, runs)
    assert P.summarize(m, runs, lenient=True)["missing"] == ["bf16_stock_s1"]
    # a real error contaminates the matrix, a benign skip does not
    (runs / "bf16_all_s2.json").write_text(json.dumps({"config": {}, "error": "CUDA error: out of memory"}))
    with pytest.raises(P.QualityError):
        P.summarize(m, runs, lenient=True)
    (runs / "bf16_all_s2.json").write_text(json.dumps({"config": {}, "error": "skipped: fp8 not available"}))
    assert P.summarize(m, runs, lenient=True)["verdicts"][("bf16", "compile_full_path")]["n"] == 2
    # ambiguous pairing is an error of its own
    with pytest.raises(P.PairingError):
        P.resolve_coherent_pairs(m + [dict(m[3])])


def test_cli_exit_codes(tmp_path):
    mj = tmp_path / "matrix.json"
    assert P.main(["matrix", "--output", str(mj), "--seeds", "1", "2"]) == 0
    m = json.loads(mj.read_text())
    runs = tmp_path / "runs"
    runs.mkdir()
    assert P.main(["summarize", "--matrix-json", str(mj), "--runs-dir", str(runs)]) == 1   # every output missing: quality gate
    _fill(runs, m, lambda e: _res(100.0 + e["seed"]))
    assert P.main(["summarize", "--matrix-json", str(mj), "--runs-dir", str(runs), "--output", str(tmp_path / "o.md")]) == 0
    assert P.main(["summarize", "--matrix-json", str(tmp_path / "nope.json"), "--runs-dir", str(runs)]) == 4


def test_bench_bookkeeping_is_idempotent_and_pairs_four_ways(tmp_path):
    calls = []

    def fake(combo, seed, **kw):
        calls.append((P.combo_name(combo), seed))
        tps = 100.0 + 20.0 * combo["compile_full_path"] + 2.0 * combo["fused_muon"] + 0.01 * seed
        return {"combo": P.combo_name(combo), **combo, "seed": seed, "tokens_per_sec": tps, "final_loss": 3.5,
                "peak_vram_mb": 10.0}

    res = P.run_bench(tmp_path, seeds=[1, 2], measure=fake)
    assert len(calls) == 16 and len(res.read_text().splitlines()) == 16
    P.run_bench(tmp_path, seeds=[1, 2], measure=fake)
    assert len(calls) == 16                                                 # nothing re-measured
    rows = [json.loads(l) for l in res.read_text().splitlines()]
    d = P.paired_deltas(rows, "compile_full_path", "tokens_per_sec")
    assert d["n"] == 8 and d["mean"] == pytest.approx(20.0)
    assert "compile_full_path | tokens_per_sec | 8" in (tmp_path / "summary.md").read_text()
    assert P.split_steps(10, 4) == [3, 3, 2, 2] and P.split_steps(2, 4) == [1, 1]


def test_one_measurement_runs_on_cpu():
    row = P.run_one_measurement({"fused_grad_clip": False, "fused_muon": False, "compile_full_path": False}, 3,
                                model_cfg=dict(vocab_size=64, dim=32, num_layers=1, batch_size=2, seq_len=16, base_lr=0.01),
                                warmup_steps=1, n_timed_steps=2, n_blocks=2, device="cpu")
    assert row["combo"] == "stock" and row["tokens_per_sec"] > 0 and row["final_loss"] == row["final_loss"]
