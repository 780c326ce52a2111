"""Throughput-lever screens: matrix shape, rate inheritance contract, decision gates on synthetic result files."""
import json
import math

import pytest

from chaoscontrol_b200 import exp18


def _write(rdir, cond, seed, bpb, loss=3.5, tps=1e6, ws=1, vocab=16384):
    rdir.mkdir(parents=True, exist_ok=True)
    (rdir / f"{cond}_s{seed}.json").write_text(json.dumps({
        "config": {"world_size": ws, "vocab_size": vocab}, "eval": {"bpb": bpb},
        "train": {"final_loss": loss, "aggregate_tokens_per_sec": tps}}))


def test_every_test_builds_a_matrix_with_one_varying_axis():
    for key, t in exp18.TESTS.items():
        entries = exp18.build_entries(key, base_lr=0.064)
        conds = {e["condition"] for e in entries}
        assert len(entries) == len(conds) * len(t.seeds)
        assert all(e["name"] == f"{e['condition']}_s{e['seed']}" for e in entries)
        cfgs = t.conditions(0.064)
        keys = set().union(*[set(c) for c in cfgs.values()])
        varying = {k for k in keys if len({json.dumps(c.get(k)) for c in cfgs.values()}) > 1}
        assert 1 <= len(varying) <= 3, (key, varying)       # the axis itself plus what it forces (stride, lr, ws)


def test_rates_follow_the_linear_rule():
    assert exp18.linear_lr(32) == pytest.approx(2e-3)
    t5 = exp18.TESTS["test5"].conditions(None)
    assert [t5[c]["base_lr"] for c in ("lr_linear", "lr_half", "lr_quarter")] == pytest.approx([0.064, 0.032, 0.016])
    t5b = exp18.TESTS["test5b"].conditions(None)
    assert t5b["lr_linear"]["base_lr"] == pytest.approx(0.128) and t5b["lr_half"]["optimizer"] == "muon"
    t4 = exp18.TESTS["test4"].conditions(None)
    assert t4["ws2_ddp"]["base_lr"] == pytest.approx(2 * t4["ws1"]["base_lr"])


def test_inheriting_tests_refuse_a_missing_or_provisional_rate(tmp_path):
    with pytest.raises(ValueError):
        exp18.build_entries("test6")                                        # no rate, nowhere to read one
    with pytest.raises(FileNotFoundError):
        exp18.build_entries("test7", results_root=tmp_path)
    d = tmp_path / "results_test5"
    d.mkdir()
    (d / "test5_summary.json").write_text(json.dumps({"_decision": {"winner_base_lr": 0.032, "winner_is_provisional": True}}))
    with pytest.raises(ValueError, match="provisional"):
        exp18.build_entries("test6", results_root=tmp_path)
    (d / "test5_summary.json").write_text(json.dumps({"_decision": {"winner_base_lr": 0.032, "winner_is_provisional": False}}))
    e = exp18.build_entries("test6", results_root=tmp_path)
    assert {x["base_lr"] for x in e} == {0.032} and {x["seq_len"] for x in e} == {512, 1024, 2048}
    assert exp18.build_entries("test6", base_lr=0.05)[0]["base_lr"] == 0.05  # explicit override wins


def test_launch_plan_packs_gpus():
    e = exp18.build_entries("test3", seeds=[1, 2, 3, 4])
    waves = exp18.launch_plan(e, 4)
    assert [len(w) for w in waves] == [4, 4, 4]
    e = exp18.build_entries("test5", seeds=[1, 2])
    assert [len(w) for w in exp18.launch_plan(e, 4)] == [2, 2, 2]            # two 2-GPU groups at a time
    with pytest.raises(ValueError):
        exp18.launch_plan(exp18.build_entries("test10", seeds=[1]), 2)


def test_rate_screen_gate(tmp_path):
    r = tmp_path / "results_test5"
    seeds = [1, 2, 3, 4]
    for i, s in enumerate(seeds):
        _write(r, "lr_linear", s, 1.50 + 0.001 * i, loss=9.6)               # stalled near ln V: unstable
        _write(r, "lr_half", s, 1.600 + 0.001 * i)
        _write(r, "lr_quarter", s, 1.602 + 0.001 * (3 - i))
    s = exp18.decide("test5", r)
    dec = s["_decision"]
    assert dec["stable_conditions"] == ["lr_half", "lr_quarter"]
    # half and quarter are 0.002 apart with crossing seeds: inside noise -> the calmer rate, and provisional without a cohort
    assert dec["stage1_candidate"] == "lr_quarter" and dec["winner_is_provisional"] is True
    assert dec["winner_base_lr"] == pytest.approx(0.016)
    base = {sd: 1.70 + 0.001 * i for i, sd in enumerate(seeds)}
    dec2 = exp18.decide("test5", r, baseline_bpb_by_seed=base)["_decision"]
    assert dec2["winner_lr_condition"] == "lr_quarter" and dec2["winner_is_provisional"] is False
    worse = {sd: 1.50 for sd in seeds}
    assert exp18.decide("test5", r, baseline_bpb_by_seed=worse)["_decision"]["winner_lr_condition"] is None


def test_ddp_and_fp8_gates(tmp_path):
    r = tmp_path / "results_test4"
    for i, s in enumerate([1, 2, 3, 4]):
        _write(r, "ws1", s, 1.70 + 0.002 * i, tps=1.0e6, ws=1)
        _write(r, "ws2_ddp", s, 1.65 + 0.002 * i + 0.0005 * (i % 2), tps=1.8e6, ws=2)
    v = exp18.decide("test4", r)["_decision"]
    assert v["winner"] == "ws2_ddp" and v["verdicts"]["ws2_ddp"]["per_gpu_rate_ratio"] == pytest.approx(0.9)
    _write(r, "ws2_ddp", 1, 1.65, tps=1.2e6, ws=2)
    _write(r, "ws2_ddp", 2, 1.652, tps=1.2e6, ws=2)
    _write(r, "ws2_ddp", 3, 1.6545, tps=1.2e6, ws=2)
    _write(r, "ws2_ddp", 4, 1.6565, tps=1.2e6, ws=2)
    assert exp18.decide("test4", r)["_decision"]["winner"] == "ws1"          # 0.6 of the per-GPU rate: below the floor

    r = tmp_path / "results_test10"
    for i, s in enumerate([1, 2, 3, 4]):
        _write(r, "bf16", s, 1.50 + 0.001 * i, tps=10e6, ws=4)
        _write(r, "fp8", s, 1.505 + 0.001 * i + 0.0003 * (i % 2), tps=14e6, ws=4)
    d = exp18.decide("test10", r)["_decision"]
    assert d["winner"] == "fp8" and d["speedup"] == pytest.approx(1.4)
    for i, s in enumerate([1, 2, 3, 4]):
        _write(r, "fp8", s, 1.505, loss=9.69, tps=14e6, ws=4)               # collapsed
    assert exp18.decide("test10", r)["_decision"]["winner"] == "bf16"


def test_non_finite_results_are_listed_not_used(tmp_path):
    r = tmp_path / "results_test7"
    for s in (1, 2, 3):
        _write(r, "adamw_baseline", s, 1.60 + 0.001 * s)
        _write(r, "muon", s, 1.40 + 0.0012 * s)
    _write(r, "lamb", 1, float("nan"))
    out = exp18.decide("test7", r, base_lr=0.032)
    assert out["_decision"]["invalid_result_files"] == ["lamb_s1"] and "lamb" not in out
    assert out["_decision"]["winner"] == "muon"


def test_dry_run_emits_torchrun_commands(tmp_path):
    out = exp18.run_test("test4b", results_root=tmp_path, data_path="/data", sp_model_path=None, seeds=[7], dry_run=True)
    assert len(out["commands"]) == 2
    assert any("--nproc-per-node=4" in c for cmd in out["commands"] for c in cmd)
    assert all("127.0.0.1" in cmd for cmd in out["commands"])
