"""Embedding-prior study: families, launcher plan, verdict report, registry import (CPU)."""
import json
import math
import types
from pathlib import Path

import pytest
import torch

from chaoscontrol_b200 import exp21


def _write(root, sub, cell, seed, bpb, *, nonfinite=False, loss=3.0):
    d = Path(root) / sub
    d.mkdir(parents=True, exist_ok=True)
    data = {"config": {"cell": cell, "seed": seed}, "eval": {"bpb": bpb}, "train": {"final_loss": loss, "elapsed_s": 600.0}}
    if nonfinite:
        data["nonfinite"] = {"flag": True, "reason": "loss"}
    (d / f"{cell}_s{seed}.json").write_text(json.dumps(data))


def test_families_and_entries():
    f = exp21.four_cell_family(0.032)
    assert list(f.conditions) == ["A_transformer_random", "B_transformer_sgns", "C_ssm_random", "D_ssm_sgns"]
    assert f.conditions["A_transformer_random"]["base_lr"] == 0.032 and f.conditions["C_ssm_random"]["base_lr"] == 0.064
    assert f.conditions["B_transformer_sgns"]["embed_init_path"] == exp21.SGNS_INIT
    assert f.conditions["A_transformer_random"]["model_type"] == "transformer_nanogpt_lean"
    es = f.entries(budget_seconds=60.0)
    assert len(es) == 20 and es[0]["name"] == "A_transformer_random_s1337" and es[0]["world_size"] == 2
    p0 = exp21.phase0_family()
    assert list(p0.conditions) == ["lr_0p016", "lr_0p032", "lr_0p064"] and len(p0.entries()) == 3
    ctl = {c.key: c for c in exp21.control_families()}
    assert ctl["zero"].conditions["ssm_zero"]["allow_nonfinite"] is True
    assert "allow_nonfinite" not in ctl["fullcov"].conditions["ssm_fullcov"]
    m = exp21.mechanism_family(exp21.parse_condition_names("ssm_norm_only, ssm_random_fullcov"))
    assert list(m.conditions) == ["ssm_norm_only", "ssm_random_fullcov"]
    assert len(exp21.mechanism_family().conditions) == 6
    with pytest.raises(ValueError, match="unknown mechanism"):
        exp21.mechanism_family(["nope"])
    assert exp21.parse_condition_names(" , ") is None


def test_artifact_validation(tmp_path):
    conds = exp21.mechanism_family(["ssm_norm_only"]).conditions
    with pytest.raises(FileNotFoundError, match="ssm_norm_only"):
        exp21.validate_embed_artifacts(conds, tmp_path)
    (tmp_path / "artifacts").mkdir()
    torch.save(torch.zeros(10, 4), tmp_path / "artifacts" / "sgns_init_norm_only.pt")
    with pytest.raises(ValueError, match="expected"):
        exp21.validate_embed_artifacts(conds, tmp_path)
    torch.save(torch.zeros(8192, 256), tmp_path / "artifacts" / "sgns_init_norm_only.pt")
    exp21.validate_embed_artifacts(conds, tmp_path)


def test_launcher_slots_skip_and_failure(tmp_path):
    fam = exp21.Family("t", "t", {"c": exp21.ssm_cell(embed_init_path=None)}, seeds=(1, 2, 3))
    _write(tmp_path, "t", "c", 1, 1.5)
    dry = exp21.run_family(fam, results_root=tmp_path, data_path="/d", sp_model_path="/m", dry_run=True)
    assert dry["skipped"] == ["c_s1"] and [c["name"] for c in dry["commands"]] == ["c_s2", "c_s3"]
    cmd = dry["commands"][0]["cmd"]
    assert "chaoscontrol_b200.runner_exp21" in cmd and "--nproc-per-node=2" in cmd and "127.0.0.1" in cmd
    assert exp21.slot_gpus(2, 2) == ["0,1", "2,3"]
    seen = []

    def fake(cmd, env, capture_output, text):
        out = Path(cmd[cmd.index("--output-json") + 1])
        seen.append(env["CUDA_VISIBLE_DEVICES"])
        if out.stem == "c_s3":
            return types.SimpleNamespace(returncode=1, stderr="boom")
        out.write_text(json.dumps({"eval": {"bpb": 1.4}, "train": {"final_loss": 2.0}}))
        return types.SimpleNamespace(returncode=0, stderr="")

    plan = exp21.run_family(fam, results_root=tmp_path, data_path="/d", sp_model_path="/m", runner=fake)
    assert plan["failed"] == ["c_s3"] and set(seen) <= {"0,1", "2,3"}
    assert json.loads((tmp_path / "t" / "c_s3.json").read_text())["error"] == "boom"
    s = exp21.summarize_family(fam, tmp_path)
    assert s["rows"]["c"]["n"] == 3 and s["rows"]["c"]["finite"] == 2 and s["rows"]["c"]["mean_bpb"] == pytest.approx(1.45)


def test_phase0_winner_and_transformer_lr(tmp_path):
    _write(tmp_path, "phase0", "lr_0p016", 1337, 1.60)
    _write(tmp_path, "phase0", "lr_0p032", 1337, 1.52)
    _write(tmp_path, "phase0", "lr_0p064", 1337, float("nan"))
    s = exp21.phase0_summary(tmp_path)
    assert s["winner_condition"] == "lr_0p032" and s["winner_lr"] == 0.032 and len(s["rows"]) == 3
    with pytest.raises(FileNotFoundError):
        exp21.load_transformer_lr(tmp_path)
    (tmp_path / "phase0" / "phase0_summary.json").write_text(json.dumps(s))
    assert exp21.load_transformer_lr(tmp_path) == 0.032 and exp21.load_transformer_lr(tmp_path, 0.1) == 0.1


def test_one_sided_t_matches_closed_form():
    # differences 1, 2, 3: t = 2 / (1 / sqrt 3) = 3.4641, df = 2 -> two-sided p = 0.07418
    p = exp21.paired_t_one_sided([2.0, 4.0, 6.0], [1.0, 2.0, 3.0])
    assert p == pytest.approx(0.07418 / 2, rel=1e-3)
    assert exp21.paired_t_one_sided([1.0, 2.0, 3.0], [2.0, 4.0, 6.0]) == pytest.approx(1 - 0.07418 / 2, rel=1e-3)
    assert exp21.paired_t_one_sided([1.0, 2.0, 3.0], [2.0, 4.0, 6.0], "less") == pytest.approx(0.07418 / 2, rel=1e-3)
    assert exp21.paired_t_one_sided([1.0, 2.0], [1.0, 2.0]) == 0.5
    assert exp21.paired_t_one_sided([2.0, 3.0], [1.0, 2.0]) == 0.0
    with pytest.raises(ValueError):
        exp21.paired_t_one_sided([1.0], [1.0])
    with pytest.raises(ValueError):
        exp21.paired_t_one_sided([1.0, 2.0], [1.0, 2.0], "two-sided")


def _full_study(root, *, control_gap):
    seeds = exp21.MAIN_SEEDS
    for i, s in enumerate(seeds):
        j = 0.001 * i
        _write(root, "four_cell", "A_transformer_random", s, 1.500 + j)
        _write(root, "four_cell", "B_transformer_sgns", s, 1.495 + j * 1.1)
        _write(root, "four_cell", "C_ssm_random", s, 1.480 + j)
        _write(root, "four_cell", "D_ssm_sgns", s, 1.440 + j * 0.8)
        _write(root, "fullcov", "ssm_fullcov", s, 1.440 + control_gap + j * 0.7)
        _write(root, "shuffled", "ssm_shuffled", s, 1.440 + control_gap + j * 1.3)
        _write(root, "zero", "ssm_zero", s, 1.60 + j, nonfinite=(i == 0))


def test_report_validating_then_weak(tmp_path):
    _full_study(tmp_path / "a", control_gap=0.03)
    warns = []
    r = exp21.build_report(tmp_path / "a", warn=warns.append)
    assert r["n_common_seeds"] == 5 and r["p_primary"] < 0.01 and r["p_secondary"] < 0.01
    assert r["controls_complete"] and r["controls_support_semantics"] and r["thesis_validating"] and not r["thesis_weak"]
    assert r["delta_ssm_mean"] == pytest.approx(0.04 + 0.0002 * 2, abs=1e-6)
    assert r["n_zero_pairs"] == 4 and r["zero"]["n"] == 4 and any("flagged non-finite" in w for w in warns)
    text = exp21.format_report(r)
    assert "thesis-validating: True" in text and "== controls ==" in text

    _full_study(tmp_path / "b", control_gap=0.0)          # controls as good as the real table
    r2 = exp21.build_report(tmp_path / "b", warn=lambda _m: None)
    assert r2["p_primary"] < 0.01 and not r2["controls_support_semantics"]
    assert not r2["thesis_validating"] and r2["thesis_weak"]


def test_report_partial_state(tmp_path):
    _write(tmp_path, "four_cell", "C_ssm_random", 42, 1.5)
    _write(tmp_path, "four_cell", "D_ssm_sgns", 42, 1.4)
    r = exp21.build_report(tmp_path, warn=lambda _m: None)
    assert r["p_primary"] is None and r["n_common_seeds"] == 0 and not r["thesis_validating"] and not r["thesis_weak"]
    assert math.isnan(r["delta_ssm_mean"]) and "n/a" in exp21.format_report(r)


def test_register_all_gates_on_canonical(tmp_path):
    _write(tmp_path / "res", "four_cell", "C_ssm_random", 42, 1.5)
    _write(tmp_path / "res", "zero", "ssm_zero", 42, float("nan"), nonfinite=True)
    _write(tmp_path / "res", "four_cell", "unrelated_cell", 42, 1.0)
    reg, canon = tmp_path / "reg.jsonl", tmp_path / "canon.json"
    assert exp21.register_all(tmp_path / "none", say=lambda _m: None) == 1
    assert exp21.register_all(tmp_path / "res", registry_path=reg, canonical_path=canon, say=lambda _m: None) == 2
    assert not reg.exists()
    h = exp21.config_hash({"cell": "C_ssm_random", "seed": 42})
    canon.write_text(json.dumps({"canonical": {h: {"experiment": "exp21", "condition": "C_ssm_random"}}}))
    assert exp21.register_all(tmp_path / "res", registry_path=reg, canonical_path=canon, say=lambda _m: None) == 0
    rows = [json.loads(x) for x in reg.read_text().splitlines()]
    assert len(rows) == 1 and rows[0]["condition"] == "C_ssm_random" and rows[0]["metrics"]["bpb"] == 1.5
    reg2 = tmp_path / "reg2.jsonl"
    assert exp21.register_all(tmp_path / "res", status="exploratory", registry_path=reg2, say=lambda _m: None) == 0
    rows = [json.loads(x) for x in reg2.read_text().splitlines()]
    assert len(rows) == 2 and {r["condition"] for r in rows} == {"C_ssm_random", "ssm_zero"}
    assert [r for r in rows if r["condition"] == "ssm_zero"][0]["metrics"]["nonfinite_flag"] == 1.0


def test_cli_dry_run_and_analyze(tmp_path, capsys):
    assert exp21.main(["run", "phase0", "--results-root", str(tmp_path), "--data-path", "/d", "--sp-model-path", "/m",
                       "--dry-run"]) == 0
    out = capsys.readouterr().out
    assert out.count("CUDA_VISIBLE_DEVICES=") == 3
    _full_study(tmp_path, control_gap=0.03)
    assert exp21.main(["analyze", "--results-root", str(tmp_path), "--json-out", str(tmp_path / "r.json")]) == 0
    assert json.loads((tmp_path / "r.json").read_text())["thesis_validating"] is True
