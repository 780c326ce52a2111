"""Test-time-training ablation matrix and job queue (CPU)."""
import json
import types
from pathlib import Path

import pytest

from chaoscontrol_b200 import exp20


def _spec(tmp_path, **kw):
    return exp20.MatrixSpec(checkpoint_path=tmp_path / "ck.pt", sp_model_path=tmp_path / "sp.model",
                            jsonl_paths=[tmp_path / "docs.jsonl"], output_root=tmp_path / "res",
                            config_dir=tmp_path / "cfg", **kw)


def test_matrix_counts_and_names(tmp_path):
    cfgs = exp20.build_configs(_spec(tmp_path))
    by = {}
    for c in cfgs:
        by.setdefault(c["phase"], []).append(c)
    assert len(by["floor"]) == 2 * 3
    assert len(by["axis1"]) == 6 * 2 * 3
    # delta scales 0.5/1/2 and log_a shifts -0.5/0.5 (the identity appears once): 5 knobs x 3 seeds
    assert len(by["axis3"]) == 5 * 3
    names = [c["name"] for c in cfgs]
    assert len(set(names)) == len(names)
    assert "floor_carry_state_s2" in names
    assert "axis1_log_a+delta_proj_lr0p016_reset_s0" in names
    assert "axis3_log_a_shift_m0p5_reset_s1" in names
    floor = by["floor"][0]
    assert floor["steps_per_chunk"] == 0 and floor["adapt_set"] == "none"
    a1 = next(c for c in by["axis1"] if c["adapt_set"] == "lm_head")
    assert a1["steps_per_chunk"] == 1 and a1["eval_lr"] in (0.016, 0.064)
    a3 = next(c for c in by["axis3"] if "delta_scale_2" in c["name"])
    assert a3["delta_scale"] == 2.0 and a3["log_a_shift"] == 0.0 and a3["steps_per_chunk"] == 0


def test_phase_filter_winner_and_all_refused(tmp_path):
    cfgs = exp20.build_configs(_spec(tmp_path, phase="axis1", persistence_winner="carry_state", seeds=[7]))
    assert {c["phase"] for c in cfgs} == {"axis1"} and len(cfgs) == 12
    assert all(c["persistence_mode"] == "carry_state" and c["seed"] == 7 for c in cfgs)
    with pytest.raises(ValueError, match="all"):
        exp20.build_configs(_spec(tmp_path, phase="axis1", axis1_adapt_sets=["log_a", "all"]))
    with pytest.raises(ValueError, match="unknown phase"):
        exp20.build_configs(_spec(tmp_path, phase="axis9"))


def test_write_configs_manifest_and_run_config_roundtrip(tmp_path):
    spec = _spec(tmp_path, seeds=[0])
    cfgs = exp20.build_configs(spec)
    man = exp20.write_configs(spec, cfgs)
    assert man["total_configs"] == len(cfgs) == 2 + 12 + 5
    assert man["counts_by_phase"] == {"axis1": 12, "axis3": 5, "floor": 2}
    files = sorted(p.name for p in (tmp_path / "cfg").glob("*.json"))
    assert "manifest.json" in files and len(files) == len(cfgs) + 1
    from chaoscontrol_b200.eval_stream.types import RunConfig
    known = set(RunConfig.__dataclass_fields__)
    for c in cfgs:
        d = json.loads((tmp_path / "cfg" / f"{c['name']}.json").read_text())
        rc = RunConfig(**{k: v for k, v in d.items() if k in known})
        assert rc.adapt_set == c["adapt_set"] and rc.persistence_mode == c["persistence_mode"]


def test_queue_resume_round_robin_and_failures(tmp_path):
    spec = _spec(tmp_path, phase="floor", seeds=[0, 1])
    cfgs = exp20.build_configs(spec)
    exp20.write_configs(spec, cfgs)
    Path(cfgs[0]["summary_path"]).write_text("{}")
    pend, skipped = exp20.pending_configs(tmp_path / "cfg", resume=True)
    assert [n for n, _ in skipped] == [cfgs[0]["name"]] and len(pend) == 3
    pend2, skipped2 = exp20.pending_configs(tmp_path / "cfg", resume=False)
    assert len(pend2) == 4 and not skipped2

    dry = exp20.run_queue(tmp_path / "cfg", ["0", "1"], log_dir=tmp_path / "logs", resume=True, dry_run=True)
    assert [g for _, g, _ in dry["plan"]] == ["0", "1", "0"] and dry["ran"] == []

    seen = []

    def fake_run(cmd, env, stdout, stderr, text):
        seen.append((cmd, env["CUDA_VISIBLE_DEVICES"]))
        stdout.write("ran\n")
        name = Path(cmd[cmd.index("--config") + 1]).stem
        return types.SimpleNamespace(returncode=3 if name.endswith("carry_state_s1") else 0)

    res = exp20.run_queue(tmp_path / "cfg", ["4", "5"], log_dir=tmp_path / "logs", resume=True, runner=fake_run)
    assert sorted(res["ran"]) == sorted(c["name"] for c in cfgs[1:])
    assert [f["name"] for f in res["failures"]] == ["floor_carry_state_s1"] and res["failures"][0]["returncode"] == 3
    assert {g for _, g in seen} <= {"4", "5"}
    cmd = seen[0][0]
    assert cmd[1:3] == ["-m", "chaoscontrol_b200.eval_stream.run_eval"]
    assert "--jsonl-paths" in cmd and "--sp-model-path" in cmd
    log = (tmp_path / "logs" / f"{res['ran'][0]}.log").read_text()
    assert log.startswith("$ ") and "ran" in log


def test_cli_build_and_dry_queue(tmp_path, capsys):
    rc = exp20.main(["build", "--checkpoint-path", str(tmp_path / "c.pt"), "--config-dir", str(tmp_path / "cfg"),
                     "--output-root", str(tmp_path / "out"), "--phase", "floor", "--seeds", "0"])
    assert rc == 0 and json.loads(capsys.readouterr().out)["total_configs"] == 2
    rc = exp20.main(["queue", "--config-dir", str(tmp_path / "cfg"), "--gpus", "0", "--dry-run"])
    out = capsys.readouterr().out
    assert rc == 0 and out.count("RUN ") == 2


def test_run_eval_cli_takes_a_matrix_config(tmp_path, monkeypatch):
    from chaoscontrol_b200.eval_stream import run_eval
    spec = _spec(tmp_path, phase="axis1", seeds=[0], axis1_adapt_sets=["log_a"], axis1_eval_lrs=[0.016])
    cfgs = exp20.build_configs(spec)
    exp20.write_configs(spec, cfgs)
    got = {}

    def fake_run(cfg, **kw):
        got.update(cfg=cfg, **kw)
        return {"bpb": 1.0, "docs_scored": 0, "tokens_scored": 0, "adapt_steps": 0, "driver": "eager"}

    monkeypatch.setattr(run_eval, "run", fake_run)
    path = tmp_path / "cfg" / f"{cfgs[0]['name']}.json"
    assert run_eval.main(exp20.default_command("py", path)[3:]) == 0
    assert got["cfg"].adapt_set == "log_a" and got["cfg"].eval_lr == 0.016
    assert got["jsonl_paths"] == [str(tmp_path / "docs.jsonl")] and got["sp_model_path"] == str(tmp_path / "sp.model")
