"""Command lines of the three runners: what they read and what they hand to the run functions (CPU)."""
import json

import pytest

from chaoscontrol_b200 import runner, runner_exp21, runner_fast_path, runner_persistent_ddp


def _capture(monkeypatch, module, name, result=None):
    seen = {}

    def fake(*args, **kw):
        seen["args"], seen["kw"] = args, kw
        return result if result is not None else {}
    monkeypatch.setattr(module, name, fake)
    return seen


def test_fast_path_cli_reads_yaml_and_budget_precedence(tmp_path, monkeypatch):
    cfg = tmp_path / "c.yaml"
    cfg.write_text("name: x\nbudget_seconds: 12.5\nmodel_dim: 16\n")
    seen = _capture(monkeypatch, runner_fast_path, "run_condition")
    assert runner_fast_path.main(["--config", str(cfg), "--data-path", "/d"]) == 0
    assert seen["args"][0] == {"name": "x", "budget_seconds": 12.5, "model_dim": 16}
    assert seen["kw"]["budget_seconds"] == 12.5 and seen["kw"]["data_path"] == "/d" and seen["kw"]["sp_model_path"] is None
    assert seen["kw"]["world_size_override"] is None and seen["kw"]["val_cache_dir"] is None
    runner_fast_path.main(["--config", str(cfg), "--data-path", "/d", "--budget", "3", "--sp-model-path", "m", "--world-size",
                           "2", "--output-json", "o.json", "--output-ckpt", "o.pt", "--val-cache-dir", "vc"])
    kw = seen["kw"]
    assert (kw["budget_seconds"], kw["sp_model_path"], kw["world_size_override"]) == (3.0, "m", 2)
    assert (kw["output_json"], kw["output_ckpt"], kw["val_cache_dir"]) == ("o.json", "o.pt", "vc")
    cfg.write_text("name: y\n")
    runner_fast_path.main(["--config", str(cfg), "--data-path", "/d"])
    assert seen["kw"]["budget_seconds"] == 90.0                         # neither flag nor config: the default


def test_exp21_cli_requires_the_tokenizer_and_passes_everything_on(tmp_path, monkeypatch):
    cfg = tmp_path / "c.yaml"
    cfg.write_text("model_type: ssm\nmodel_dim: 16\n")
    seen = _capture(monkeypatch, runner_exp21, "run_ddp")
    with pytest.raises(SystemExit):
        runner_exp21.main(["--config", str(cfg), "--data-path", "/d"])
    assert runner_exp21.main(["--config", str(cfg), "--data-path", "/d", "--sp-model-path", "m", "--budget", "7",
                              "--output-json", "o.json", "--world-size", "2"]) == 0
    assert seen["args"][0] == {"model_type": "ssm", "model_dim": 16}
    kw = seen["kw"]
    assert (kw["data_path"], kw["sp_model_path"], kw["budget_seconds"], kw["output_json"], kw["world_size_override"],
            kw["output_ckpt"]) == ("/d", "m", 7.0, "o.json", 2, None)


def test_legacy_cli_writes_the_result_file(tmp_path, monkeypatch, capsys):
    seen = _capture(monkeypatch, runner, "run_experiment", result={"eval": {"bpb": 1.25}, "path": tmp_path})
    out = tmp_path / "deep" / "r.json"
    assert runner.main(["--config", "c.yaml", "--enwik8-path", "/d", "--budget", "5", "--output-json", str(out),
                        "--checkpoint-dir", "ck", "--checkpoint-name", "n"]) == 0
    assert seen["args"] == ("c.yaml",) and seen["kw"] == {"data_path": "/d", "budget_seconds": 5.0, "checkpoint_dir": "ck",
                                                           "checkpoint_name": "n"}
    assert json.loads(out.read_text())["eval"]["bpb"] == 1.25 and "Saved to" in capsys.readouterr().out
    runner.main(["--config", "c.yaml", "--data-path", "/d"])
    assert seen["kw"]["budget_seconds"] == 300 and capsys.readouterr().out == ""


def test_persistent_worker_runs_one_seed_through_the_production_entry_point(tmp_path, monkeypatch):
    seen = _capture(monkeypatch, runner_fast_path, "run_condition", result={"train": {}, "eval": {}})
    applied = []
    monkeypatch.setattr(runner_persistent_ddp, "apply_seed", applied.append)
    cfg = {"name": "a", "seed": 9, "model_dim": 16}
    res = runner_persistent_ddp.run_one_seed(config=cfg, out_path=tmp_path / "a_s9.json", data_path="/d", sp_model_path=None,
                                             budget_seconds=4, world_size=2)
    assert res == {"train": {}, "eval": {}} and applied == [9] and seen["args"][0] == cfg and seen["args"][0] is not cfg
    kw = seen["kw"]
    assert kw["keep_process_group"] is True and kw["output_json"] == str(tmp_path / "a_s9.json") and kw["output_ckpt"] is None
    assert kw["budget_seconds"] == 4.0 and kw["world_size_override"] == 2
    assert runner_persistent_ddp.fp8_is_available() in (True, False)
