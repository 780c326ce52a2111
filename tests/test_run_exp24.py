"""Bundle launcher: matrix dispatch, defaults, dry run, smoke-result checks."""
import json

import pytest

from chaoscontrol_b200 import run_exp24 as R


def test_defaults_per_matrix():
    assert R.default_world_size("scopt_overhead_gate") == 1 and R.default_world_size("cd_multiseed") == 1
    assert R.default_world_size("crct_v1") == 4 and R.default_world_size("all") == 8
    assert R.default_budget("semantic_overhead_gate") == 90.0 and R.default_budget("crct_v1") == 600.0
    assert R.default_budget("scopt_calibration_sweep") == 1200.0


def test_build_entries_dispatch():
    kw = dict(speed_config={"batch_size": 8}, world_size=2, budget_seconds=5.0)
    assert len(R.build_entries(matrix="scopt_overhead_gate", seeds=[1, 2], **kw)) == 4      # per-seed builder
    assert len(R.build_entries(matrix="crct_v1", seeds=[1], **kw)) == 4
    allm = R.build_entries(matrix="all", seeds=[1], **kw)
    assert len(allm) == 1 + 3 + 2 + 6 and all(e["world_size"] == 2 for e in allm)
    with pytest.raises(ValueError, match="unsupported matrix"):
        R.build_entries(matrix="nope", seeds=[1], **kw)
    for name in R.MATRICES:
        assert R.build_entries(matrix=name, seeds=[7], **kw)


def test_dry_run_writes_matrix_and_commands(tmp_path, capsys, monkeypatch):
    monkeypatch.setenv("EPISODIC_CONTROLLER_V1_TRACE_DIR", str(tmp_path / "traces"))
    cfg = tmp_path / "speed.yaml"
    cfg.write_text("batch_size: 8\nseq_len: 16\n")
    rc = R.main(["--matrix", "episodic_controller_v1", "--config", str(cfg), "--output-dir", str(tmp_path / "out"),
                 "--seeds", "3", "--dry-run", "--limit", "2", "--full-val-score", "--val-cache-dir",
                 str(tmp_path / "val"), "--data-path", str(tmp_path / "d")])
    assert rc == 0
    matrix = json.loads((tmp_path / "out" / "matrix.json").read_text())
    assert len(matrix) == 6 and (tmp_path / "traces").is_dir()
    out = capsys.readouterr().out
    summary = json.loads(out[out.index("{\n"):])
    assert len(summary["commands"]) == 2 and len(summary["full_val_commands"]) == 2
    cmd = summary["commands"][0]
    assert "--nproc-per-node=4" in cmd and "--output-ckpt" in cmd and "127.0.0.1" in cmd
    assert "chaoscontrol_b200.fast_score" in summary["full_val_commands"][0]
    assert not list((tmp_path / "out").glob("exp24_*.json"))                   # nothing ran


def test_full_val_pass_routes_ttt_cells_to_the_adapting_driver(tmp_path):
    entries = R.build_entries(matrix="episodic_ttt_v1", speed_config={}, world_size=4, budget_seconds=5.0, seeds=[1])
    cmds = R.full_val_commands(entries=entries, checkpoint_dir=tmp_path / "ck", results_dir=tmp_path / "res",
                               world_size=4, cache_dir=tmp_path / "val", budget_seconds=60.0, dry_run=True)
    assert len(cmds) == 4
    kinds = ["run_eval" if "chaoscontrol_b200.eval_stream.run_eval" in c else "fast_score" for c in cmds]
    assert kinds == ["fast_score", "run_eval", "fast_score", "run_eval"]          # arms a, b, c, d
    ttt = cmds[1]
    assert ttt[ttt.index("--adapt-set") + 1] == "lm_head" and ttt[ttt.index("--steps-per-chunk") + 1] == "1"


def _result(tmp_path, train):
    p = tmp_path / "r.json"
    p.write_text(json.dumps({"config": {}, "train": train}))
    return p


def test_smoke_check_catches_silent_fallbacks(tmp_path):
    entry = {"name": "smoke_x_arm_e_simplex_warm_online_s1", "episodic_enabled": True,
             "controller_query_enabled": True,
             "episodic_controller_simplex_trace_path": str(tmp_path / "t.ndjson")}
    ok, fails = R.smoke_check_result(result_path=tmp_path / "missing.json", entry=entry)
    assert not ok and "not produced" in fails[0]
    bad = tmp_path / "bad.json"
    bad.write_text("{")
    assert "malformed" in R.smoke_check_result(result_path=bad, entry=entry)[1][0]
    err = tmp_path / "err.json"
    err.write_text(json.dumps({"error": "boom"}))
    assert "boom" in R.smoke_check_result(result_path=err, entry=entry)[1][0]
    assert "missing train" in R.smoke_check_result(result_path=_result(tmp_path, {}), entry=entry)[1][0]

    quiet = {"steps": 5, "episodic": {"enabled": True, "role": "solo", "write_events_emitted": 0,
                                      "write_events_ingested": 0, "replays": 0}}
    ok, fails = R.smoke_check_result(result_path=_result(tmp_path, quiet), entry=entry)
    text = " ".join(fails)
    assert not ok and "write_events_emitted=0" in text and "replays=0" in text and "trace not produced" in text

    live = {"steps": 5, "episodic": {"enabled": True, "role": "solo", "write_events_emitted": 40,
                                     "write_events_ingested": 40, "replays": 6, "write_events_dropped": 0}}
    rows = [{"row_type": "decision", "entropy": 2.76}, {"row_type": "decision", "entropy": 2.75}]
    (tmp_path / "t.ndjson").write_text("\n".join(json.dumps(r) for r in rows) + "\nnot json\n")
    ok, fails = R.smoke_check_result(result_path=_result(tmp_path, live), entry=entry)
    assert not ok and any("no credit rows" in f for f in fails) and any("entropy > 2.5" in f for f in fails)
    rows += [{"row_type": "decision", "entropy": 1.9}, {"row_type": "credit"}]
    (tmp_path / "t.ndjson").write_text("\n".join(json.dumps(r) for r in rows))
    assert R.smoke_check_result(result_path=_result(tmp_path, live), entry=entry) == (True, [])
    off = {"name": "control", "episodic_enabled": False}
    assert R.smoke_check_result(result_path=_result(tmp_path, {"steps": 1}), entry=off) == (True, [])


def test_smoke_without_registered_arm_is_skipped(tmp_path):
    ok, msgs = R.run_smoke(matrix="crct_v1", entries=[], data_path="d", sp_model_path=None,
                           results_dir=tmp_path, world_size=1)
    assert ok and "smoke skipped" in msgs[0]
    ok, msgs = R.run_smoke(matrix="episodic_controller_v1", entries=[{"name": "other"}], data_path="d",
                           sp_model_path=None, results_dir=tmp_path, world_size=1)
    assert not ok and "matched no entries" in msgs[0]


# ---------------------------------------------------------------------------
# every mechanism family of the bundle runs through the production runner (CPU, one rank)
# ---------------------------------------------------------------------------
_TINY = dict(vocab_size=64, model_dim=16, num_layers=2, ff_mult=2, seq_len=16, stride=8, batch_size=4,
             dtype="fp32", precision="fp32", device="cpu", optimizer="muon", base_lr=0.02, warmup_steps=0,
             max_steps=6, eval_batches=0, lm_head_backward_mode="fused", stop_check_interval=2,
             episodic_capacity=64, episodic_writes_per_step=4, episodic_fingerprint_window=2,
             episodic_controller_sgd_interval=2, criticality_distill_num_layers=2, criticality_distill_dim=16)

_CELLS = [("first_wave", "fastslow_i32_a050", "fast_slow"),
          ("first_wave", "spectral_dead", "spectral"),
          ("first_wave", "predictive_h4", "predictive_aux"),
          ("first_wave", "eventsleep", "dreamworld"),
          ("scopt_overhead_gate", "scopt_gate_scopt", "scopt"),
          ("semantic_overhead_gate", "semantic_gate_semantic", None),
          ("phase_a_sampling", "shuffled_epoch", None),
          ("cd_first_smoke", "treatment", "criticality_distillation"),
          ("episodic_controller_v1", "arm_f_simplex_sharp_online", "episodic"),
          ("crct_v1", "arm_d_crct_replay_active", "crct")]


@pytest.mark.parametrize("matrix,arm,block", _CELLS)
def test_bundle_cell_runs_through_the_runner(tmp_path, monkeypatch, matrix, arm, block):
    import numpy as np
    from chaoscontrol_b200.episodic import native
    from chaoscontrol_b200.episodic.controller import save_simplex_policy
    from chaoscontrol_b200.runner_fast_path import run_condition
    rng = np.random.default_rng(0)
    rng.integers(0, 64, 20000, dtype=np.uint16).tofile(tmp_path / "fineweb_train_000.bin")
    rng.integers(0, 64, 5000, dtype=np.uint16).tofile(tmp_path / "fineweb_val_000.bin")
    save_simplex_policy(tmp_path / "w.pt", native.SimplexPolicy(seed=1))
    monkeypatch.setenv("EPISODIC_CONTROLLER_V1_WEIGHTS_PATH", str(tmp_path / "w.pt"))
    monkeypatch.setenv("EPISODIC_CONTROLLER_V1_TRACE_DIR", str(tmp_path / "traces"))
    entries = R.build_entries(matrix=matrix, speed_config=_TINY, world_size=1, budget_seconds=60.0, seeds=[3])
    entry = dict(next(e for e in entries if arm in e["name"]))
    # the locked sizes are for the full model; shrink what scales with it, keep every switch
    entry.update(batch_size=4)
    shrink = {"outer_max_slots": 0, "outer_model_dim": 8, "prototype_dim": 8, "dreamworld_replay_batch_size": 2,
              "dreamworld_prefix_tokens": 8, "dreamworld_replay_tokens": 4, "scopt_warmup_steps": 2}
    entry.update({k: v for k, v in shrink.items() if entry.get(k)})
    for key in ("replay_eviction_trace_path", "crct_gradient_conflict_trace_path"):
        if entry.get(key):
            entry[key] = str(tmp_path / key)
    res = run_condition(entry, data_path=str(tmp_path), sp_model_path=None, budget_seconds=60.0, output_json=None,
                        output_ckpt=None, world_size_override=None)
    tr = res["train"]
    assert tr["steps"] == 6 and np.isfinite(tr["final_loss"])
    if block:
        assert block in tr, sorted(tr)
    if block == "scopt":
        # every fourth step is a split step once the optimizer's warm-up allows writes: rare gradients and
        # channel pressures reached the optimizer
        assert 1 <= tr["scopt"]["split_steps"] <= 2 and tr["scopt"]["trace"]["step"] == 6
        assert "row_pressure" in tr["scopt"]["trace"] and "pressure_stats" in tr["scopt"]["trace"]
    if block == "spectral":
        assert tr["spectral"]["regularized_steps"] == 6
    if block == "predictive_aux":
        assert tr["predictive_aux"]["steps"] == 6 and np.isfinite(tr["predictive_aux"]["last_loss"])
    if block == "episodic":
        c = tr["episodic"]["controller"]
        assert c["temperature"] == pytest.approx(0.2) and c["train_online"] and c["decisions"] >= 1
        trace = tmp_path / "traces" / f"episodic_controller_v1_{arm}_s3.ndjson"
        assert trace.exists() and '"row_type":"decision"' in trace.read_text()
        ok, fails = R.smoke_check_result(
            result_path=_result(tmp_path, json.loads(json.dumps(tr, default=str))), entry=entry)
        assert ok or all("entropy" in f or "credit" in f for f in fails), fails
