"""Run-matrix builders: entry counts, names, locked keys, arm selection."""
import json

import pytest

from chaoscontrol_b200 import exp24

SPEED = {"batch_size": 1024, "seq_len": 512, "eval_batches": "8",
         "dreamworld_buffer_size": 32, "nested": {"a": [1, 2]}}


def test_base_entry_normalises_and_copies():
    e = exp24._base_entry(speed_config=SPEED, world_size=4, budget_seconds=30)
    assert e["mode"] == "exp24_training_time_bundle"
    assert e["world_size"] == 4 and e["budget_seconds"] == 30.0
    assert e["eval_batches"] == 8 and isinstance(e["eval_batches"], int)
    assert e["dreamworld_buffer_size"] == 32          # speed config wins over default
    assert e["fast_slow_eval_copy"] == "fast" and e["optimizer_param_grouping"] == "flat"
    assert e["spectral_reg_max_a"] == 0.98 and e["event_sleep_loss_ratio"] == 1.10
    e["nested"]["a"].append(3)
    assert SPEED["nested"]["a"] == [1, 2]


def test_named_entry_phase_and_first_wave():
    a = exp24._named_entry(base={}, phase="phase0", mechanism="m", arm="x", seed=7)
    b = exp24._named_entry(base={}, phase=None, mechanism="m", arm="x", seed=7)
    assert a["name"] == "exp24_phase0_x_s7" and a["exp24_phase"] == "phase0"
    assert b["name"] == "exp24_x_s7" and b["exp24_phase"] == "first_wave"


@pytest.mark.parametrize("builder,count", [
    ("ring0_control_matrix", 3), ("phase_a_sampling_matrix", 3),
    ("semantic_overhead_gate_matrix", 2), ("scopt_overhead_gate_matrix", 2),
    ("scopt_calibration_sweep_matrix", 3), ("first_wave_mechanism_matrix", 18),
    ("first_wave_matrix", 18), ("fastslow_dreamworld_matrix", 3),
    ("phase0_dreamworld_sweep", 9), ("phase0_fastslow_sweep", 18),
    ("phase0_confirm", 6), ("phase0_fastslow_only_control", 3),
    ("episodic_dw_curation_v1_matrix", 12), ("episodic_controller_v1_matrix", 18),
    ("episodic_ttt_v1_matrix", 12), ("crct_v1_matrix", 12),
    ("criticality_distillation_first_smoke_matrix", 24),
    ("criticality_distillation_multiseed_matrix", 25),
])
def test_matrix_sizes_and_unique_names(builder, count):
    entries = exp24.MATRIX_BUILDERS[builder](speed_config=SPEED)
    assert len(entries) == count
    names = [e["name"] for e in entries]
    assert len(set(names)) == count and all(n.startswith("exp24_") for n in names)
    for e in entries:
        assert e["batch_size"] in (1024, 512) and e["seq_len"] == 512
        assert isinstance(e["seed"], int)
        json.dumps(e)                                   # plain data only


def test_first_wave_arms():
    entries = exp24.build_first_wave_mechanism_matrix(speed_config=SPEED, seed_values=(1,))
    by = {e["exp24_mechanism"]: e for e in entries}
    assert list(by) == ["fast_slow", "spectral", "predictive_aux", "dreamworld",
                        "fast_slow_dreamworld", "fast_slow_dreamworld_event_sleep"]
    assert by["fast_slow"]["name"] == "exp24_fastslow_i32_a050_s1"
    assert by["fast_slow"]["fast_slow_alpha"] == 0.5
    assert by["spectral"]["artifact_impact"] == exp24.ARTIFACT_CHANGES_WEIGHTS_ONLY
    assert by["dreamworld"]["dreamworld_replay_batch_size"] == 0
    assert by["fast_slow_dreamworld"]["dreamworld_replay_batch_size"] == 128
    ev = by["fast_slow_dreamworld_event_sleep"]
    assert ev["event_sleep_enabled"] and ev["dreamworld_cache_interval"] == 8
    assert "name_arm" not in ev
    assert exp24.build_first_wave_matrix(speed_config=SPEED, seeds=(1,)) == entries


def test_phase0_names():
    sweep = exp24.build_phase0_dreamworld_sweep(speed_config=SPEED)
    assert sweep[0]["name"] == "exp24_phase0_fs_i32a050_dw_c4i4_w010_s1337"
    assert sweep[-1]["name"] == "exp24_phase0_fs_i32a050_dw_c16i16_w050_s1337"
    fs = exp24.build_phase0_fastslow_sweep(speed_config=SPEED)
    assert fs[0]["name"] == "exp24_phase0_fs_i16a025_dw_c16i16_w010_s1337"
    assert {e["world_size"] for e in fs} == {4}
    conf = exp24.build_phase0_confirm(speed_config=SPEED)
    assert conf[3]["name"] == "exp24_phase0_confirm_B_fs_i64a025_dw_c16i16_w010_s1337"
    ctl = exp24.build_phase0_fastslow_only_control(speed_config=SPEED)
    assert not ctl[0]["dreamworld_enabled"] and ctl[0]["fast_slow_interval"] == 64


def test_scopt_gate():
    muon, scopt = exp24.build_scopt_overhead_gate_matrix(speed_config=SPEED)
    assert muon["optimizer"] == "muon" and "scopt_warmup_steps" not in muon
    assert scopt["scopt_pressure_upper_c"] == 3.0 and scopt["batch_size"] == 512
    assert scopt["optimizer_param_grouping"] == "ssm_three_group"
    cal = exp24.build_scopt_calibration_sweep_matrix(speed_config=SPEED)
    assert [e["scopt_baseline_decay"] for e in cal] == [0.95, 0.99, 0.99]
    assert cal[2]["scopt_rare_ema_decay"] == 0.95 and cal[0]["budget_seconds"] == 1200.0


def test_arm_selection_and_unknown_arm():
    only = exp24.build_crct_v1_matrix(speed_config=SPEED, arms=["arm_d_crct_replay_active"])
    assert len(only) == 3 and only[0]["replay_eviction_mode"] == "active"
    assert only[1]["replay_eviction_trace_path"].endswith(
        "crct_replay_eviction_arm_d_crct_replay_active_s2674.ndjson")
    for fn in (exp24.build_crct_v1_matrix, exp24.build_episodic_ttt_v1_matrix,
               exp24.build_episodic_dw_curation_v1_matrix):
        with pytest.raises(ValueError, match="unknown arm"):
            fn(speed_config=SPEED, arms=["arm_z"])


def test_crct_matrix_locks():
    entries = exp24.build_crct_v1_matrix(speed_config={**SPEED, "train_sampling_mode":
                                                       "sequential_epoch"}, seed_values=(5,))
    a, b, c, d = entries
    assert [e["arm"] for e in entries] == list(exp24.CRCT_V1_ARMS)
    assert all(e["train_sampling_mode"] == "random" for e in entries)
    assert "crct_enabled" not in a and b["crct_enabled"] and not b.get("replay_eviction_enabled")
    assert b["crct_async_teacher_transport_backend"] == "mailbox" and b["cuda_graph_mode"] == "none"
    assert c["replay_eviction_mode"] == "shadow" and d["replay_eviction_mode"] == "active"
    assert d["name"] == "exp24_phase3_crct_v1_arm_d_crct_replay_active_s5"


def test_controller_matrix_env_and_traces(monkeypatch):
    monkeypatch.setenv(exp24.EPISODIC_CONTROLLER_V1_WEIGHTS_PATH_ENV, "/w/x.pt")
    monkeypatch.setenv(exp24.EPISODIC_CONTROLLER_V1_TRACE_DIR_ENV, "/t")
    entries = exp24.build_episodic_controller_v1_matrix(
        speed_config={**SPEED, "train_sampling_mode": "shuffled_epoch"}, seed_values=(9,))
    by = {e["arm"]: e for e in entries}
    assert list(by) == list(exp24.EPISODIC_CONTROLLER_V1_ARMS)
    assert by["arm_a_control"]["train_sampling_mode"] == "shuffled_epoch"
    assert by["arm_b_heuristic"]["train_sampling_mode"] == "random"
    assert "episodic_controller_simplex_trace_path" not in by["arm_b_heuristic"]
    c = by["arm_c_simplex_frozen"]
    assert c["episodic_controller_weights_path"] == "/w/x.pt"
    assert c["episodic_controller_simplex_trace_path"] == (
        "/t/episodic_controller_v1_arm_c_simplex_frozen_s9.ndjson")
    assert not c["controller_train_online"] and by["arm_d_simplex_online"]["controller_train_online"]
    assert by["arm_e_simplex_warm_online"]["eval_episodic_cache_mode"] == "warm"
    assert by["arm_f_simplex_sharp_online"]["episodic_controller_initial_temperature"] == 0.2
    assert by["arm_a_control"]["eval_episodic_cache_mode"] == "none"


def test_ttt_and_curation_matrices():
    ttt = {e["name"].split("v1_")[1].rsplit("_s", 1)[0]: e
           for e in exp24.build_episodic_ttt_v1_matrix(speed_config=SPEED, seed_values=(1,))}
    assert ttt["arm_b_cache_train_ttt_with_cache"]["eval_adapt_set"] == "lm_head"
    assert ttt["arm_b_cache_train_ttt_with_cache"]["episodic_enabled"]
    assert ttt["arm_a_no_cache_no_ttt"]["eval_steps_per_chunk"] == 0
    assert not ttt["arm_d_no_cache_train_ttt_only"]["dreamworld_enabled"]
    cur = exp24.build_episodic_dw_curation_v1_matrix(
        speed_config=SPEED, seed_values=exp24.EPISODIC_DW_CURATION_V1_ESCALATION_SEEDS,
        arms=exp24.EPISODIC_DW_CURATION_V1_ESCALATION_ARMS)
    assert len(cur) == 9 and cur[0]["dreamworld_cache_interval"] == 16
    assert cur[3]["controller_query_mode"] == "cosine_utility_weighted"
    assert cur[6]["controller_query_mode"] == "pressure_only"


def test_criticality_cells():
    first = exp24.build_criticality_distillation_first_smoke_matrix(speed_config=SPEED,
                                                                    seed_values=(1,))
    arms = [e["name"].split("cd_first_smoke_")[1][:-3] for e in first]
    assert arms == ["treatment", "telemetry", "shuffled", "budget_only",
                    "hl_short", "hl_long", "H_short", "H_long"]
    assert first[1]["criticality_distill_weight"] == 0.0
    assert first[0]["criticality_distill_weight"] == 1e-3 and first[0]["rare_bucket_ce_enabled"]
    assert first[7]["criticality_distill_horizon_H"] == 32
    multi = exp24.build_criticality_distillation_multiseed_matrix(speed_config=SPEED)
    assert multi[-1]["name"] == "exp24_cd_multiseed_H_short_s2024"


def test_control_noise_summary():
    rows = [{"config": {"seed": s}, "eval": {"bpb": b},
             "train": {"elapsed_s": 600.0, "aggregate_tokens_per_sec": t}}
            for s, b, t in ((1, 1.50, 1e6), (2, 1.52, 2e6), (3, 1.54, 3e6))]
    out = exp24.summarize_control_noise(rows)
    assert out["count"] == 3 and out["seeds"] == [1, 2, 3]
    assert out["bpb_mean"] == pytest.approx(1.52) and out["bpb_sample_std"] == pytest.approx(0.02)
    assert out["tokens_per_sec_mean"] == pytest.approx(2e6)
    assert exp24.summarize_control_noise(rows[:1])["bpb_sample_std"] == 0.0


def test_cli_writes_matrix(tmp_path, capsys):
    cfg = tmp_path / "speed.yaml"
    cfg.write_text("batch_size: 1024\nseq_len: 512\n")
    out = tmp_path / "m.json"
    assert exp24.main(["ring0_control_matrix", "--speed-config", str(cfg),
                       "--world-size", "2", "--out", str(out)]) == 0
    entries = json.loads(out.read_text())
    assert len(entries) == 3 and entries[0]["world_size"] == 2
    assert "exp24_ring0_control_s1337" in capsys.readouterr().out
