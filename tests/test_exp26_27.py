"""Adaptive-residual-memory validation matrix, calibration manifest + probe, headline matrix."""
import json

import pytest
import torch

from chaoscontrol_b200 import exp26, exp27
from chaoscontrol_b200.eval_stream import load_val_cache, write_synthetic_val_cache
from chaoscontrol_b200.models.model import CareStudentLM

SPEED = {"batch_size": 64, "seq_len": 128, "fast_slow_interval": 64}


def test_validation_matrix_locks(tmp_path):
    ctl, full = exp26.build_validation_matrix(speed_config=SPEED, seed=9, trace_dir=tmp_path)
    assert [ctl["arm"], full["arm"]] == list(exp26.VALIDATION_ARMS)
    assert ctl["name"] == "exp26_validation_validation_fastslow_control_s9" and ctl["budget_seconds"] == 45.0
    for e in (ctl, full):
        assert e["model_dim"] == 384 and e["ssm_delta_rank"] == 32 and e["lm_head_tile_size"] == 4096
        assert "fast_slow_interval" not in e and e["episodic_controller_action_space_enabled"]
        assert e["exp26_mechanism"] == "arm_v1" and e["train_sampling_mode"] == "random"
    assert "crct_enabled" not in ctl and "replay_eviction_arm_runtime_namespace" not in ctl
    assert full["crct_enabled"] and full["crct_teacher_score_interval_steps"] == 1
    assert full["crct_memory_write_tokens_per_step"] == 32 and "crct_async_teacher_pending_batches" not in full
    assert full["replay_eviction_mode"] == "active" and full["replay_eviction_commit_policy"] == "learned"
    assert full["replay_eviction_arm_runtime_namespace"] == full["name"]
    assert full["replay_eviction_trace_path"] == str(
        tmp_path / "arm_validation_adaptive_residual_memory_s9.ndjson")
    assert full["replay_eviction_evidence_engine_d_model"] == 384
    json.dumps([ctl, full])


def test_manifest_round_trip_and_validation(tmp_path):
    man = exp27.write_manifest(tmp_path / "cal" / "m.json")
    assert set(man["calc_type_hyperparams"]) == {"score_only_reset", "adaptive_carry", "carry_state",
                                                 "dreamworld_eval"}
    assert exp27.load_manifest(tmp_path / "cal" / "m.json")["calc_type_hyperparams"]["dreamworld_eval"]["K"] == 8
    with pytest.raises(FileNotFoundError):
        exp27.load_manifest(tmp_path / "none.json")
    (tmp_path / "bad.json").write_text("{")
    with pytest.raises(ValueError, match="malformed"):
        exp27.load_manifest(tmp_path / "bad.json")
    (tmp_path / "thin.json").write_text(json.dumps({"calibrated_at": "now"}))
    with pytest.raises(ValueError, match="calc_type_hyperparams"):
        exp27.load_manifest(tmp_path / "thin.json")


def test_headline_matrix(tmp_path):
    exp27.write_manifest(tmp_path / "m.json")
    train = exp27.build_ttt_headline_matrix(speed_config=SPEED, calibration_manifest_path=tmp_path / "m.json")
    assert [e["name"] for e in train] == [f"exp27_ttt_headline_s{s}" for s in exp27.DEFAULT_HEADLINE_SEEDS]
    e = train[0]
    assert e["arm"] == exp27.EXP26_ARM_NAME and e["crct_enabled"] and e["checkpoint_path"] is None
    assert "eval_only" not in e and e["headline_calc_type"] == "adaptive_carry"
    assert e["calc_type_configs"]["adaptive_carry"]["horizon_shifts"] == [-0.5, 0.0, 0.5]
    ev = exp27.build_ttt_headline_matrix(speed_config=SPEED, calibration_manifest_path=tmp_path / "m.json",
                                         checkpoint_path=tmp_path / "ck.pt", seed_values=[5],
                                         calc_types=["carry_state", "score_only_reset"])
    assert ev[0]["eval_only"] and ev[0]["max_steps"] == 0 and ev[0]["headline_calc_type"] == "score_only_reset"
    assert list(ev[0]["calc_type_configs"]) == ["carry_state", "score_only_reset"]
    with pytest.raises(ValueError, match="unknown calc_type"):
        exp27.build_ttt_headline_matrix(speed_config=SPEED, calibration_manifest_path=tmp_path / "m.json",
                                        calc_types=["nope"])


def test_probe_shrinks_the_expensive_pass_to_fit(tmp_path):
    write_synthetic_val_cache(tmp_path / "vc", n_docs=12, vocab=64, median_len=24, sigma=0.4, min_len=8,
                              max_len=40, seed=2)
    vc = load_val_cache(tmp_path / "vc")
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    ticks = iter(range(10_000))

    def clock():                                    # every pass "takes" one second
        return float(next(ticks))

    hp0 = exp27.default_calc_type_hyperparams()
    hp0["dreamworld_eval"].update(K=4, L=4, prefix_len=4)
    # probe covers ~1/3 of the tokens: the estimate is ~3 s; a 2 s budget can never fit, so the
    # knob is halved down to its floor; a 100 s budget fits at once
    hp, rep = exp27.probe_calc_types(model=model, val_cache=vc, device=torch.device("cpu"),
                                     luts=(None, None, None), calc_types=["score_only_reset", "dreamworld_eval"],
                                     budget_seconds=2.0, probe_docs=4, hyperparams=hp0, time_fn=clock)
    dw = rep["calc_types"]["dreamworld_eval"]
    assert [r["value"] for r in dw["rounds"]] == [4, 2, 1] and hp["dreamworld_eval"]["K"] == 1
    assert not dw["fits_budget"] and len(rep["calc_types"]["score_only_reset"]["rounds"]) == 1
    assert hp0["dreamworld_eval"]["K"] == 4                                   # the input is not edited
    hp, rep = exp27.probe_calc_types(model=model, val_cache=vc, device=torch.device("cpu"),
                                     luts=(None, None, None), calc_types=["dreamworld_eval"],
                                     budget_seconds=100.0, probe_docs=4, hyperparams=hp0, time_fn=clock)
    assert rep["calc_types"]["dreamworld_eval"]["fits_budget"] and hp["dreamworld_eval"]["K"] == 4
    man = exp27.write_manifest(tmp_path / "m.json", exp27.build_manifest(hyperparams=hp, source="ck", probe=rep))
    assert man["probe"]["total_tokens"] == vc.total_tokens and "note" not in man


def test_cli(tmp_path, capsys):
    assert exp27.main(["calibrate", "--manifest", str(tmp_path / "m.json")]) == 0
    assert exp27.main(["matrix", "--manifest", str(tmp_path / "m.json"), "--seeds", "1", "2",
                       "--out", str(tmp_path / "o" / "matrix.json")]) == 0
    assert "exp27_ttt_headline_s2" in capsys.readouterr().out
    assert len(json.loads((tmp_path / "o" / "matrix.json").read_text())) == 2
