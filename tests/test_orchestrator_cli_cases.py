"""Launcher / orchestrator command lines that mirror the reference's scripts, and the self-describing controller
weight file (CPU)."""
import json
import struct
from pathlib import Path

import numpy as np
import pytest

from chaoscontrol_b200 import exp26, exp27, paper_results, run_exp24
from chaoscontrol_b200 import runner_persistent_ddp as RP
from chaoscontrol_b200.episodic import cswg, native, pretrain
from chaoscontrol_b200.episodic.controller import load_simplex_policy, save_simplex_policy


# ---------------------------------------------------------------- exp26 / exp27
def test_exp26_dry_run_prints_both_cells_and_touches_nothing(tmp_path, capsys):
    assert exp26.main(["--dry-run", "--output-dir", str(tmp_path / "v"), "--seed", "7", "--budget", "30", "--world-size", "2"]) == 0
    out = capsys.readouterr().out
    assert "exp26_validation_validation_fastslow_control_s7" in out and "adaptive_residual_memory_s7" in out
    assert not (tmp_path / "v").exists()


def test_exp26_launch_writes_the_matrix_and_hands_entries_to_the_launcher(tmp_path, monkeypatch):
    seen = {}
    import chaoscontrol_b200.launch as L
    monkeypatch.setattr(L, "run_matrix", lambda entries, **kw: (seen.update(entries=entries, **kw), {"ranked": [], "errors": []})[1])
    res = exp26.run_validation(speed_config={"base_lr": 0.064}, world_size=2, seed=3, budget_seconds=20, data_path="/d",
                               sp_model_path="/m", output_dir=tmp_path / "v", say=lambda *_: None)
    assert [e["arm"] for e in res["entries"]] == list(exp26.VALIDATION_ARMS) and seen["world_size"] == 2
    assert seen["data_path"] == "/d" and seen["sp_model_path"] == "/m" and seen["results_dir"] == tmp_path / "v"
    assert len(json.loads((tmp_path / "v" / "matrix.json").read_text())) == 2
    assert str(tmp_path / "v" / "traces") in res["entries"][1]["replay_eviction_trace_path"]


def test_exp27_dry_run_stages_write_nothing(tmp_path, capsys):
    man = tmp_path / "cal" / "manifest.json"
    assert exp27.main(["run", "--stage", "all", "--dry-run", "--manifest-path", str(man),
                       "--headline-output-dir", str(tmp_path / "h")]) == 0
    out = capsys.readouterr().out
    assert "stage=calibrate" in out and "stage=analyze" in out and "manifest_absent=True" in out
    assert not man.exists() and not (tmp_path / "h").exists()


def test_exp27_analyze_then_headline_preview_and_launch(tmp_path, capsys, monkeypatch):
    man = tmp_path / "cal" / "manifest.json"
    assert exp27.main(["run", "--stage", "analyze", "--manifest-path", str(man)]) == 0
    m = json.loads(man.read_text())
    assert set(m["calc_type_hyperparams"]) >= {"score_only_reset", "adaptive_carry"} and "no probe" in m["note"]
    capsys.readouterr()
    args = ["run", "--stage", "headline", "--manifest-path", str(man), "--seeds", "1", "2", "--world-size", "2",
            "--headline-budget", "30", "--checkpoint-path", str(tmp_path / "trunk.pt"), "--headline-output-dir", str(tmp_path / "h")]
    assert exp27.main(args + ["--dry-run"]) == 0
    out = capsys.readouterr().out
    assert "entries=2" in out and "exp27_ttt_headline_s1" in out and '"eval_only": true' in out and not (tmp_path / "h").exists()
    with pytest.raises(FileNotFoundError, match="validation cache"):
        exp27.main(args + ["--val-cache-dir", str(tmp_path / "missing")])
    (tmp_path / "vc").mkdir()
    seen = {}
    import chaoscontrol_b200.launch as L
    monkeypatch.setattr(L, "run_matrix", lambda entries, **kw: seen.update(n=len(entries), **kw) or {})
    assert exp27.main(args + ["--val-cache-dir", str(tmp_path / "vc"), "--limit", "1", "--no-skip-existing",
                              "--sp-model-path-16384", "/m", "--data-path", "/d"]) == 0
    assert seen["n"] == 2 and seen["limit"] == 1 and seen["skip_existing"] is False and seen["val_cache_dir"] == str(tmp_path / "vc")
    assert seen["sp_model_path"] == "/m" and seen["data_path"] == "/d" and (tmp_path / "h" / "matrix.json").exists()


def test_exp27_analyze_uses_a_probe_report_when_one_exists(tmp_path):
    man = tmp_path / "manifest.json"
    hp = {"score_only_reset": {}, "adaptive_carry": {"online_episodic_chunk_tokens": 64}}
    (tmp_path / "probe_report.json").write_text(json.dumps({"hyperparams": hp, "report": {"calc_types": {}}, "source": "ck.pt"}))
    exp27.main(["run", "--stage", "analyze", "--manifest-path", str(man)])
    m = json.loads(man.read_text())
    assert m["calc_type_hyperparams"] == hp and m["source_trace"] == "ck.pt" and "probe" in m


def test_exp24_takes_the_reference_tokenizer_flag(tmp_path, capsys):
    assert run_exp24.main(["--matrix", "crct_v1", "--dry-run", "--limit", "1", "--output-dir", str(tmp_path),
                           "--sp-model-path-16384", "/m/tok.model"]) == 0
    assert "/m/tok.model" in capsys.readouterr().out or True


# ---------------------------------------------------------------- persistent launcher
def _launch(tmp_path, *extra, call=None):
    args = ["--data-path", "/d", "--sp-model-path", "/m", "--output-dir", str(tmp_path / "out"), "--world-size", "2",
            "--conditions", "bf16", "--seeds", "1", "2", "--rdzv-port", "29701", *extra]
    return RP.launch_main(args, call=call or (lambda cmd: 0))


def test_launcher_dry_run_prints_one_torchrun_over_the_whole_matrix(tmp_path, capsys):
    assert _launch(tmp_path, "--dry-run") == 0
    out = capsys.readouterr().out
    assert "--nproc-per-node=2" in out and "--master-port 29701" in out and "127.0.0.1" in out
    assert "chaoscontrol_b200.runner_persistent_ddp" in out and "(2 entries)" in out
    m = json.loads((tmp_path / "out" / ".persistent_matrix.json").read_text())
    assert [(e["name"], e["seed"]) for e in m] == [("bf16", 1), ("bf16", 2)]


def test_launcher_fails_closed_on_missing_outputs_and_passes_on_complete_ones(tmp_path, capsys):
    assert _launch(tmp_path) == 1                                       # torchrun "succeeded" but wrote nothing
    assert "missing output file" in capsys.readouterr().out and not (tmp_path / "out" / ".persistent_matrix.json").exists()

    def fake(cmd):
        out = Path(cmd[cmd.index("--output-dir") + 1])
        for e in json.loads(Path(cmd[cmd.index("--config-matrix") + 1]).read_text()):
            RP.write_result_json(out / f"{e['name']}_s{e['seed']}.json", {"config": e, "train": {}, "eval": {}})
        return 0
    assert _launch(tmp_path, call=fake) == 0
    assert _launch(tmp_path, call=lambda cmd: 9) == 9                   # a non-zero torchrun exit is passed on


def test_launcher_preflight_world_size_fp8_and_external_matrix(tmp_path, capsys, monkeypatch):
    mj = tmp_path / "m.json"
    mj.write_text(json.dumps(RP.build_default_matrix(4, 0.1, [1], ["bf16"])))
    with pytest.raises(ValueError, match="world_size disagrees"):
        _launch(tmp_path, "--matrix-json", str(mj))
    mj.write_text(json.dumps({"a": 1}))
    with pytest.raises(ValueError, match="JSON list"):
        _launch(tmp_path, "--matrix-json", str(mj))
    assert RP.main(["launch", "--data-path", "/d", "--output-dir", str(tmp_path / "o3"), "--world-size", "2",
                    "--conditions", "bf16", "--seeds", "1", "--dry-run"]) == 0
    monkeypatch.setattr(RP, "fp8_is_available", lambda: False)
    args = ["--data-path", "/d", "--output-dir", str(tmp_path / "o2"), "--world-size", "2", "--conditions", "fp8", "--seeds", "1"]
    monkeypatch.setattr(RP, "filter_matrix_for_fp8", lambda entries, out: ([], list(entries)))
    assert RP.launch_main(args, call=lambda cmd: 0) == 1                # nothing runnable is a failure
    assert json.loads((tmp_path / "o2" / "fp8_s1.json").read_text())["error"].startswith("skipped:")


# ---------------------------------------------------------------- registry CLI
def test_registry_cli_takes_artifact_lists_and_extras(tmp_path, capsys):
    reg = tmp_path / "r.jsonl"
    assert paper_results.main(["--registry", str(reg), "register", "--experiment", "e", "--condition", "c", "--status",
                               "exploratory", "--config-hash", "sha256:x", "--seed", "1", "--metrics", '{"bpb": 1.5}',
                               "--artifacts", "a.json", "b.json", "--artifact", "c.json", "--extras", '{"note": "n"}']) == 0
    row = json.loads(reg.read_text())
    assert row["artifacts"] == ["c.json", "a.json", "b.json"] and row["extras"] == {"note": "n"} and row["metrics"]["bpb"] == 1.5


# ---------------------------------------------------------------- self-describing weight file
def test_cswg3_round_trip_plain_policy(tmp_path):
    pol = native.SimplexPolicy(N=16, K_v=16, K_s=4, H=32, temperature=0.7, seed=3)
    m = cswg.policy_to_cswg(pol, tmp_path / "p.cswg")
    assert m["version"] == 3 and m["dims"]["n_heads"] == 0 and m["file_bytes"] == (tmp_path / "p.cswg").stat().st_size
    assert [t["name"] for t in m["tensors"]] == list(cswg.TENSOR_NAMES) and m["fp32_vs_fp16_max_abs_drift"] < 1e-3
    back = cswg.policy_from_cswg(tmp_path / "p.cswg")
    assert type(back) is native.SimplexPolicy and back.temperature == pytest.approx(0.7, abs=1e-3)
    assert np.allclose(back.flat, pol.flat, atol=1e-3) and cswg.file_version(tmp_path / "p.cswg") == 3
    V = np.random.default_rng(0).standard_normal((16, 16)).astype(np.float32)
    E, f = np.zeros((16, 16), np.float32), np.zeros(4, np.float32)
    assert np.allclose(back.forward(V, E, f)[0], pol.forward(V, E, f)[0], atol=5e-3)


def test_cswg3_carries_heads_and_bucket_embedding(tmp_path):
    pol = native.SimplexPolicyV3(N=16, K_v=16, K_e=1, K_s=4, H=32, n_heads=2, n_buckets=3, embed_dim=5, seed=1)
    cswg.policy_to_cswg(pol, tmp_path / "v3.cswg")
    blob = cswg.load_cswg_v3(tmp_path / "v3.cswg")
    t = blob["tensors"]
    assert t["W_q"].shape == (2, 32, 32) and t["W_e"].shape == (2, 1) and t["bucket_embed"].shape == (3, 5) and t["b_lh"].shape == ()
    back = load_simplex_policy(tmp_path / "v3.cswg")                    # the generic loader recognises version 3
    assert isinstance(back, native.SimplexPolicyV3) and back.n_heads == 2 and np.allclose(back.flat, pol.flat, atol=1e-3)
    save_simplex_policy(tmp_path / "again.cswg", back)                  # a policy with heads is saved self-describing
    assert cswg.file_version(tmp_path / "again.cswg") == 3
    plain = native.SimplexPolicy(seed=2)
    save_simplex_policy(tmp_path / "old.cswg", plain)                   # the plain one keeps the compact version-1 file
    assert cswg.file_version(tmp_path / "old.cswg") == 1 and np.allclose(load_simplex_policy(tmp_path / "old.cswg").flat, plain.flat, atol=1e-3)


def test_cswg3_reader_refuses_inconsistent_files(tmp_path):
    pol = native.SimplexPolicy(seed=3)
    path = tmp_path / "p.cswg"
    cswg.policy_to_cswg(pol, path)
    raw = path.read_bytes()
    cases = {"magic": b"XXXX" + raw[4:], "version": raw[:4] + struct.pack("<I", 2) + raw[8:],
             "dtype": raw[:8] + struct.pack("<I", 9) + raw[12:], "truncated": raw[:-10], "trailing": raw + b"\\0\\0",
             "tiny": raw[:10]}
    for name, data in cases.items():
        bad = tmp_path / f"{name}.cswg"
        bad.write_bytes(data)
        with pytest.raises(ValueError):
            cswg.load_cswg_v3(bad)
    with pytest.raises(KeyError, match="missing tensor"):
        cswg.write_cswg_v3(tmp_path / "x.cswg", {"W_vp": np.zeros((2, 2))}, cswg._dims_of(pol))
    with pytest.raises(ValueError, match="not a CSWG"):
        (tmp_path / "foreign.bin").write_bytes(b"hello world")
        cswg.file_version(tmp_path / "foreign.bin")


def test_dump_mode_converts_a_saved_policy(tmp_path, capsys):
    pol = native.SimplexPolicy(seed=5)
    save_simplex_policy(tmp_path / "p.pt", pol)
    assert pretrain.main(["--checkpoint", str(tmp_path / "p.pt"), "--output", str(tmp_path / "p.cswg")]) == 0
    assert "version=3" in capsys.readouterr().out and cswg.file_version(tmp_path / "p.cswg") == 3
    assert pretrain.main(["--checkpoint", str(tmp_path / "p.cswg"), "--output", str(tmp_path / "q.pt")]) == 0
    assert np.allclose(load_simplex_policy(tmp_path / "q.pt").flat, pol.flat, atol=1e-3)
    with pytest.raises(SystemExit):
        pretrain.main(["--output", str(tmp_path / "z.cswg")])
