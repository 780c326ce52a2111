"""Warm multi-run worker and launcher checks, one property per test (CPU)."""
import json
from pathlib import Path

import pytest
import torch
import torch.nn as nn

from chaoscontrol_b200 import runner_persistent_ddp as RP


def _entries(n=2, precision="bf16", ws=2):
    return [RP.base_config(world_size=ws, base_lr=0.064, precision=precision, seed=s, name=precision) for s in range(n)]


def _ok(out: Path, e, **extra):
    RP.write_result_json(out / f"{e['name']}_s{e['seed']}.json", {"config": e, "train": {}, "eval": {"bpb": 1.5}, **extra})


# ---------------------------------------------------------------- output integrity
def test_all_successful_results(tmp_path):
    es = _entries(3)
    for e in es:
        _ok(tmp_path, e)
    assert RP.check_output_integrity(tmp_path, es) == (3, 0, [])


def test_real_error_is_surfaced(tmp_path):
    es = _entries(1)
    RP.write_result_json(tmp_path / "bf16_s0.json", {"config": es[0], "error": "CUDA out of memory"})
    ok, benign, bad = RP.check_output_integrity(tmp_path, es)
    assert (ok, benign) == (0, 0) and bad == ["bf16_s0: error=CUDA out of memory"]


def test_benign_skip_is_counted_separately(tmp_path):
    es = _entries(1, precision="fp8")
    RP.write_skip_markers(es, tmp_path)
    assert RP.check_output_integrity(tmp_path, es) == (0, 1, [])
    assert json.loads((tmp_path / "fp8_s0.json").read_text())["error"].startswith("skipped:")


def test_missing_and_malformed_outputs_are_errors(tmp_path):
    es = _entries(2)
    (tmp_path / "bf16_s1.json").write_text("{not json")
    ok, benign, bad = RP.check_output_integrity(tmp_path, es)
    assert ok == benign == 0 and bad[0] == "bf16_s0: missing output file" and bad[1].startswith("bf16_s1: malformed JSON")


def test_file_without_result_keys_is_an_error(tmp_path):
    es = _entries(1)
    RP.write_result_json(tmp_path / "bf16_s0.json", {"config": es[0], "train": {}})
    assert "neither" in RP.check_output_integrity(tmp_path, es)[2][0]


def test_mixed_matrix_counts_each_kind(tmp_path):
    es = _entries(2) + _entries(2, precision="fp8")
    _ok(tmp_path, es[0])
    RP.write_result_json(tmp_path / "bf16_s1.json", {"config": es[1], "error": "boom"})
    RP.write_skip_markers(es[2:3], tmp_path)
    ok, benign, bad = RP.check_output_integrity(tmp_path, es)
    assert (ok, benign, len(bad)) == (1, 1, 2)


# ---------------------------------------------------------------- world size
def test_world_size_match_passes_and_mismatch_or_missing_field_raises():
    RP.validate_matrix_world_size(_entries(3, ws=4), 4)
    with pytest.raises(ValueError, match="world_size disagrees"):
        RP.validate_matrix_world_size(_entries(3, ws=4), 2)
    es = _entries(1, ws=2)
    del es[0]["world_size"]
    with pytest.raises(ValueError):
        RP.validate_matrix_world_size(es, 2)


def test_world_size_error_previews_at_most_five():
    with pytest.raises(ValueError, match=r"\+2 more"):
        RP.validate_matrix_world_size(_entries(7, ws=8), 2)


# ---------------------------------------------------------------- fp8 gating
def test_fp8_dropped_when_unavailable_kept_when_available_and_bf16_needs_no_probe(tmp_path):
    es = _entries(1) + _entries(2, precision="fp8")
    run, skip = RP.filter_matrix_for_fp8(es, tmp_path, probe=lambda: False)
    assert [e["precision"] for e in run] == ["bf16"] and len(skip) == 2
    run, skip = RP.filter_matrix_for_fp8(es, tmp_path, probe=lambda: True)
    assert len(run) == 3 and skip == []

    def never():
        raise AssertionError("probe must not run for a matrix without fp8")
    assert RP.filter_matrix_for_fp8(_entries(2), tmp_path, probe=never) == (_entries(2), [])


def test_stale_skip_markers_block_the_run_only_when_fp8_can_run(tmp_path):
    es = _entries(2, precision="fp8")
    RP.write_result_json(tmp_path / "fp8_s0.json", {"config": es[0], "error": "skipped: fp8 unavailable on this host"})
    RP.reject_stale_skip_markers(es, tmp_path, probe=lambda: False)
    with pytest.raises(RuntimeError, match="stale skip markers") as ei:
        RP.reject_stale_skip_markers(es, tmp_path, probe=lambda: True)
    assert str(tmp_path / "fp8_s0.json") in str(ei.value)
    RP.reject_stale_skip_markers(_entries(2), tmp_path, probe=lambda: True)               # no fp8 in the matrix


def test_real_errors_and_real_successes_are_not_stale_markers(tmp_path):
    es = _entries(2, precision="fp8")
    RP.write_result_json(tmp_path / "fp8_s0.json", {"config": es[0], "error": "CUDA out of memory"})
    _ok(tmp_path, es[1])
    RP.reject_stale_skip_markers(es, tmp_path, probe=lambda: True)


def test_stale_marker_preview_is_capped_at_five(tmp_path):
    es = _entries(8, precision="fp8")
    RP.write_skip_markers(es, tmp_path)
    with pytest.raises(RuntimeError, match=r"\+3 more"):
        RP.reject_stale_skip_markers(es, tmp_path, probe=lambda: True)


# ---------------------------------------------------------------- idempotent skip
def test_config_match_exact_and_error_marker_with_matching_config(tmp_path):
    e = _entries(1)[0]
    p = tmp_path / "o.json"
    RP.write_result_json(p, {"config": e, "eval": {}, "train": {}})
    RP.require_config_match(p, dict(e))
    RP.write_result_json(p, {"config": e, "error": "boom"})
    RP.require_config_match(p, dict(e))


def test_config_change_added_field_and_malformed_file_raise_with_both_hashes(tmp_path):
    e = _entries(1)[0]
    p = tmp_path / "o.json"
    RP.write_result_json(p, {"config": e, "eval": {}, "train": {}})
    changed = dict(e, base_lr=0.128)
    with pytest.raises(RuntimeError, match="config mismatch") as ei:
        RP.require_config_match(p, changed)
    assert RP.config_hash(e) in str(ei.value) and RP.config_hash(changed) in str(ei.value)
    with pytest.raises(RuntimeError):
        RP.require_config_match(p, dict(e, extra=1))
    p.write_text("{oops")
    with pytest.raises(RuntimeError, match="could not read"):
        RP.require_config_match(p, e)
    RP.write_result_json(p, {"eval": {}})
    with pytest.raises(RuntimeError, match="config mismatch"):
        RP.require_config_match(p, e)


def test_config_hash_is_order_free_and_short():
    assert RP.config_hash({"a": 1, "b": 2}) == RP.config_hash({"b": 2, "a": 1}) != RP.config_hash({"a": 1, "b": 3})
    assert len(RP.config_hash({})) == 8


# ---------------------------------------------------------------- worker helpers
def test_warmup_restores_weights_clears_grads_and_builds_after_the_warmup():
    torch.manual_seed(0)
    model = nn.Linear(4, 4)
    before = {k: v.clone() for k, v in model.state_dict().items()}
    order = []

    def warm():
        order.append("warmup")
        opt = torch.optim.SGD(model.parameters(), lr=1.0)
        model(torch.randn(2, 4)).sum().backward()
        opt.step()

    def build():
        order.append("build")
        return torch.optim.SGD(model.parameters(), lr=0.1)
    opt = RP.warmup_and_restore(model=model, warmup_call_fn=warm, build_optimizer_fn=build, device=torch.device("cpu"),
                                ddp_active=False)
    assert order == ["warmup", "build"] and isinstance(opt, torch.optim.SGD) and len(opt.state) == 0
    assert all(torch.equal(v, before[k]) for k, v in model.state_dict().items())
    assert all(p.grad is None for p in model.parameters())


def test_apply_seed_resets_every_generator():
    import random

    import numpy as np
    RP.apply_seed(11)
    a = (random.random(), float(np.random.rand()), float(torch.rand(())))
    random.random(), np.random.rand(), torch.rand(())
    RP.apply_seed(11)
    assert (random.random(), float(np.random.rand()), float(torch.rand(()))) == a


def test_result_file_is_written_through_a_rename(tmp_path):
    p = tmp_path / "deep" / "r.json"
    RP.write_result_json(p, {"x": Path("/a")})                        # non-JSON values are stringified
    assert json.loads(p.read_text()) == {"x": "/a"} and not p.with_suffix(".tmp").exists()


def test_error_flag_without_ddp_is_local():
    assert RP.sync_error_flag(True, torch.device("cpu"), False) is True
    assert RP.sync_error_flag(False, torch.device("cpu"), False) is False


def test_default_matrix_is_conditions_by_seeds_in_the_submission_regime():
    es = RP.build_default_matrix(4, 0.064, [1, 2], ["bf16", "fp8"])
    assert [(e["name"], e["seed"]) for e in es] == [("bf16", 1), ("bf16", 2), ("fp8", 1), ("fp8", 2)]
    e = es[0]
    assert (e["model_dim"], e["num_layers"], e["vocab_size"], e["seq_len"], e["batch_size"]) == (256, 4, 16384, 512, 1024)
    assert e["world_size"] == 4 and e["optimizer"] == "muon" and all(f in e for f in RP.REQUIRED_ENTRY_FIELDS)
    assert RP.base_config(world_size=1, base_lr=0.1, precision="bf16", seed=0, name="x", model_dim=384)["model_dim"] == 384


def test_cli_dry_run_and_matrix_must_be_a_list(tmp_path, capsys):
    m = tmp_path / "m.json"
    m.write_text(json.dumps(_entries(2)))
    assert RP.main(["--data-path", "/d", "--config-matrix", str(m), "--output-dir", str(tmp_path / "o"), "--dry-run"]) == 0
    assert "entries=2" in capsys.readouterr().out
    m.write_text(json.dumps({"not": "a list"}))
    with pytest.raises(ValueError, match="list of entry dicts"):
        RP.main(["--data-path", "/d", "--config-matrix", str(m), "--output-dir", str(tmp_path / "o"), "--dry-run"])
