"""Command-line tools that do not need a GPU: artifact headroom."""


def test_artifact_headroom_estimate_and_exit_code(tmp_path):
    from chaoscontrol_b200 import cli
    h = cli.artifact_headroom(dim=384)
    assert h["under_budget"] and h["raw_bf16_bytes"] > h["baseline_dim256_raw_bf16_bytes"]
    ratio = h["raw_bf16_bytes"] / h["baseline_dim256_raw_bf16_bytes"]
    assert h["estimated_compressed_model_bytes"] == round(cli.MEASURED_DIM256_COMPRESSED_BYTES * ratio)
    assert h["margin_bytes"] == 16_000_000 - h["estimated_total_bytes"]
    assert cli.artifact_headroom(dim=256)["estimated_compressed_model_bytes"] == cli.MEASURED_DIM256_COMPRESSED_BYTES
    out = tmp_path / "h.json"
    assert cli.main(["artifact-headroom", "--dim", "640", "--output", str(out)]) == 2
    import json
    assert json.loads(out.read_text())["under_budget"] is False
    small = cli.artifact_headroom(dim=64, vocab_size=512, num_layers=1, measure=True)
    assert 0 < small["measured_random_init_int6_bytes"] < small["raw_bf16_bytes"]
