"""CPU controller latency bench: structure of the report, honesty about missing CPU paths (CPU)."""
import json

from chaoscontrol_b200.episodic import controller_bench as CB
from chaoscontrol_b200.episodic import native as N


def test_report_structure_and_unavailable_paths(tmp_path):
    out = tmp_path / "b.json"
    assert CB.main(["--iterations", "60", "--warmup", "10", "--output", str(out)]) == 0
    r = json.loads(out.read_text())
    feats = N.cpu_features()
    assert r["cpu_features"] == feats and r["simplex_dims"] == CB.SIMPLEX
    k = r["isolated_kernel"]
    for name in ("generic_fp32_recurrence", "generic_bf16_matmul_16x32x16", "generic_bf16_matmul_64x64x32_tiled"):
        assert k[name]["median_us"] > 0 and k[name]["p99_us"] >= k[name]["median_us"]
    if not feats["avx512f"]:
        assert k["avx512_recurrence"] == {"available": False, "reason": "this CPU has no AVX-512F"}
    else:
        assert k["avx512_recurrence"]["median_us"] > 0
    for label in ("16x32x16", "64x64x32_tiled"):
        amx = k[f"amx_bf16_matmul_{label}"]
        if feats["amx_bf16"] and feats["amx_enabled"]:
            assert amx["median_us"] > 0
        else:
            assert amx["available"] is False and "AMX" in amx["reason"]
    q = r["simplex_per_query"]
    assert q["forward_only"]["median_us"] > 0
    assert q["decision_record"]["median_us"] >= 0.5 * q["forward_only"]["median_us"]
    assert q["full_replay_event"]["median_us"] > q["decision_record"]["median_us"]
    # every timed event was credited and, at sgd_interval 1, applied
    assert q["full_replay_event"]["sgd_steps"] == q["full_replay_event"]["credited_actions"] > 0
    assert q["event_budget_us"] == 150.0 and isinstance(q["within_event_budget"], bool)


def test_time_us_orders_samples():
    calls = []
    s = CB.time_us(lambda: calls.append(1), iterations=50, warmup=5)
    assert len(calls) == 55 and 0 <= s["median_us"] <= s["p99_us"] and s["mean_us"] >= 0
