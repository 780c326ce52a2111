"""Simplex bootstrap microbench and learner-trace comparison."""
import json
import math

from chaoscontrol_b200.episodic import bootstrap_bench as B


def test_sharper_start_unblocks_policy_gradient_learning():
    flat = B.run_bootstrap(temperature=1.0, events=1500, seed=0)
    sharp = B.run_bootstrap(temperature=0.2, events=1500, seed=0)
    assert abs(flat["initial_max_p"] - 1 / 16) < 0.01 and abs(sharp["initial_max_p"] - 1 / 16) < 0.01
    assert flat["sgd_steps"] > 0 and sharp["sgd_steps"] > 0
    # near-uniform sampling at T=1 leaves the policy close to uniform; the sharper start finds the vertex
    assert flat["final"]["entropy"] > 0.95 * math.log(16)
    assert sharp["final"]["p_good"] > 0.5 and sharp["final"]["entropy"] < 0.5 * math.log(16)
    assert sharp["final"]["weight_drift_l2"] > flat["final"]["weight_drift_l2"]
    assert [c["event"] for c in sharp["curve"]] == [500, 1000, 1500]


def test_trace_summary_and_arm_comparison(tmp_path, capsys):
    def write(path, entropies, credits):
        rows = [{"row_type": "decision", "entropy": e, "p_chosen": 0.1, "sgd_steps": i}
                for i, e in enumerate(entropies)]
        rows += [{"row_type": "credit", "current_entropy": 2.0, "advantage_final": a, "gerber_weight": 1.0,
                  "sgd_steps": 5} for a in credits]
        rows += [{"row_type": "skip", "status_reason": "missing_decision"}]
        path.write_text("\n".join(json.dumps(r) for r in rows) + "\n{broken\n")
    write(tmp_path / "d1.ndjson", [2.77, 2.76], [0.01])
    write(tmp_path / "f1.ndjson", [2.5, 1.2, 0.9], [0.5, -0.8])
    write(tmp_path / "f2.ndjson", [2.4, 1.0], [0.3])
    s = B.summarize_trace(tmp_path / "f1.ndjson")
    assert s["rows"] == {"decision": 3, "credit": 2, "skip": 1, "malformed": 1}
    assert s["skip_reasons"] == {"missing_decision": 1} and s["sgd_steps"] == 5
    assert s["stats"]["decision.entropy"]["min"] == 0.9
    cmp = B.compare_traces({"arm_d": [tmp_path / "d1.ndjson"],
                            "arm_f": [tmp_path / "f1.ndjson", tmp_path / "f2.ndjson"]})
    assert cmp["arm_f"]["seeds"] == 2 and cmp["arm_f"]["credits"] == 3 and cmp["arm_d"]["decisions"] == 2
    assert cmp["arm_f"]["decision_entropy_min"] < cmp["arm_d"]["decision_entropy_min"]
    assert cmp["arm_f"]["abs_advantage_max"] == 0.8
    assert B.main(["--traces", f"arm_d={tmp_path / 'd1.ndjson'}"]) == 0
    assert "arm_d" in capsys.readouterr().out
