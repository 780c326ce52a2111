"""Simplex bootstrap microbench and learner-trace comparison."""
import json
import math

import pytest

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


def test_credit_rows_carry_gradient_diagnostics_and_the_headline_ratio(tmp_path):
    """A sharper start accumulates a larger policy gradient per credited action than the default start."""
    import json
    paths = {}
    for arm, T in (("arm_d", 1.0), ("arm_f", 0.2)):
        paths[arm] = tmp_path / f"{arm}.ndjson"
        B.run_bootstrap(temperature=T, events=400, seed=0, trace_path=paths[arm])
    rows = [json.loads(l) for l in paths["arm_f"].read_text().splitlines()]
    credit = [r for r in rows if r["row_type"] == "credit"]
    assert credit and all(set(B.GRADIENT_COLUMNS) <= set(r) for r in credit)
    assert all(r["grad_w_lh_accum_l2"] >= 0 and r["w_lh_l2"] >= 0 and r["entropy"] is not None for r in credit)
    # the accumulator holds this credit's own gradient right after an SGD apply emptied it
    first = credit[0]
    assert first["grad_w_lh_accum_l2"] == pytest.approx(first["grad_w_lh_l2"], rel=1e-4)
    cmp = B.compare_traces({k: [v] for k, v in paths.items()})
    assert cmp["arm_f"]["grad_logits_l2_mean"] > 0 and cmp["arm_f"]["entropy_drift_mean"] is not None
    h = B.headline_ratio(cmp, "arm_d", "arm_f")
    assert h["grad_logits_l2"]["ratio"] > 1.0 and isinstance(h["confirmed"], bool)
