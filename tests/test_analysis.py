"""Result analysis: loading, per-arm summaries, seed-paired comparisons, verdicts, scaling fit."""
import json
import math

import pytest

from chaoscontrol_b200 import analysis as A


def _res(name, seed, arm, bpb, tok, loss=2.0, vram=1000.0, params=1000):
    return {"config": {"name": name, "seed": seed, "arm": arm}, "params": params,
            "train": {"aggregate_tokens_per_sec": tok, "steps": 10, "final_loss": loss, "peak_vram_mb": vram},
            "eval": {"bpb": bpb, "loss": 1.0}}


def test_load_summarize_compare_and_verdict(tmp_path, capsys):
    runs = []
    for s in range(5):
        runs.append(_res(f"ctl_s{s}", s, "control", 1.50 + 0.01 * s, 1000 + 5 * s))
        runs.append(_res(f"fast_s{s}", s, "fast", 1.47 + 0.01 * s, 1100 + 5 * s + (s % 2)))
        runs.append(_res(f"leaky_s{s}", s, "leaky", 1.50 + 0.01 * s, 1100 + 5 * s + (s % 2), vram=1200.0))
    for i, r in enumerate(runs):
        (tmp_path / f"r{i}.json").write_text(json.dumps(r))
    (tmp_path / "err.json").write_text(json.dumps({"error": "boom", "config": {"name": "x_s0", "seed": 0}}))
    (tmp_path / "junk.json").write_text("{not json")
    rows = A.load_results([tmp_path])
    assert len(rows) == 16 and sum(1 for r in rows if r["error"]) == 1
    table = A.summary_table(rows, "bpb")
    assert [t["arm"] for t in table][0] == "fast" and table[0]["n"] == 5
    assert abs(table[0]["std"] - math.sqrt(sum((0.01 * (s - 2)) ** 2 for s in range(5)) / 4)) < 1e-9
    cmp_ = {c["arm"]: c for c in A.paired_comparison(rows, control="control", metric="bpb")}
    assert abs(cmp_["fast"]["mean_delta"] + 0.03) < 1e-9 and cmp_["fast"]["fraction_beating_control"] == 1.0
    assert cmp_["fast"]["p"] == 0.0 and cmp_["leaky"]["fraction_beating_control"] == 0.0
    assert A.lever_verdict(rows, on="fast", off="control")["verdict"] == "SHIP"
    assert A.lever_verdict(rows, on="leaky", off="control")["verdict"] == "PARK"          # +20 % memory
    assert A.lever_verdict(rows, on="control", off="fast")["verdict"] == "PARK"          # slower
    assert A.main(["summarize", str(tmp_path)]) == 0 and "fast" in capsys.readouterr().out
    assert A.main(["compare", str(tmp_path), "--control", "control"]) == 0
    with pytest.raises(KeyError):
        A.paired_comparison(rows, control="nope")


def test_paired_ttest_matches_known_values():
    # hand-checked against the closed form: d = [1,2,3,4], mean 2.5, sd 1.2910, t = 3.873, df = 3, p = 0.03047
    t, p = A.paired_ttest([2, 4, 6, 8], [1, 2, 3, 4])
    assert abs(t - 3.8729833) < 1e-6 and abs(p - 0.030466) < 1e-5
    t, p = A.paired_ttest([1, 2, 3], [1, 2, 3])
    assert t == 0.0 and p == 1.0
    assert all(math.isnan(v) for v in A.paired_ttest([1.0], [2.0]))


def test_power_law_fit_recovers_its_parameters():
    A0, alpha, irr = 30.0, 0.25, 0.9
    params = [1e5, 3e5, 1e6, 3e6, 1e7]
    bpbs = [A0 * n ** -alpha + irr for n in params]
    fit = A.fit_power_law(params, bpbs)
    assert abs(fit["alpha"] - alpha) < 0.02 and abs(fit["bpb_irr"] - irr) < 0.02 and fit["r2"] > 0.999
    with pytest.raises(ValueError):
        A.fit_power_law([1, 2], [1.0, 0.9])


# ---------------------------------------------------------------------------
# replay-curation falsifier
# ---------------------------------------------------------------------------
def _curation_dir(tmp_path, rare):
    import json
    for arm, vals in rare.items():
        for i, v in enumerate(vals):
            (tmp_path / f"exp24_phase3_episodic_dw_curation_v1_{arm}_s{i}.json").write_text(json.dumps(
                {"name": f"exp24_phase3_episodic_dw_curation_v1_{arm}_s{i}", "val_bpb": 1.5,
                 "train": {"per_bucket_val_ce": [v, 1.0, 0.5]}, "config": {"seed": i}}))
    return tmp_path


@pytest.mark.parametrize("b,bp,want", [
    ([2.480, 2.481, 2.479], [2.498, 2.500, 2.499], "pass_mechanism_specific"),
    ([2.480, 2.481, 2.479], [2.480, 2.482, 2.479], "pass_mechanism_agnostic"),
    ([2.498, 2.497, 2.499], [2.50, 2.50, 2.50], "mixed_null"),          # better, but by less than 0.005
    ([2.520, 2.521, 2.519], [2.50, 2.50, 2.50], "regression"),
])
def test_curation_gate_verdicts(tmp_path, b, bp, want):
    from chaoscontrol_b200 import analysis as A
    d = _curation_dir(tmp_path, {"arm_a_uncurated": [2.500, 2.501, 2.499], "arm_b_cosine_utility": b,
                                 "arm_bp_pressure_only": bp, "arm_c_no_dw": [2.51, 2.51, 2.51]})
    cells = A.load_curation_cells(d)
    g = A.curation_gate(cells)
    assert g["verdict"] == want and g["by_arm_count"]["arm_b_cosine_utility"] == 3
    assert not g["needs_escalation"]
    text = A.render_curation(cells, g)
    assert "verdict:" in text and "arm_bp_pressure_only" in text
    assert A.main(["curation", str(d)]) == 0


def test_curation_gate_escalation_and_errors(tmp_path):
    from chaoscontrol_b200 import analysis as A
    d = _curation_dir(tmp_path, {"arm_a_uncurated": [2.5, 2.5, 2.5], "arm_b_cosine_utility": [2.46, 2.48, 2.47],
                                 "arm_bp_pressure_only": [2.5, 2.5, 2.5], "arm_c_no_dw": [2.5]})
    g = A.curation_gate(A.load_curation_cells(d))
    assert g["needs_escalation"] and g["sigma_b"] == pytest.approx(0.01)
    with pytest.raises(FileNotFoundError):
        A.load_curation_cells(tmp_path / "nothing")


def test_controller_arm_report_reads_results_and_learner_traces(tmp_path, capsys):
    """Per-arm table, event-path health and the sharp-over-default gradient ratios from real learner traces."""
    import json
    from chaoscontrol_b200 import analysis as A
    from chaoscontrol_b200.episodic import bootstrap_bench as B
    res, tr = tmp_path / "results", tmp_path / "traces"
    res.mkdir(); tr.mkdir()
    for arm, T in (("arm_d_simplex_online", 1.0), ("arm_f_simplex_sharp_online", 0.2)):
        for seed in (1, 2):
            cell = {"train": {"steps": 100 + seed, "elapsed_s": 10.0, "final_loss": 4.0 + 0.1 * seed,
                              "episodic": {"write_events_emitted": 50, "write_events_dropped": seed, "write_events_ingested": 49}}}
            (res / f"exp_{arm}_s{seed}.json").write_text(json.dumps(cell))
            B.run_bootstrap(temperature=T, events=200, seed=seed, trace_path=tr / f"ctl_{arm}_s{seed}.ndjson")
    (res / "exp_unrelated.json").write_text("{}")
    rep = A.controller_arm_report(res, tr, prefix="exp_", trace_prefix="ctl_",
                                  headline=("arm_d_simplex_online", "arm_f_simplex_sharp_online"))
    assert [r["arm"] for r in rep["arms"]] == ["arm_d_simplex_online", "arm_f_simplex_sharp_online"]
    d = rep["arms"][0]
    assert d["n"] == 2 and abs(d["steps_per_s"] - 10.15) < 1e-9 and abs(d["final_loss"] - 4.15) < 1e-9 and d["final_loss_std"] > 0
    assert [h["dropped"] for h in rep["health"]] == [1, 2, 1, 2] and all(h["sgd_steps"] > 0 for h in rep["health"])
    assert rep["traces"]["arm_f_simplex_sharp_online"]["seeds"] == 2 and rep["headline"]["grad_logits_l2"]["ratio"] > 1
    assert A.main(["controller-arms", str(res), "--traces-dir", str(tr), "--prefix", "exp_", "--trace-prefix", "ctl_",
                   "--headline", "arm_d_simplex_online", "arm_f_simplex_sharp_online"]) == 0
    out = capsys.readouterr().out
    assert "## Per arm" in out and "Event path health" in out and "arm_f_simplex_sharp_online over arm_d_simplex_online" in out
    # without traces the report still has the two result tables
    rep2 = A.controller_arm_report(res, None, prefix="exp_")
    assert "traces" not in rep2 and all(h["sgd_steps"] is None for h in rep2["health"])
