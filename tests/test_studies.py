"""Experiments 09-17 as data: statistics against closed forms / scipy, matrix contents against the
reference's condition names and values, the layered protocol's inheritance, decisions on synthetic results."""
import json
import math

import pytest

from chaoscontrol_b200 import studies as S


def test_wilcoxon_exact_small_samples():
    assert S.wilcoxon_signed_rank_p([0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7]) == pytest.approx(2 / 128)
    assert S.wilcoxon_signed_rank_p([-0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7]) == pytest.approx(4 / 128)
    assert S.wilcoxon_signed_rank_p([0.0, 0.0]) == 1.0
    assert S.wilcoxon_signed_rank_p([1.0, -1.0]) == 1.0
    scipy_stats = pytest.importorskip("scipy.stats")
    d = [0.31, -0.12, 0.45, 0.07, -0.02, 0.22, 0.15, -0.3, 0.11]
    assert S.wilcoxon_signed_rank_p(d) == pytest.approx(scipy_stats.wilcoxon(d, mode="exact").pvalue)
    tied = [0.2, -0.2, 0.3, 0.3, 0.5, -0.1]
    assert 0 < S.wilcoxon_signed_rank_p(tied) <= 1


def test_welch_holm_cohens():
    scipy_stats = pytest.importorskip("scipy.stats")
    a, b = [1.50, 1.52, 1.49, 1.51], [1.60, 1.58, 1.63, 1.61, 1.59]
    t, p = S.welch_ttest(a, b)
    ref = scipy_stats.ttest_ind(a, b, equal_var=False)
    assert t == pytest.approx(ref.statistic) and p == pytest.approx(ref.pvalue, rel=1e-6)
    rows = S.holm_bonferroni([("x", 0.01), ("y", 0.04), ("z", 0.03)])
    assert [r[0] for r in rows] == ["x", "y", "z"]
    assert rows[0][2] == pytest.approx(0.03) and rows[2][2] == pytest.approx(0.06) and rows[1][2] == pytest.approx(0.06)
    assert [r[3] for r in rows] == [True, False, False]
    assert S.cohens_d(a, b) < -3
    lo, hi = S.bootstrap_ci(a)
    assert min(a) <= lo <= hi <= max(a) and S.bootstrap_ci(a) == (lo, hi)


def test_flat_study_matrices_carry_the_reference_condition_names():
    assert list(S.SLEEP_CYCLE.conditions) == ["no_sleep", "n3_only", "n2_n3", "n2_n3_rem_base", "n2_n3_rem_validate",
                                              "n2_n3_rem_cfr", "n2_n3_rem_reactivate", "n2_n3_rem_all", "full_cycle"]
    fc = S.SLEEP_CYCLE.conditions["full_cycle"]
    assert fc["sleep_stages"] == "full_cycle" and fc["sleep_interval"] == 256 and fc["batch_size"] == 64
    assert fc["outer_max_slots"] == 64 and fc["wernicke_k_max"] == 16 and fc["typed_storage"] is True
    assert len(S.entries(S.SLEEP_CYCLE)) == 63
    assert S.POLYPHASIC.conditions["polyphasic_K3_N4_striped"]["polyphasic_k_awake"] == 3
    c = S.CONSTANTS.conditions
    assert len(c) == 5 + 3 + 3 + 1 + 9 + 5 and "sem_b8_r1em02" in c and c["crit_088"]["crit_target_coupling"] == 0.88
    assert c["merge_090"]["sleep_stages"] == "n3_only" and c["memdim_128"]["outer_model_dim"] == 128
    assert "outer_model_dim" not in c["crit_080"]
    t3 = S.BUFFER_ROUTING.conditions
    assert t3["flat_64"]["wernicke_expert_dim"] == 32 and t3["hier_8x32"]["wernicke_expert_dim"] == 51
    assert S.BUFFER_RETRIEVAL.conditions["softmax_all_32"]["buffer_mode"] == "legacy"
    assert S.SUBWORD_SHAPES.conditions["sp_d192_L6"]["num_layers"] == 6
    assert S.SPARSE_ATTENTION.conditions["oracle_buf128_k8_xonly"]["oracle_query_source"] == "x"
    la = S.LOCAL_ATTENTION.conditions
    assert la["topk_random_16"]["local_attn_topk_random"] is True and la["local_w32"]["local_attn_window"] == 32
    assert S.resolve_data_paths("/d", 8192) == ("/d/datasets/fineweb10B_sp8192", "/d/tokenizers/fineweb_8192_bpe.model")


def test_architecture_baseline_study(tmp_path):
    st = S.ARCHITECTURE_BASELINES
    assert list(st.conditions)[:4] == ["mamba2", "bare_ssm", "ssm_wernicke_k16", "full_stack_k16"] and len(st.conditions) == 8
    assert st.conditions["ssm_wernicke_k64"]["wernicke_expert_dim"] == 16 and st.conditions["full_stack_k32"]["outer_max_slots"] == 64
    assert st.conditions["mamba2"]["model_type"] == "mamba2" and "wernicke_enabled" not in st.conditions["bare_ssm"]
    for i, s in enumerate(S.SEEDS7):
        j = 0.001 * ((i * 3) % 4)
        _write(tmp_path, "mamba2", s, 1.80 + j)
        _write(tmp_path, "bare_ssm", s, 1.80 + j + (0.002 if i % 2 else -0.002))
        _write(tmp_path, "full_stack_k16", s, 1.70 + j)
    out = S.analyse(st, tmp_path)
    assert out["decision"] == "FULL STACK BEATS MAMBA-2"
    assert {r["name"]: r["significant"] for r in out["confirmatory"]} == {"full_vs_mamba2": True, "core_vs_mamba2": False}


def _write(d, cond, seed, bpb):
    d.mkdir(parents=True, exist_ok=True)
    (d / f"{cond}_s{seed}.json").write_text(json.dumps({"eval": {"bpb": bpb}, "train": {"final_loss": 1.0}}))


def test_sleep_study_decision(tmp_path):
    for i, s in enumerate(S.SEEDS7):
        noise = 0.002 * ((i * 37) % 5)
        _write(tmp_path, "no_sleep", s, 2.00 + noise)
        _write(tmp_path, "full_cycle", s, 1.95 + noise * 0.8)
        _write(tmp_path, "n3_only", s, 1.97 + noise)
        _write(tmp_path, "n2_n3", s, 1.97 + noise + (0.001 if i % 2 else -0.001))
        _write(tmp_path, "n2_n3_rem_all", s, 1.96 + noise)
    out = S.analyse(S.SLEEP_CYCLE, tmp_path)
    conf = {r["name"]: r for r in out["confirmatory"]}
    assert conf["sleep_vs_none"]["p_raw"] == pytest.approx(2 / 128) and conf["sleep_vs_none"]["significant"]
    assert not conf["n2_value"]["significant"]
    assert out["decision"] == "ADOPT FULL CYCLE" and out["ranked"][0] == "full_cycle"
    for s in S.SEEDS7:
        _write(tmp_path, "full_cycle", s, 2.01)
    assert S.analyse(S.SLEEP_CYCLE, tmp_path)["decision"] == "SLEEP NOT HELPFUL YET"


def test_layered_protocol_hands_winner_settings_down(tmp_path):
    seen = {}

    def fake_run(cfgs, seeds, budget):
        seen[tuple(cfgs)] = (cfgs, budget)
        prefer = {"L0_fixed_k512", "L05_align_diversity", "L1_gate_mcts_k4", "L2_mem_both_warm_fullseq", "L3_wernicke_cfr",
                  "L35_full_stack_mc", "L4_full_256", "L5_full_256", "L6_wm_plus_all"}
        return {n: {s: (1.0 if n in prefer else 1.5) + 1e-3 * i for i, s in enumerate(seeds)} for n in cfgs}

    st = S.LayeredStudy(fake_run, state_path=tmp_path / "state.json")
    rep = st.run()
    assert [rep[l.tag]["winner"] for l in S.LAYERS] == ["L0_fixed_k512", "L05_align_diversity", "L1_gate_mcts_k4",
                                                        "L2_mem_both_warm_fullseq", "L3_wernicke_cfr", "L35_full_stack_mc",
                                                        "L4_full_256", "L5_full_256", "L6_wm_plus_all"]
    l3 = next(v for k, v in seen.items() if "L3_wernicke" in k)[0]
    base = l3["L3_no_wernicke"]
    assert base["tokenizer_codebook_size"] == 512 and base["align_type"] == "diversity"       # L0 + L0.5
    assert base["metabolic_mode"] == "mcts" and base["mcts_horizon"] == 8                      # L1
    assert base["consolidation_write"] == "full_sequence" and base["semantic_tier_bases"] == 8   # L2
    l6 = next(v for k, v in seen.items() if "L6_wm_only" in k)[0]
    assert l6["L6_wm_only"]["cfr_enabled"] is True and l6["L6_wm_only"]["eval_warmup"] is False
    assert next(v for k, v in seen.items() if "L5_full_128" in k)[1] == 1200.0                 # longer budget for the full matrix
    assert rep["L0"]["significant"] and rep["L0"]["runner_up"] is not None
    # resuming from the state file runs nothing again
    calls = len(seen)
    S.LayeredStudy(fake_run, state_path=tmp_path / "state.json").run()
    assert len(seen) == calls
    # a byte-level winner skips the alignment layer
    st2 = S.LayeredStudy(lambda c, s, b: {n: {x: (1.0 if n == "L0_bytes" else 2.0) for x in s} for n in c})
    assert "skipped" in st2.run(until="L05")["L05"]


def test_scaling_helpers():
    from chaoscontrol_b200.models.model import CareStudentLM
    m = CareStudentLM(vocab_size=256, dim=64, num_layers=2, ff_mult=2)
    assert sum(p.numel() for p in m.parameters()) == S.count_ssm_params(64, 2)
    for tag, (d, nl) in S.SIZE_TABLE.items():
        t = S.match_transformer_to_ssm(d, nl)
        assert abs(t["param_count"] - S.count_ssm_params(d, nl)) / S.count_ssm_params(d, nl) < (0.08 if tag == "XS" else 0.05), tag
    f_ssm = S.estimate_flops_per_step("ssm", 128, 4, 2, 256, 32)
    assert f_ssm == 6 * (4 * (5 + 4) * 128 * 128 + 2 * 256 * 128) * 32 * 256
    assert S.estimate_flops_per_step("transformer", 128, 4, 2, 256, 32) > 6 * 4 * 8 * 128 * 128 * 32 * 256
    assert S.estimate_flops_per_step("ssm", 128, 4, 2, 256, 32, metabolic_gate=True) > f_ssm
    cfgs = S.scaling_configs(full_stack={"wernicke_enabled": True, "model_dim": 999})
    assert cfgs["full_ssm_M"]["model_dim"] == 256 and cfgs["full_ssm_M"]["wernicke_enabled"] is True
    assert cfgs["our_tfm_XL"]["model_type"] == "transformer" and len(cfgs) == 15


def test_scaling_table_fits_a_power_law(tmp_path):
    cfgs = S.scaling_configs()
    for tag, (d, nl) in S.SIZE_TABLE.items():
        n = S.count_ssm_params(d, nl)
        for s in S.SEEDS3:
            _write(tmp_path, f"bare_ssm_{tag}", s, 1.2 + 40.0 * n ** -0.3)
    fit = S.scaling_table(tmp_path, cfgs)["bare_ssm"]["fit"]
    assert fit["alpha"] == pytest.approx(0.3, abs=0.03) and fit["bpb_irr"] == pytest.approx(1.2, abs=0.05)
