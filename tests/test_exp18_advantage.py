"""Sweep-then-target protocol: coverage arithmetic, tokenizer rule, subset selection, budgets, a tiny run."""
import pytest
import torch

from chaoscontrol_b200 import exp18_advantage as A
from chaoscontrol_b200.models.model import CareStudentLM


def test_sweep_starts_do_not_overlap_and_cover_unique_targets():
    s = A.generate_sweep_starts(1000, 64)
    assert s[0] == 0 and all(b - a == 64 for a, b in zip(s, s[1:])) and s[-1] + 64 + 1 <= 1000
    assert A.count_unique_targets(s, 64) == len(s) * 64
    assert A.generate_sweep_starts(1000, 64, max_windows=3) == [0, 64, 128]
    assert A.generate_sweep_starts(10, 64) == []


def test_coverage_plan_marks_the_low_coverage_regime():
    full = A.build_coverage_plan(100_000, seq_len=100)
    assert full.coverage_frac == 1.0 and not full.low_coverage_regime
    low = A.build_coverage_plan(100_000, seq_len=100, projected_windows=full.total_windows // 5)
    assert low.low_coverage_regime and low.coverage_frac == pytest.approx(0.2, abs=0.01)


def test_phase_budget_accounts_selection_overhead():
    b = A.PhaseBudget(total_s=600.0, sweep_s=400.0, rescore_s=45.0, subset_s=5.0)
    assert b.remaining_s == 150.0 and b.selection_overhead_s == 50.0
    b.retarget_s = 200.0
    assert b.remaining_s == 0.0


def test_tokenizer_rule():
    a = {"tokenizer": "sp8192", "stable": True, "projected_coverage_frac": 0.50, "tokens_per_s": 9e5, "prior_mean_bpb": 1.967}
    b = {"tokenizer": "sp16384", "stable": True, "projected_coverage_frac": 0.47, "tokens_per_s": 8e5, "prior_mean_bpb": 1.959}
    assert A.choose_tokenizer([a, b])["tokenizer"] == "sp16384"            # within 10 % of coverage: better prior wins
    far = dict(b, projected_coverage_frac=0.30)
    assert A.choose_tokenizer([a, far])["tokenizer"] == "sp8192"           # coverage gap is material
    lowcov = dict(a, low_coverage_regime=True)
    assert A.choose_tokenizer([lowcov, dict(far, low_coverage_regime=False)])["tokenizer"] == "sp16384"
    assert A.choose_tokenizer([dict(a, stable=False), far])["tokenizer"] == "sp16384"
    with pytest.raises(ValueError):
        A.choose_tokenizer([dict(a, stable=False)])


def test_subset_selection():
    scored = [{"start": float(i * 8), "loss": float((i * 7) % 10)} for i in range(20)]
    top = A.select_subset(scored, fraction=0.1, mode="top", seed=0)
    assert len(top) == 2 and all(next(r for r in scored if r["start"] == s)["loss"] == 9.0 for s in top)
    r1, r2 = A.select_subset(scored, fraction=0.25, mode="random", seed=1), A.select_subset(scored, fraction=0.25, mode="random", seed=1)
    assert r1 == r2 and len(r1) == 5 and A.select_subset(scored, fraction=0.25, mode="random", seed=2) != r1
    with pytest.raises(ValueError):
        A.select_subset(scored, fraction=0.0, mode="top", seed=0)
    with pytest.raises(ValueError):
        A.select_subset(scored, fraction=0.5, mode="bottom", seed=0)


def test_phase_a_conditions():
    ph0 = {"selected": {"model_config": {"model_dim": 256, "vocab_size": 16384}, "batch_size": 512, "selected_lr": 0.016}}
    c = A.build_phase_a_conditions(ph0, total_budget_s=600.0)
    assert list(c) == ["baseline_b32", "sweep_only", "sweep_target_top10", "sweep_random_retrain"]
    assert c["baseline_b32"]["model_config"]["batch_size"] == 32 and c["baseline_b32"]["model_config"]["base_lr"] == 2e-3
    assert c["sweep_only"]["sweep_budget_s"] == 600.0 and c["sweep_only"]["model_config"]["base_lr"] == 0.016
    t, r = c["sweep_target_top10"], c["sweep_random_retrain"]
    assert (t["sweep_budget_s"], t["rescore_budget_s"], t["selection_budget_s"]) == (400.0, 45.0, 5.0)
    strip = lambda d: {k: v for k, v in d.items() if k not in ("condition", "subset_mode")}      # noqa: E731
    assert strip(t) == strip(r)                      # the control differs in the selection only


def test_scoring_and_a_tiny_sweep_target_run():
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=1, ff_mult=2)
    g = torch.Generator().manual_seed(1)
    easy = torch.arange(400) % 4                              # a period-4 pattern the model learns fast
    hard = torch.randint(0, 32, (400,), generator=g)
    tokens = torch.cat([easy, hard])
    dev = torch.device("cpu")
    starts = A.generate_sweep_starts(int(tokens.numel()), 16)
    sc = A.score_windows_by_loss(m, tokens=tokens, starts=starts, seq_len=16, batch_size=8, device=dev)
    assert sc["coverage_scored_frac"] == 1.0 and len(sc["scored"]) == len(starts)
    x = tokens[0:17]
    ref = torch.nn.functional.cross_entropy(m(x[None, :-1])["logits"][0].float(), x[1:]).item()
    assert sc["scored"][0]["loss"] == pytest.approx(ref, rel=1e-4)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-2)
    cond = {"condition": "sweep_target_top10", "train_mode": "target", "subset_fraction": 0.25, "subset_mode": "top",
            "total_budget_s": 20.0, "sweep_budget_s": 10.0, "rescore_budget_s": 5.0}
    # the retarget phase has no epoch limit: bound it through the budget
    cond["total_budget_s"] = 3.0
    out = A.run_sweep_target(m, opt, tokens=tokens, seq_len=16, batch_size=8, device=dev, condition=cond, seed=0)
    assert out["sweep"]["windows_seen"] == len(starts) and out["coverage"]["coverage_frac"] == 1.0
    assert out["subset_size"] == len(starts) // 4 and out["retarget"]["steps"] > 0
    assert out["budget"]["remaining_s"] <= 0.5 and out["budget"]["selection_overhead_s"] > 0
