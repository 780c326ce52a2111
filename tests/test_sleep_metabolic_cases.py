"""Sleep cycle stages and the metabolic gate, one property per test (CPU)."""
import copy
import math

import pytest
import torch

from chaoscontrol_b200.metabolic import StructuredProjections, metabolic_fork, metabolic_monte_carlo, micro_mcts
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.regret import RegretTable
from chaoscontrol_b200.sleep import SleepConfig, SleepCycle
from chaoscontrol_b200.wake_cache import WakeCache


def _memory_model(**kw):
    torch.manual_seed(0)
    base = dict(vocab_size=48, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot", outer_max_slots=32)
    base.update(kw)
    return CareStudentLM(**base)


def _sleepy(survival=(1.0, 1.0, 1.0, 0.0, 1.0, 0.01), moments=2, **kw):
    m = _memory_model(**kw)
    om = m.outer_model
    torch.manual_seed(1)
    base = torch.randn(1, 8)
    om.append_kv_batch(torch.cat([base, base * 1.01, torch.randn(4, 8)], 0), torch.tensor([0, 0, 1, 1, 2, 2]))
    om._survival[:] = list(survival)
    cache = WakeCache()
    for s in range(moments):
        ids = torch.randint(0, 48, (2, 9))
        cache.record_moment(surprise=2.0 + s, inputs=ids[:, :-1], targets=ids[:, 1:], hidden=torch.zeros(2, 8, 16),
                            bucket_ids=torch.zeros(2, 8, dtype=torch.long))
    return m, cache


# ---------------------------------------------------------------- configuration
@pytest.mark.parametrize("stages,n1,n2,rem", [
    ("n3_only", False, False, False), ("n2_n3", False, True, False), ("n2_n3_rem_base", False, True, True),
    ("n2_n3_rem_validate", False, True, True), ("n2_n3_rem_cfr", False, True, True),
    ("n2_n3_rem_reactivate", False, True, True), ("n2_n3_rem_all", False, True, True), ("full_cycle", True, True, True)])
def test_stage_names_select_the_stages(stages, n1, n2, rem):
    c = SleepConfig(stages=stages)
    assert (c.use_n1, c.use_n2, c.use_n3, c.use_rem) == (n1, n2, True, rem)


def test_config_defaults():
    c = SleepConfig()
    assert c.stages == "full_cycle" and c.budget == 128 and c.n2_budget == 64 and c.rem_budget == 64
    assert c.merge_sim_threshold == 0.85 and c.survival_floor == 0.1 and c.rem_dreams == 4 and c.rem_length == 128
    assert c.rem_validate and c.rem_cfr and c.rem_reactivate


# ---------------------------------------------------------------- N1 / N2
def test_n1_flags_slots_with_zero_survival():
    m, _ = _sleepy()
    d = SleepCycle()._n1_transition(m.outer_model)
    assert d == {"unstable_count": 1, "unstable_indices": [3]}


def test_n2_moves_survival_by_the_leave_one_out_utility():
    m, cache = _sleepy()
    om = m.outer_model
    before = list(om._survival)
    d = SleepCycle(SleepConfig(stages="n2_n3"))._n2_tag(m, om, cache, "cpu")
    util = dict(d["utilities"])
    assert set(util) == set(range(6)) and d["ops"] == 6
    for i in range(6):
        assert om._survival[i] == pytest.approx(before[i] + util[i])
    assert any(abs(u) > 0 for u in util.values())


def test_n2_respects_its_budget_and_skip_set():
    m, cache = _sleepy()
    d = SleepCycle(SleepConfig(stages="n2_n3", n2_budget=2))._n2_tag(m, m.outer_model, cache, "cpu")
    assert d["slots_scored"] == 2
    d2 = SleepCycle(SleepConfig(stages="n2_n3"))._n2_tag(m, m.outer_model, cache, "cpu", skip_indices={0, 1, 2})
    assert d2["slots_scored"] == 3 and d2["slots_skipped_unstable"] == 3 and not {0, 1, 2} & {s for s, _ in d2["utilities"]}


def test_n2_without_cached_batches_or_slots_is_a_no_op():
    m, _ = _sleepy()
    before = list(m.outer_model._survival)
    d = SleepCycle()._n2_tag(m, m.outer_model, WakeCache(), "cpu")
    assert d["ops"] == 0 and d["reason"] == "no cached batches" and list(m.outer_model._survival) == before
    empty = _memory_model()
    assert SleepCycle()._n2_tag(empty, empty.outer_model, WakeCache(), "cpu") == {"ops": 0, "slots_scored": 0}


def test_n2_group_size_does_not_change_the_utilities():
    a, cache = _sleepy()
    b = copy.deepcopy(a)
    ua = dict(SleepCycle(SleepConfig(stages="n2_n3", loo_group=1))._n2_tag(a, a.outer_model, cache, "cpu")["utilities"])
    ub = dict(SleepCycle(SleepConfig(stages="n2_n3", loo_group=6))._n2_tag(b, b.outer_model, cache, "cpu")["utilities"])
    assert ua.keys() == ub.keys() and all(ua[k] == pytest.approx(ub[k], abs=1e-5) for k in ua)


# ---------------------------------------------------------------- N3
def test_n3_prunes_below_the_floor_and_leaves_latent_traces():
    m, _ = _sleepy()
    om = m.outer_model
    doomed = [om.table._store[i].clone() for i in (3, 5)]
    d = SleepCycle(SleepConfig(stages="n2_n3", merge_sim_threshold=2.0))._n3_rewrite(m, om)
    assert d["pruned"] == 2 and d["latent_traces_created"] == 2 and d["slots_remaining"] == 4 == len(om.table)
    assert [t["bucket_id"] for t in om._latent_traces] == [1, 2]
    assert all(torch.equal(t["centroid_contrib"][0], v) for t, v in zip(om._latent_traces, doomed))


def test_n3_keeps_everything_above_the_floor():
    m, _ = _sleepy(survival=(1.0,) * 6)
    d = SleepCycle(SleepConfig(stages="n2_n3", merge_sim_threshold=2.0))._n3_rewrite(m, m.outer_model)
    assert d["pruned"] == 0 and d["merges_proposed"] == 0 and len(m.outer_model.table) == 6 and not m.outer_model._latent_traces


def test_n3_only_commits_merges_at_once_and_rem_modes_defer_them():
    m, _ = _sleepy(survival=(1.0,) * 6)
    cyc = SleepCycle(SleepConfig(stages="n3_only"))
    d = cyc._n3_rewrite(m, m.outer_model)
    assert d["merges_committed"] == 1 and len(m.outer_model.table) == 5 and cyc._provisional_merges == []
    m2, _ = _sleepy(survival=(1.0,) * 6)
    cyc2 = SleepCycle(SleepConfig(stages="n2_n3_rem_validate"))
    d2 = cyc2._n3_rewrite(m2, m2.outer_model)
    assert d2["merges_committed"] == 0 and d2["merges_proposed"] == 1 and len(m2.outer_model.table) == 6
    assert len(cyc2._provisional_merges) == 1 and {cyc2._provisional_merges[0]["idx_a"], cyc2._provisional_merges[0]["idx_b"]} == {0, 1}


def test_merge_is_the_survival_weighted_mean_and_retires_the_partner():
    m, _ = _sleepy(survival=(3.0, 1.0, 1.0, 1.0, 1.0, 1.0))
    om = m.outer_model
    a, b = om.table._store[0].clone(), om.table._store[1].clone()
    id_a, id_b = om.table.physical_to_slot_id(0), om.table.physical_to_slot_id(1)
    SleepCycle(SleepConfig(stages="n3_only"))._n3_rewrite(m, om)
    assert torch.allclose(om.table.get_tensor(id_a)[0], (3 * a + b) / 4, atol=1e-6) and om.table.get_tensor(id_b) is None
    assert om.table._survival[om.table.slot_id_to_physical(id_a)] == pytest.approx(2.0)
    assert om._latent_traces[-1]["bucket_id"] == 0 and torch.equal(om._latent_traces[-1]["centroid_contrib"][0], b)


def test_commit_merge_is_addressed_by_slot_id():
    m, _ = _sleepy(survival=(1.0,) * 6)
    om = m.outer_model
    cyc = SleepCycle()
    prop = cyc._proposal(om, 0, 1, 0.99)
    om.table.retire(om.table.physical_to_slot_id(1))                    # the partner vanished meanwhile
    assert cyc._commit_merge(om, prop) is False and len(om.table) == 5


def test_pair_candidates_threshold_and_first_fit():
    m, _ = _sleepy(survival=(1.0,) * 6)
    cyc = SleepCycle()
    pairs = cyc._pair_candidates(m.outer_model, list(range(6)), 0.9)
    assert [(i, j) for i, j, _ in pairs] == [(0, 1)] and pairs[0][2] > 0.999
    assert cyc._pair_candidates(m.outer_model, [0], 0.0) == []
    everything = cyc._find_similar_pairs(m.outer_model, list(range(6)), -1.0)
    used = [p["idx_a"] for p in everything] + [p["idx_b"] for p in everything]
    assert len(everything) == 3 and sorted(used) == list(range(6))        # each slot joins one proposal


# ---------------------------------------------------------------- REM
def test_validation_accepts_a_duplicate_merge_and_rejects_a_harmful_one(monkeypatch):
    m, cache = _sleepy(survival=(1.0,) * 6)
    om, cyc = m.outer_model, SleepCycle()
    batches = cyc._gather_batches(cache, "cpu", None)
    good = cyc._proposal(om, 0, 1, 0.99)
    seq = iter([1.0])
    monkeypatch.setattr(cyc, "_compute_mean_ce", lambda *a, **k: 1.0)
    monkeypatch.setattr(cyc, "_ce_variants", lambda *a, **k: torch.tensor([0.9]))
    assert cyc._validate_merge(m, om, good, batches, "cpu") is True
    monkeypatch.setattr(cyc, "_ce_variants", lambda *a, **k: torch.tensor([1.5]))
    assert cyc._validate_merge(m, om, good, batches, "cpu") is False
    assert cyc._validate_merge(m, om, good, [], "cpu") is True            # nothing to judge by: accept


def test_rem_counts_dreams_and_cfr_updates_move_the_regret_table():
    m, cache = _sleepy(survival=(1.0,) * 6)
    reg = RegretTable(4, 4)
    cyc = SleepCycle(SleepConfig(stages="n2_n3_rem_cfr", rem_dreams=3, rem_length=2, rem_budget=64))
    d = cyc._rem_dream(m, m.outer_model, cache, "cpu", regret_table=reg, validate_merges=False)
    assert d["dreams"] == 3 and d["cfr_updates"] == 3 and d["ops"] >= 3 * 2 and float(reg.cumulative_regret.abs().sum()) > 0
    assert d["merges_accepted"] == d["merges_rejected"] == 0 and math.isfinite(d["mean_dream_score"])


def test_rem_with_no_slots_returns_early():
    empty = _memory_model()
    d = SleepCycle()._rem_dream(empty, empty.outer_model, WakeCache(), "cpu")
    assert d == {"ops": 0, "dreams": 0, "reason": "no slots to dream from"}


def test_rem_budget_caps_dream_length():
    m, cache = _sleepy(survival=(1.0,) * 6)
    cyc = SleepCycle(SleepConfig(stages="n2_n3_rem_base", rem_dreams=4, rem_length=100, rem_budget=8))
    d = cyc._rem_dream(m, m.outer_model, cache, "cpu", validate_merges=False)
    assert d["ops"] == 4 * 2 and d["dreams"] == 4                          # 8 // 4 tokens per dream


# ---------------------------------------------------------------- whole cycle
@pytest.mark.parametrize("stages", ["n3_only", "n2_n3", "n2_n3_rem_base", "n2_n3_rem_all", "full_cycle"])
def test_every_stage_set_runs_and_reports_ops(stages):
    m, cache = _sleepy()
    d = SleepCycle(SleepConfig(stages=stages, rem_dreams=2, rem_length=2, rem_budget=16)).run(m, cache, "cpu",
                                                                                             regret_table=RegretTable(4, 4))
    assert ("n1" in d) == (stages == "full_cycle") and ("n2" in d) == (stages != "n3_only") and "n3" in d
    assert ("rem" in d) == stages.startswith(("n2_n3_rem", "full")) and d["total_ops"] >= d["n3"]["ops"] > 0
    ids = torch.randint(0, 48, (1, 6))
    assert torch.isfinite(m(ids)["logits"]).all()


def test_total_ops_is_the_sum_of_the_stage_ops():
    m, cache = _sleepy()
    d = SleepCycle(SleepConfig(stages="n2_n3_rem_base", rem_dreams=2, rem_length=2, rem_budget=16)).run(m, cache, "cpu")
    assert d["total_ops"] == d["n2"]["ops"] + d["n3"]["ops"] + d["rem"]["ops"]


def test_cycle_without_memory_module_is_skipped_and_semantic_tier_is_recomputed_when_present():
    plain = CareStudentLM(vocab_size=48, dim=16, num_layers=1)
    assert SleepCycle().run(plain, WakeCache(), "cpu") == {"total_ops": 0, "skipped": "no multislot outer model"}
    m, cache = _sleepy(semantic_tier_bases=3)
    d = SleepCycle(SleepConfig(stages="n3_only")).run(m, cache, "cpu")
    assert d["semantic_recomputed"] is True and float(m.semantic_tier.bases.abs().sum()) > 0
    m2, cache2 = _sleepy()
    assert "semantic_recomputed" not in SleepCycle(SleepConfig(stages="n3_only")).run(m2, cache2, "cpu")


# ---------------------------------------------------------------- metabolic gate
def _lm():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=32, dim=16, num_layers=1).eval()


IDS = torch.randint(0, 32, (2, 7), generator=torch.Generator().manual_seed(3))


@pytest.mark.parametrize("mode", ["ensemble_agreement", "loss_lookahead", "memory_consistency", "something_else"])
def test_fork_returns_one_candidate_for_every_score_mode(mode):
    torch.manual_seed(1)
    r = metabolic_fork(_lm(), IDS, k=3, noise_std=0.05, score_mode=mode)
    assert r["logits"].shape == (2, 7, 32) and r["hidden"].shape == (2, 7, 16) and 0 <= r["best_idx"] < 3


def test_fork_with_zero_noise_equals_the_plain_forward():
    m = _lm()
    r = metabolic_fork(m, IDS, k=3, noise_std=0.0, score_mode="ensemble_agreement")
    assert torch.allclose(r["logits"], m(IDS)["logits"], atol=1e-5)


def test_fork_prior_bias_can_pick_the_candidate():
    torch.manual_seed(1)
    r = metabolic_fork(_lm(), IDS, k=4, noise_std=0.05, score_mode="loss_lookahead",
                       prior_bias=torch.tensor([0.0, 0.0, 50.0, 0.0]))
    assert r["best_idx"] == 2


def test_structured_projections_give_k_distinct_views():
    torch.manual_seed(0)
    sp = StructuredProjections(16, k=3)
    views = sp(torch.randn(2, 5, 16))
    assert len(views) == 3 and all(v.shape == (2, 5, 16) for v in views) and not torch.allclose(views[0], views[1])
    r = metabolic_fork(_lm(), IDS, k=3, generation_mode="structured", structured_proj=sp, score_mode="ensemble_agreement")
    assert r["logits"].shape == (2, 7, 32)


@torch.no_grad()
def test_monte_carlo_statistics_are_bounded_and_shaped():
    torch.manual_seed(1)
    r = metabolic_monte_carlo(_lm(), IDS, k=5, noise_std=0.05)
    st = r["mc_stats"]
    assert r["logits"].shape == (2, 7, 32) and st["logits_var"].shape == st["entropy"].shape == (2, 7)
    assert float(st["entropy"].min()) >= 0 and float(st["entropy"].max()) <= math.log(32) + 1e-4
    assert float(st["agreement"].min()) >= 0 and float(st["agreement"].max()) <= 1
    assert float(st["uncertainty_map"].min()) >= 0 and float(st["uncertainty_map"].max()) <= 1 + 1e-4
    assert float(st["candidate_divergence"]) >= 0


@torch.no_grad()
def test_monte_carlo_more_noise_means_more_variance_and_divergence():
    m = _lm()
    torch.manual_seed(1)
    lo = metabolic_monte_carlo(m, IDS, k=6, noise_std=0.01)["mc_stats"]
    torch.manual_seed(1)
    hi = metabolic_monte_carlo(m, IDS, k=6, noise_std=0.3)["mc_stats"]
    assert float(hi["logits_var"].mean()) > float(lo["logits_var"].mean())
    assert float(hi["candidate_divergence"]) > float(lo["candidate_divergence"])


@torch.no_grad()
def test_monte_carlo_with_zero_noise_has_no_disagreement():
    st = metabolic_monte_carlo(_lm(), IDS, k=4, noise_std=0.0)["mc_stats"]
    assert float(st["logits_var"].abs().max()) < 1e-10 and float(st["candidate_divergence"]) < 1e-6


def test_mcts_zero_rollouts_is_the_plain_forward_and_rollouts_touch_only_the_last_position():
    m = _lm()
    plain = m(IDS)["logits"]
    assert torch.allclose(micro_mcts(m, IDS, n_rollouts=0)["logits"], plain)
    torch.manual_seed(2)
    r = micro_mcts(m, IDS, n_rollouts=4, horizon=2)
    assert torch.allclose(r["logits"][:, :-1], plain[:, :-1]) and not torch.allclose(r["logits"][:, -1], plain[:, -1])
    st = r["mcts_stats"]
    assert int(st["visit_counts"].sum()) == 4 and st["visit_counts"].numel() == 8 and math.isfinite(st["root_value"])


def test_mcts_exploration_constant_changes_the_visits():
    m = _lm()
    torch.manual_seed(2)
    a = micro_mcts(m, IDS, n_rollouts=8, horizon=1, ucb_c=0.0)["mcts_stats"]["visit_counts"]
    torch.manual_seed(2)
    b = micro_mcts(m, IDS, n_rollouts=8, horizon=1, ucb_c=50.0)["mcts_stats"]["visit_counts"]
    assert int((a > 0).sum()) <= int((b > 0).sum())                       # more exploration: at least as many arms
