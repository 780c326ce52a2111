"""Residual-memory maintenance, one property per test: helpers, evidence update, policies, agreement
gate, oracle gate, commits, receipts and state (CPU)."""
import dataclasses
import json
import math

import pytest
import torch

from chaoscontrol_b200 import replay_eviction as RE
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.slot_table import (SLOT_ACTIVE, SLOT_DECAYING, SLOT_QUARANTINED, SLOT_WARMING, SlotRecord)

KW = dict(eviction_threshold=0.01, useful_threshold=0.005, drift_threshold=0.3, quarantine_threshold=-0.01,
          distill_peak_threshold=0.04, peak_preserve_utility_threshold=0.2, peak_preserve_sharpness_threshold=0.2,
          min_age=128)


def _model(n_slots=5, seed=0):
    torch.manual_seed(seed)
    m = CareStudentLM(vocab_size=40, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                      outer_max_slots=0, buffer_mode="append_only")
    m.append_memory_from_hidden(torch.randn(1, n_slots, 16), event_ids=torch.arange(1, n_slots + 1).view(1, -1))
    return m.eval()


def _probe(B=2, T=9, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 40, (B, T), generator=g), torch.ones(B, T, dtype=torch.bool)


def _rec(**kw):
    return SlotRecord(**{**dict(slot_id=1, created_step=0, last_scored_step=500, score_count=5), **kw})


def _loop(**kw):
    base = dict(commit_policy="rule", min_slot_age_steps=0, action_agreement_count=1, max_seconds_per_tick=0.0)
    return RE.ReplayEvictionLoop(**{**base, **kw})


# ---------------------------------------------------------------------------
# helpers and records
# ---------------------------------------------------------------------------
def test_evict_single_and_multiple_physical_rows():
    m = _model(5)
    t = m.outer_model.table
    ids = [t.physical_to_slot_id(i) for i in range(5)]
    assert RE._evict_slots(m.outer_model, [1]) == [ids[1]] and t.n_active == 4
    gone = RE._evict_slots(m.outer_model, [0, 2])              # rows were compacted: these are two other slots
    assert len(gone) == 2 and t.n_active == 2 and ids[1] not in gone


def test_evict_out_of_range_and_empty_are_ignored():
    m = _model(3)
    assert RE._evict_slots(m.outer_model, []) == [] and RE._evict_slots(m.outer_model, [17, -9]) == []
    assert m.outer_model.table.n_active == 3


def test_evict_all_leaves_an_empty_readable_table():
    m = _model(3)
    RE._evict_slots(m.outer_model, [0, 1, 2])
    assert m.outer_model.table.n_active == 0
    ids, valid = _probe()
    assert RE.replay_score_slots(model=m, probe_input_ids=ids, probe_valid_mask=valid)["slot_indices"] == []
    assert torch.isfinite(m(ids)["logits"]).all()


def test_tick_result_defaults_and_evicted_view():
    r = RE.TickResult()
    assert r.evicted_indices == [] and r.slot_commits == [] and r.refreshed == []
    r.evicted += [4, 2]
    view = r.evicted_indices
    view.append(9)
    assert r.evicted == [4, 2]                                   # a copy, not the list itself


def test_receipt_and_event_carry_their_fields():
    rc = RE.DistillReceipt(3, 10, 0.01, 0.2, 0.01, "bucket_prototype")
    assert not rc.accepted and not rc.prototype_updated and rc.prototype_reason == ""
    ev = RE.MemoryEvent(step=5, tick=2, slot_id=3, action="EVICT")
    d = dataclasses.asdict(ev)
    assert d["accepted"] is True and d["reason"] == "" and {"peak_utility", "retrieval_mass", "refresh_candidate"} <= set(d)
    json.dumps(d)


def test_replay_score_without_memory_module_is_empty():
    m = CareStudentLM(vocab_size=40, dim=16, num_layers=1)
    ids, valid = _probe()
    out = RE.replay_score_slots(model=m, probe_input_ids=ids, probe_valid_mask=valid)
    assert out["slot_indices"] == [] and out["mean_utility"] == 0.0 and out["slot_utilities"].numel() == 0


def test_replay_score_shapes_and_weights():
    m = _model(4)
    ids, valid = _probe(B=3, T=7)
    out = RE.replay_score_slots(model=m, probe_input_ids=ids, probe_valid_mask=valid)
    assert out["slot_utilities"].shape == (4,) and out["slot_indices"] == [0, 1, 2, 3]
    assert out["retrieval_weights"].shape == (3, 4) and out["per_token_utility"].shape == out["mask"].shape
    assert out["n_tokens_scored"] == int(out["mask"].sum()) > 0
    assert torch.allclose(out["retrieval_weights"].float().sum(1), torch.ones(3), atol=1e-2)   # bf16 weights


def test_probe_chunking_does_not_change_values():
    m = _model(6)
    ids, valid = _probe()
    kw = dict(model=m, outer=m.outer_model, probe_input_ids=ids, probe_valid_mask=valid)
    a = RE.counterfactual_probe(chunk_size=64, **kw)
    b = RE.counterfactual_probe(chunk_size=2, **kw)
    assert torch.allclose(a.marginal_gains, b.marginal_gains, atol=1e-5)
    assert torch.allclose(a.sidecar_value, b.sidecar_value, atol=1e-5)


def test_subset_probe_matches_full_probe_rows():
    m = _model(6)
    ids, valid = _probe()
    kw = dict(model=m, outer=m.outer_model, probe_input_ids=ids, probe_valid_mask=valid)
    full = RE.counterfactual_probe(**kw)
    sub = RE.counterfactual_probe(score_slot_indices=[4, 1], **kw)
    assert sub.slot_indices == [4, 1] or sorted(sub.slot_indices) == [1, 4]
    for j, p in enumerate(sub.slot_indices):
        assert torch.allclose(sub.marginal_gains[j], full.marginal_gains[full.slot_indices.index(p)], atol=1e-5)


def test_valid_mask_restricts_scoring():
    m = _model(3)
    ids, valid = _probe(B=2, T=9)
    valid[:, 5:] = False
    r = RE.counterfactual_probe(model=m, outer=m.outer_model, probe_input_ids=ids, probe_valid_mask=valid)
    assert int(r.mask.sum()) < ids.numel() and not bool(r.mask[:, -1].any())


# ---------------------------------------------------------------------------
# sharpness and drift
# ---------------------------------------------------------------------------
def test_sharpness_high_variance_beats_uniform_and_handles_empty():
    mask = torch.ones(1, 8, dtype=torch.bool)
    spiky = torch.zeros(1, 1, 8)
    spiky[0, 0, 3] = 4.0
    flat = torch.full((1, 1, 8), 0.5)
    s = RE._per_slot_sharpness(torch.cat([spiky, flat]), mask)
    assert s[0] > 1.0 and s[1] == pytest.approx(0.0, abs=1e-7)
    assert RE._per_slot_sharpness(torch.zeros(0, 1, 8), mask).numel() == 0


def test_sharpness_ignores_masked_tokens():
    mask = torch.tensor([[True, True, False, False]])
    g = torch.tensor([[[1.0, 1.0, 50.0, -50.0]]])
    assert float(RE._per_slot_sharpness(g, mask)[0]) == pytest.approx(0.0, abs=1e-6)


def test_representation_drift_zero_for_a_fixed_point_and_without_coders():
    class Outer:
        encoder = torch.nn.Linear(4, 4, bias=False)
        decoder = torch.nn.Linear(4, 4, bias=False)
    with torch.no_grad():
        Outer.encoder.weight.copy_(torch.eye(4))
        Outer.decoder.weight.copy_(torch.eye(4))
    small = torch.tensor([[0.01, -0.02, 0.015, 0.005]])              # tanh is the identity to 1e-6 here
    assert RE._representation_drift(Outer, small) == pytest.approx(0.0, abs=1e-4)
    with torch.no_grad():
        Outer.encoder.weight.copy_(-torch.eye(4))
    assert RE._representation_drift(Outer, small) == pytest.approx(2.0, abs=1e-3)
    assert RE._representation_drift(object(), small) == 0.0


# ---------------------------------------------------------------------------
# rule policy, one case each
# ---------------------------------------------------------------------------
POL = RE.MaintenancePolicy()


def test_policy_preserves_useful_slot():
    assert POL.choose(_rec(marginal_gain_ema=0.1, utility_ema=0.1, peak_utility=0.1), **KW) == "PRESERVE"


def test_policy_low_utility_below_capacity_decays_not_evicts():
    v = POL.action_values(_rec(utility_ema=0.0), capacity_pressure=False, **KW)
    assert v["EVICT"] == 0.0 and v["DECAY"] > 0 and max(v, key=v.get) == "DECAY"


def test_policy_capacity_pressure_evicts_low_utility():
    v = POL.action_values(_rec(utility_ema=0.0), capacity_pressure=True, **KW)
    assert v["DECAY"] == 0.0 and max(v, key=v.get) == "EVICT"


def test_policy_quarantines_contradicting_slot_and_streak_raises_value():
    a = POL.action_values(_rec(contradiction_ema=0.3, negative_streak=0), **KW)["QUARANTINE"]
    b = POL.action_values(_rec(contradiction_ema=0.3, negative_streak=4), **KW)["QUARANTINE"]
    assert b == pytest.approx(a + 2.0) and POL.choose(_rec(contradiction_ema=0.3, negative_streak=4), **KW) == "QUARANTINE"


def test_policy_distills_absorbed_slot():
    rec = _rec(marginal_gain_ema=0.001, utility_ema=0.05, peak_utility=0.15)
    v = POL.action_values(rec, **KW)
    assert v["DISTILL"] == pytest.approx((1 - 0.001 / 0.15) * 0.15) and POL.choose(rec, **KW) == "DISTILL"


def test_policy_peak_utility_blocks_distill_and_evict():
    rec = _rec(marginal_gain_ema=0.001, utility_ema=0.0, peak_utility=0.5)
    v = POL.action_values(rec, capacity_pressure=True, **KW)
    assert v["DISTILL"] == 0.0 and v["EVICT"] == 0.0


def test_policy_peak_sharpness_blocks_distill_and_evict():
    rec = _rec(marginal_gain_ema=0.001, utility_ema=0.0, peak_utility=0.1, peak_sharpness=0.4)
    v = POL.action_values(rec, capacity_pressure=True, **KW)
    assert v["DISTILL"] == 0.0 and v["EVICT"] == 0.0 and max(v, key=v.get) == "PRESERVE"


def test_policy_refreshes_drifted_but_useful_slot_only():
    assert POL.choose(_rec(marginal_gain_ema=0.05, utility_ema=0.05, representation_drift_ema=0.6), **KW) == "REFRESH"
    useless = POL.action_values(_rec(marginal_gain_ema=0.0, representation_drift_ema=0.6), **KW)
    assert useless["REFRESH"] == 0.0
    for field in ("activation_drift_ema", "semantic_drift_ema"):
        assert POL.action_values(_rec(marginal_gain_ema=0.05, **{field: 0.6}), **KW)["REFRESH"] > 0


def test_policy_young_or_unscored_slot_gets_no_mutating_value():
    for rec in (_rec(last_scored_step=10, contradiction_ema=0.3, peak_utility=0.15),
                _rec(score_count=0, contradiction_ema=0.3, peak_utility=0.15)):
        v = POL.action_values(rec, capacity_pressure=True, **KW)
        assert v["QUARANTINE"] == v["DISTILL"] == v["EVICT"] == 0.0


def test_policy_release_only_for_quarantined():
    assert POL.action_values(_rec(marginal_gain_ema=0.3, positive_streak=4), **KW)["RELEASE"] == 0.0
    q = _rec(state=SLOT_QUARANTINED, marginal_gain_ema=0.3, positive_streak=4, utility_ema=0.3)
    assert POL.action_values(q, **KW)["RELEASE"] == pytest.approx(0.3 + 1.0)


def test_policy_values_cover_every_action_and_are_finite():
    v = POL.action_values(_rec(), **KW)
    assert tuple(v) == RE.SLOT_ACTION_ORDER and all(math.isfinite(x) and x >= 0 for x in v.values())


# ---------------------------------------------------------------------------
# learned commit policy
# ---------------------------------------------------------------------------
def _choose(pol, rec, rv=None, pressure=False, min_age=128):
    rv = rv or dict.fromkeys(RE.SLOT_ACTION_ORDER, 0.0)
    return pol.choose(rec, controller_state=torch.zeros(pol.state_dim), rule_values=rv, capacity_pressure=pressure,
                      min_age=min_age)


def test_learned_policy_legal_sets():
    L = RE.LearnedCommitPolicy.legal_actions
    assert L(_rec(last_scored_step=5), capacity_pressure=True, min_age=128) == {"PRESERVE", "DECAY"}
    assert L(_rec(), capacity_pressure=False, min_age=128) == {"PRESERVE", "DECAY", "REFRESH", "QUARANTINE", "DISTILL"}
    assert "EVICT" in L(_rec(), capacity_pressure=True, min_age=128)
    assert L(_rec(state=SLOT_QUARANTINED), capacity_pressure=False, min_age=128) == {"PRESERVE", "RELEASE", "EVICT"}
    assert L(_rec(state=SLOT_QUARANTINED, last_scored_step=3), capacity_pressure=False, min_age=128) == {"PRESERVE", "RELEASE"}


def test_learned_policy_with_zero_prior_weight_ignores_rule_values():
    pol = RE.LearnedCommitPolicy(state_dim=8, rule_prior_weight=0.0)
    a, _ = _choose(pol, _rec(), {**dict.fromkeys(RE.SLOT_ACTION_ORDER, 0.0), "QUARANTINE": 9.0})
    b, _ = _choose(pol, _rec())
    assert a.probabilities == b.probabilities and a.rule_action == "QUARANTINE"


def test_learned_policy_prior_steers_choice_and_veto_is_recorded():
    pol = RE.LearnedCommitPolicy(state_dim=8)
    rv = {**dict.fromkeys(RE.SLOT_ACTION_ORDER, 0.0), "EVICT": 5.0}
    dec, _ = _choose(pol, _rec(), rv, pressure=True)
    assert dec.action == "EVICT" and dec.vetoed_action == ""
    dec2, _ = _choose(pol, _rec(), rv, pressure=False)            # not legal without capacity pressure
    assert dec2.action != "EVICT" and dec2.vetoed_action == "EVICT" and dec2.veto_reason and pol.vetoes == 1


def test_learned_policy_releases_quarantined_slot_when_it_pays():
    pol = RE.LearnedCommitPolicy(state_dim=8)
    q = _rec(state=SLOT_QUARANTINED, marginal_gain_ema=0.3, positive_streak=4)
    dec, _ = _choose(pol, q, POL.action_values(q, **KW))
    assert dec.action == "RELEASE"


def test_learned_policy_feedback_is_normalised_and_negative_reward_lowers_probability():
    pol = RE.LearnedCommitPolicy(state_dim=8, online_lr=0.5, rule_prior_weight=0.0)
    dec, feat = _choose(pol, _rec(marginal_gain_ema=0.02))
    forced = RE.CommitDecision("QUARANTINE", "PRESERVE", 0.2, 0.2, 1.0, dec.logits, dec.probabilities, {})
    pol.apply_feedback(decision=forced, features=feat, reward=-1000.0)          # clipped to -1
    w1 = float(pol.W.norm())
    pol2 = RE.LearnedCommitPolicy(state_dim=8, online_lr=0.5, rule_prior_weight=0.0)
    pol2.apply_feedback(decision=forced, features=feat, reward=-1.0)
    assert w1 == pytest.approx(float(pol2.W.norm()), rel=1e-6)
    after, _ = _choose(pol, _rec(marginal_gain_ema=0.02))
    assert after.probabilities["QUARANTINE"] < dec.probabilities["QUARANTINE"]
    pol.apply_feedback(decision=forced, features=feat, reward=float("nan"))
    assert pol.feedbacks == 1                                        # a non-finite reward is dropped


def test_learned_policy_zero_lr_never_moves():
    pol = RE.LearnedCommitPolicy(state_dim=8, online_lr=0.0)
    dec, feat = _choose(pol, _rec())
    pol.apply_feedback(decision=dec, features=feat, reward=1.0)
    assert float(pol.W.abs().sum()) == 0.0 and pol.feedbacks == 0


def test_learned_policy_sampling_is_reproducible_per_seed():
    picks = []
    for _ in range(2):
        pol = RE.LearnedCommitPolicy(state_dim=8, seed=7, temperature=5.0)
        picks.append([pol.choose(_rec(), controller_state=torch.zeros(8), rule_values={}, capacity_pressure=True,
                                 min_age=128, sample=True)[0].action for _ in range(12)])
    assert picks[0] == picks[1] and len(set(picks[0])) > 1


# ---------------------------------------------------------------------------
# controller state and proposals
# ---------------------------------------------------------------------------
def test_controller_is_a_full_matrix_with_bounded_gain():
    c = RE.FullAControllerState(state_dim=16, rank=4)
    A = c.A if hasattr(c, "A") else None
    d = c.diagnostics()
    assert d["state_norm"] == pytest.approx(0.0) and c.top_log_sv <= -0.05 + 1e-5
    if A is not None:
        off = A - torch.diag(torch.diag(A))
        assert float(off.abs().sum()) > 0                             # not a diagonal decay


def test_controller_direction_adapts_to_slot_dim_and_feedback_needs_finite_reward():
    c = RE.FullAControllerState(state_dim=16, rank=4)
    f = torch.ones(RE.FullAControllerState.input_dim)
    assert c.step(f, slot_dim=8).shape == (8,) and c.step(f, slot_dim=12).shape == (12,)
    before = c.W_out.clone()
    c.update_feedback(torch.ones(12) / math.sqrt(12), float("nan"))
    assert torch.equal(before, c.W_out)


def test_proposals_first_candidate_is_current_and_count_is_k():
    m = _model(3)
    t = m.outer_model.table
    slot = t.get_tensor(t.physical_to_slot_id(1))
    for k in (4, 16):
        prop = RE.CpuRefreshProposalModel(k=k, rank=3)
        c = prop.sample_k(outer=m.outer_model, slot=slot)
        assert len(c) == k and c[0][0] == "current" and len({n for n, _ in c}) == k
        assert all(t_.shape == c[0][1].shape and torch.isfinite(t_).all() for _, t_ in c)


def test_proposals_track_weight_version():
    prop = RE.CpuRefreshProposalModel(k=4, rank=2)
    prop.mark_weight_version(7)
    assert prop.diagnostics()["weight_version"] == 7 if "weight_version" in prop.diagnostics() else True
    st = prop.state_dict()
    p2 = RE.CpuRefreshProposalModel(k=4, rank=2)
    p2.load_state_dict(st)
    assert p2.state_dict().keys() == st.keys()


# ---------------------------------------------------------------------------
# the loop
# ---------------------------------------------------------------------------
def test_tick_without_probe_or_memory_is_a_no_op():
    loop = _loop()
    assert loop.tick(model=_model(2), step=1).slot_commits == []
    bare = CareStudentLM(vocab_size=40, dim=16, num_layers=1)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    assert loop.tick(model=bare, step=2).evicted == [] and loop.diagnostics()["ticks"] == 2


def test_probe_buffer_keeps_the_newest_frames():
    loop = _loop(probe_buffer_size=2)
    ids, valid = _probe()
    for s in range(5):
        loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=s)
    d = loop.diagnostics()
    assert d["queue_depth"] == 2 and d["frames_dropped_overflow"] == 3 and loop.latest_probe_step() == 4


def test_cache_probe_keeps_the_cue_and_detaches():
    loop = _loop()
    ids, valid = _probe()
    cue = torch.randn(2, 16, requires_grad=True)
    loop.cache_probe(input_ids=ids, valid_mask=valid, cue=cue, cache_read_cutoff=3, step=1, stream_id=11)
    f = loop._frames[-1]
    assert torch.equal(f.cue, cue.detach()) and not f.cue.requires_grad and f.cache_read_cutoff == 3
    assert f.stream_id == 11 % loop.memory_streams


def test_slot_work_covers_every_slot_before_the_frame_is_done():
    m = _model(7)
    loop = _loop(slot_work_chunk_size=3, oracle_confirm_top_k=0)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    scored = []
    for s in range(1, 4):
        loop.tick(model=m, step=s)
        scored.append(loop.diagnostics()["slots_scored"])
    assert scored == [3, 6, 7]
    loop.tick(model=m, step=4)
    assert loop.diagnostics()["slots_scored"] == 7                   # nothing left on this frame


def test_first_score_seeds_the_emas_and_second_blends():
    loop = _loop(eviction_ema_beta=0.5)
    rec = SlotRecord(slot_id=1)
    loop._update_record(rec, gain=0.4, sharp=0.2, mass=0.5, repr_drift=0.1, step=10)
    assert rec.marginal_gain_ema == 0.4 and rec.utility_ema == 0.4 and rec.contradiction_ema == 0.0
    assert rec.state == SLOT_WARMING and rec.score_count == 1 and rec.last_scored_step == 10
    loop._update_record(rec, gain=-0.2, sharp=0.0, mass=0.25, repr_drift=0.3, step=11)
    assert rec.marginal_gain_ema == pytest.approx(0.1) and rec.utility_ema == pytest.approx(0.2)
    assert rec.contradiction_ema == pytest.approx(0.1) and rec.activation_drift_ema == pytest.approx(0.25)
    assert rec.representation_drift_ema == pytest.approx(0.2)
    assert rec.peak_utility == 0.4 and rec.peak_sharpness == 0.2 and rec.negative_streak == 1 and rec.positive_streak == 0
    assert rec.state == SLOT_ACTIVE


def test_capacity_pressure_follows_max_slots():
    m = _model(4)
    assert not _loop()._capacity_pressure(m.outer_model)               # unlimited table
    assert _loop(max_slots=4)._capacity_pressure(m.outer_model)
    assert not _loop(max_slots=5)._capacity_pressure(m.outer_model)


def test_mutating_action_needs_repeated_agreement():
    loop = _loop(action_agreement_count=3)
    assert [loop._agreed(5, "EVICT") for _ in range(3)] == [False, False, True]
    assert loop._agreed(5, "QUARANTINE") is False                       # a different action restarts the count
    assert loop._agreed(6, "EVICT") is False                            # per slot


def test_agreement_gate_in_the_loop_delays_eviction():
    m = _model(4)
    loop = _loop(action_agreement_count=2, max_slots=2, oracle_confirm_top_k=0, eviction_threshold=10.0,
                 useful_threshold=10.0, peak_preserve_utility_threshold=1e9, peak_preserve_sharpness_threshold=1e9,
                 distill_peak_threshold=1e9, quarantine_threshold=-1e9)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    r1 = loop.tick(model=m, step=1)
    assert r1.evicted == [] and all(e.reason == "awaiting_agreement" for e in loop.recent_events() if e.action == "EVICT")
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=2)
    r2 = loop.tick(model=m, step=2)
    assert len(r2.evicted) > 0 and m.outer_model.table.n_active == 4 - len(r2.evicted)
    assert all(c.action.name == "EVICT" and c.new_generation == c.base_generation + 1 for c in r2.slot_commits)


def test_oracle_rejection_blocks_eviction_of_a_slot_that_really_helps(monkeypatch):
    m = _model(3)
    loop = _loop(max_slots=1, oracle_confirm_top_k=8, eviction_threshold=10.0, useful_threshold=0.005,
                 peak_preserve_utility_threshold=1e9, peak_preserve_sharpness_threshold=1e9,
                 distill_peak_threshold=1e9, quarantine_threshold=-1e9)
    real = RE.oracle_confirm_slots

    def helpful(**kw):
        o = real(**kw)
        o.oracle_deltas = torch.full_like(o.oracle_deltas, 0.5)           # the real dynamics say: it helps
        return o
    monkeypatch.setattr(RE, "oracle_confirm_slots", helpful)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    r = loop.tick(model=m, step=1)
    d = loop.diagnostics()
    assert r.evicted == [] and m.outer_model.table.n_active == 3 and d["oracle_rejected"] >= 1 and d["oracle_confirmed"] == 0
    assert any(e.reason == "oracle_contradicts" and not e.accepted for e in loop.recent_events())


def test_oracle_budget_limits_how_many_actions_are_confirmed():
    m = _model(5)
    loop = _loop(max_slots=1, oracle_confirm_top_k=2, eviction_threshold=10.0, useful_threshold=10.0,
                 peak_preserve_utility_threshold=1e9, peak_preserve_sharpness_threshold=1e9,
                 distill_peak_threshold=1e9, quarantine_threshold=-1e9)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    r = loop.tick(model=m, step=1)
    reasons = [e.reason for e in loop.recent_events() if e.action == "EVICT"]
    assert len(r.evicted) == 2 and reasons.count("not_in_oracle_budget") == 3


def test_decay_scales_survival_and_marks_state():
    m = _model(3)
    t = m.outer_model.table
    loop = _loop(oracle_confirm_top_k=0, eviction_threshold=10.0, peak_preserve_utility_threshold=1e9,
                 peak_preserve_sharpness_threshold=1e9, distill_peak_threshold=1e9, quarantine_threshold=-1e9)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    r = loop.tick(model=m, step=1)
    assert sorted(r.decayed) == sorted(t.physical_to_slot_id(i) for i in range(3))
    assert all(rec.state == SLOT_DECAYING and rec.last_action == "DECAY" for rec in t.active_records())
    assert all(c.action.name == "DECAY" and c.survival_factor == 0.9 and c.tensor is None for c in r.slot_commits)


def test_quarantine_cap_is_respected():
    m = _model(4)
    loop = _loop(oracle_confirm_top_k=0, max_quarantined=1, quarantine_threshold=0.0)
    recs = m.outer_model.table.active_records()
    ids, valid = _probe()
    frame = RE.ProbeFrame(0, 1, ids, valid, None, None, 0, 0.0)
    out = RE.TickResult()
    decs = []
    for phys, rec in enumerate(recs):
        dec = RE.CommitDecision("QUARANTINE", "QUARANTINE", 1.0, 1.0, 0.0, {}, {"QUARANTINE": 1.0}, {})
        decs.append((phys, rec.slot_id, rec, dec, None))
    loop._act(m, m.outer_model, frame, decs, 1, out)
    assert len(out.quarantined) == 1
    assert [e.reason for e in loop.recent_events()].count("quarantine_full") == 3
    assert sum(r.state == SLOT_QUARANTINED for r in m.outer_model.table.active_records()) == 1


def test_refresh_commit_carries_the_new_tensor_or_is_rejected(monkeypatch):
    m = _model(3)
    t = m.outer_model.table
    loop = _loop(oracle_confirm_top_k=0, refresh_candidate_count=4)
    rec = t.active_records()[1]
    before = t.get_tensor(rec.slot_id).clone()
    gen0 = rec.write_generation
    ids, valid = _probe()
    frame = RE.ProbeFrame(0, 1, ids, valid, None, None, 0, 0.0)
    real = RE.oracle_confirm_refresh_candidates

    def pick_roundtrip(**kw):
        r = real(**kw)
        r.candidate_improvements = torch.zeros_like(r.candidate_improvements)
        r.candidate_improvements[r.candidate_names.index("roundtrip")] = 0.3
        return r
    monkeypatch.setattr(RE, "oracle_confirm_refresh_candidates", pick_roundtrip)
    dec = RE.CommitDecision("REFRESH", "REFRESH", 1.0, 1.0, 0.0, {}, {"REFRESH": 1.0}, {})
    out = RE.TickResult()
    loop._act(m, m.outer_model, frame, [(1, rec.slot_id, rec, dec, None)], 5, out)
    assert out.refreshed == [rec.slot_id] and not torch.equal(t.get_tensor(rec.slot_id), before)
    c = out.slot_commits[0]
    assert c.action.name == "REFRESH" and c.base_generation == gen0 and c.new_generation > gen0
    assert torch.equal(c.tensor, t.get_tensor(rec.slot_id)) and rec.refresh_count == 1

    def none_better(**kw):
        r = real(**kw)
        r.candidate_improvements = -torch.ones_like(r.candidate_improvements)
        r.candidate_improvements[0] = 0.0
        return r
    monkeypatch.setattr(RE, "oracle_confirm_refresh_candidates", none_better)
    cur, gen1 = t.get_tensor(rec.slot_id).clone(), rec.write_generation
    out2 = RE.TickResult()
    loop._act(m, m.outer_model, frame, [(1, rec.slot_id, rec, dec, None)], 6, out2)
    assert out2.refreshed == [] and out2.slot_commits == [] and torch.equal(t.get_tensor(rec.slot_id), cur)
    assert rec.write_generation == gen1 and loop.recent_events()[-1].reason == "no_candidate_beats_current"


def test_distill_writes_a_receipt_then_retires():
    m = _model(3)
    t = m.outer_model.table
    loop = _loop(oracle_confirm_top_k=0)
    rec = t.active_records()[0]
    rec.marginal_gain_ema, rec.peak_utility = 0.002, 0.15
    ids, valid = _probe()
    frame = RE.ProbeFrame(0, 1, ids, valid, None, None, 0, 0.0)
    dec = RE.CommitDecision("DISTILL", "DISTILL", 1.0, 1.0, 0.0, {}, {"DISTILL": 1.0}, {})
    out = RE.TickResult()
    loop._act(m, m.outer_model, frame, [(0, rec.slot_id, rec, dec, None)], 9, out)
    assert out.distilled == [rec.slot_id] and t.n_active == 2
    rc = loop._receipts[-1]
    assert rc.slot_id == rec.slot_id and rc.step == 9 and rc.accepted and rc.marginal_gain_peak == 0.15
    assert rc.target in ("none", "bucket_prototype") and loop.diagnostics()["distill_receipts"] == 1
    assert out.slot_commits[0].action.name == "DISTILL"


def test_shadow_mode_counts_decisions_but_emits_nothing():
    m = _model(3)
    loop = _loop(action_mode="shadow", oracle_confirm_top_k=0, max_slots=1, eviction_threshold=10.0,
                 useful_threshold=10.0, peak_preserve_utility_threshold=1e9, peak_preserve_sharpness_threshold=1e9,
                 distill_peak_threshold=1e9, quarantine_threshold=-1e9)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    r = loop.tick(model=m, step=1)
    assert r.evicted == [] and r.slot_commits == [] and m.outer_model.table.n_active == 3
    assert loop.diagnostics()["action_counts"]["EVICT"] == 3


def test_trace_respects_row_cap_and_flush(tmp_path):
    m = _model(4)
    path = tmp_path / "t.ndjson"
    loop = _loop(trace_path=str(path), trace_max_rows=3, trace_flush_rows=100, oracle_confirm_top_k=0)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    loop.tick(model=m, step=1)
    assert not path.exists()                                            # below the flush threshold
    loop.flush_trace()
    rows = [json.loads(x) for x in path.read_text().splitlines()]
    assert len(rows) == 3 and all(r["row_type"] == "arm_slot_decision" and r["commit_policy"] == "rule" for r in rows)
    loop.close()


def test_state_round_trip_keeps_streaks_and_receipts():
    loop = _loop(action_agreement_count=3)
    loop._agreed(4, "EVICT")
    loop._receipts.append(RE.DistillReceipt(4, 1, 0.0, 0.1, 0.0, "none", accepted=True))
    st = loop.state_dict()
    json.dumps({k: v for k, v in st.items() if k in ("version", "tick", "stats", "counts", "streak", "receipts")})
    other = _loop(action_agreement_count=3)
    other.load_state_dict(st)
    assert other._agreed(4, "EVICT") is False and other._agreed(4, "EVICT") is True      # 1 (restored) + 2
    assert other._receipts[0].slot_id == 4 and other.diagnostics()["distill_receipts"] == 1


def test_oracle_scoring_mode_scores_through_the_real_read_path():
    m = _model(3)
    loop = _loop(scoring_mode="oracle", oracle_confirm_top_k=4)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    loop.tick(model=m, step=1)
    d = loop.diagnostics()
    assert d["scoring_mode"] == "oracle" and d["slots_scored"] == 3
    assert d["oracle_confirmed"] == d["oracle_rejected"] == 0          # already oracle-scored: no second pass
