"""Residual-memory maintenance: probes against hand computation, policies, and the tick loop."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200 import replay_eviction as RE
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.slot_table import SLOT_QUARANTINED, SlotRecord


def _model(n_slots=5, seed=0):
    torch.manual_seed(seed)
    m = CareStudentLM(vocab_size=40, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                      outer_max_slots=0, buffer_mode="append_only")
    hidden = torch.randn(1, n_slots, 16)
    m.append_memory_from_hidden(hidden, event_ids=torch.arange(1, n_slots + 1).view(1, -1))
    return m.eval()


def _probe(B=2, T=9, seed=1):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 40, (B, T), generator=g)
    return ids, torch.ones(B, T, dtype=torch.bool)


def test_counterfactual_probe_matches_direct_recomputation():
    m = _model()
    outer = m.outer_model
    ids, valid = _probe()
    r = RE.counterfactual_probe(model=m, outer=outer, probe_input_ids=ids, probe_valid_mask=valid, chunk_size=3)
    assert r.marginal_gains.shape == (5, 2, 8) and r.slot_indices == [0, 1, 2, 3, 4]
    with torch.no_grad():
        x, y = ids[:, :-1], ids[:, 1:]
        h = m.encode(x, memory_mode="off")
        M = outer.table.slot_matrix()
        q = outer.cue_proj(h.mean(1))

        def nll(mat):
            w = F.softmax(q @ mat.T, -1) if mat.numel() else None
            rr = w @ mat if w is not None else torch.zeros(2, 8)
            hv = h + outer.decoder(rr).unsqueeze(1)
            lg = m.lm_head(m.final_norm(hv))
            return F.cross_entropy(lg.reshape(-1, 40), y.reshape(-1), reduction="none").view(2, 8)

        base = nll(M)
        assert torch.allclose(r.nll_baseline, base, atol=2e-2)
        assert torch.allclose(r.sidecar_value, nll(M[:0]) - base, atol=2e-2)
        keep = [0, 1, 3, 4]
        assert torch.allclose(r.marginal_gains[2], nll(M[keep]) - base, atol=2e-2)
    sub = RE.counterfactual_probe(model=m, outer=outer, probe_input_ids=ids, probe_valid_mask=valid,
                                  score_slot_indices=[3, 1, 99])
    assert sub.slot_indices == [3, 1] and torch.allclose(sub.marginal_gains[0], r.marginal_gains[3], atol=1e-5)
    cut = RE.counterfactual_probe(model=m, outer=outer, probe_input_ids=ids, probe_valid_mask=valid, cache_read_cutoff=2)
    assert cut.slot_indices == [0, 1]
    s = RE.replay_score_slots(model=m, probe_input_ids=ids, probe_valid_mask=valid)
    assert s["slot_utilities"].shape == (5,) and s["n_tokens_scored"] == 16
    plain = CareStudentLM(vocab_size=40, dim=16, num_layers=1)
    assert RE.replay_score_slots(model=plain, probe_input_ids=ids, probe_valid_mask=valid)["slot_indices"] == []


def test_oracle_passes_use_the_real_read_path():
    m = _model()
    outer = m.outer_model
    ids, valid = _probe()
    o = RE.oracle_confirm_slots(model=m, outer=outer, probe_input_ids=ids, probe_valid_mask=valid,
                                slot_indices=[1, 4, 4, 77], variant_chunk_size=2)
    assert o.slot_indices == [1, 4] and o.oracle_deltas.shape == (2, 2, 8)
    with torch.no_grad():
        x, y = ids[:, :-1], ids[:, 1:]
        mask = torch.ones(2, 5, dtype=torch.bool)
        mask[:, 4] = False
        hid = m.encode(x, memory_mode="force_on", memory_slot_mask=mask)
        nll = F.cross_entropy(m.lm_head(m.final_norm(hid)).reshape(-1, 40), y.reshape(-1), reduction="none").view(2, 8)
        assert torch.allclose(o.oracle_deltas[1], nll - o.nll_baseline, atol=2e-2)
    cur = outer.table.get_tensor(outer.table.physical_to_slot_id(2))
    r = RE.oracle_confirm_refresh_candidates(model=m, outer=outer, probe_input_ids=ids, probe_valid_mask=valid,
                                             slot_index=2, candidate_tensors=[("current", cur), ("zero", cur * 0),
                                                                              ("flip", -cur)], variant_chunk_size=2)
    assert r.candidate_names == ["current", "zero", "flip"] and r.chunk_count == 2 and r.variants_total == 3
    assert float(r.candidate_improvements[0]) == 0.0
    base_score = ((o.nll_no_sidecar - o.nll_baseline) * 1.0).mean()
    assert float(r.candidate_scores[0]) == pytest.approx(float(base_score), abs=2e-2)
    with pytest.raises(ValueError):
        RE.oracle_confirm_refresh_candidates(model=m, outer=outer, probe_input_ids=ids, probe_valid_mask=valid,
                                             slot_index=2, candidate_tensors=[("bad", torch.zeros(2, 8))])
    empty = RE.oracle_confirm_slots(model=m, outer=outer, probe_input_ids=ids, probe_valid_mask=valid, slot_indices=[])
    assert empty.slot_indices == []


def _rec(**kw):
    base = dict(slot_id=1, created_step=0, last_scored_step=500, score_count=5)
    base.update(kw)
    return SlotRecord(**base)


_KW = dict(eviction_threshold=0.01, useful_threshold=0.005, drift_threshold=0.3, quarantine_threshold=-0.01,
           distill_peak_threshold=0.04, peak_preserve_utility_threshold=0.2, peak_preserve_sharpness_threshold=0.2,
           min_age=128)


def test_rule_policy_cases():
    pol = RE.MaintenancePolicy()
    assert pol.choose(_rec(marginal_gain_ema=0.1, utility_ema=0.1, peak_utility=0.1), **_KW) == "PRESERVE"
    assert pol.choose(_rec(utility_ema=0.0), capacity_pressure=True, **_KW) == "EVICT"
    assert pol.choose(_rec(utility_ema=0.0), capacity_pressure=False, **_KW) == "DECAY"
    assert pol.choose(_rec(utility_ema=0.0, peak_utility=0.5), capacity_pressure=True, **_KW) != "EVICT"   # protected
    assert pol.choose(_rec(contradiction_ema=0.3, negative_streak=3), **_KW) == "QUARANTINE"
    assert pol.choose(_rec(marginal_gain_ema=0.05, utility_ema=0.05, representation_drift_ema=0.6), **_KW) == "REFRESH"
    assert pol.choose(_rec(marginal_gain_ema=0.001, utility_ema=0.05, peak_utility=0.15), **_KW) == "DISTILL"
    assert pol.choose(_rec(state=SLOT_QUARANTINED, marginal_gain_ema=0.3, positive_streak=4, utility_ema=0.3), **_KW) == "RELEASE"
    young = _rec(last_scored_step=10, contradiction_ema=0.3)
    assert pol.action_values(young, **_KW)["QUARANTINE"] == 0.0


def test_learned_policy_masks_learns_and_round_trips():
    pol = RE.LearnedCommitPolicy(state_dim=8, online_lr=0.5, rule_prior_weight=0.0)
    rec = _rec(marginal_gain_ema=0.02)
    rv = dict.fromkeys(RE.SLOT_ACTION_ORDER, 0.0)
    dec, feat = pol.choose(rec, controller_state=torch.zeros(8), rule_values=rv, capacity_pressure=False, min_age=128)
    assert dec.probabilities["EVICT"] == 0.0 and dec.probabilities["RELEASE"] == 0.0
    assert abs(sum(dec.probabilities.values()) - 1.0) < 1e-6 and dec.entropy > 0
    young = _rec(last_scored_step=5)
    d2, _ = pol.choose(young, controller_state=torch.zeros(8), rule_values=rv, capacity_pressure=True, min_age=128)
    assert set(k for k, v in d2.probabilities.items() if v > 0) == {"PRESERVE", "DECAY"}
    forced = RE.CommitDecision("REFRESH", "PRESERVE", 0.2, 0.2, 1.0, dec.logits, dec.probabilities, rv)
    for _ in range(20):
        pol.apply_feedback(decision=forced, features=feat, reward=1.0)
    d3, _ = pol.choose(rec, controller_state=torch.zeros(8), rule_values=rv, capacity_pressure=False, min_age=128)
    assert d3.probabilities["REFRESH"] > dec.probabilities["REFRESH"]
    other = RE.LearnedCommitPolicy(state_dim=8)
    other.load_state_dict(pol.state_dict())
    assert torch.equal(other.W, pol.W) and other.feedbacks == pol.feedbacks
    with pytest.raises(ValueError):
        RE.LearnedCommitPolicy(state_dim=4).load_state_dict(pol.state_dict())


def test_controller_state_and_refresh_proposals():
    c = RE.FullAControllerState(state_dim=16, rank=4)
    assert c.top_log_sv <= -0.05 + 1e-5
    for _ in range(300):
        d = c.step(torch.full((12,), 50.0), slot_dim=8)
    assert d.shape == (8,) and abs(float(d.norm()) - 1) < 1e-4 and c.diagnostics()["state_norm"] <= 8.0 + 1e-4
    before = c.W_out.clone()
    c.update_feedback(d, 1.0)
    assert not torch.equal(before, c.W_out)
    c2 = RE.FullAControllerState(state_dim=16, rank=4)
    c2.load_state_dict(c.state_dict())
    assert torch.equal(c2.h, c.h) and torch.equal(c2.W_out, c.W_out)
    m = _model()
    prop = RE.CpuRefreshProposalModel(k=8, rank=3)
    slot = m.outer_model.table.get_tensor(m.outer_model.table.physical_to_slot_id(0))
    cands = prop.sample_k(outer=m.outer_model, slot=slot, cue_outer=torch.randn(8), controller_direction=torch.randn(8))
    assert len(cands) == 8 and cands[0][0] == "current" and torch.allclose(cands[0][1], slot.float().cpu().reshape(1, -1))
    assert {"roundtrip", "cue_blend", "controller_dir"} <= {n for n, _ in cands}
    basis0 = prop.basis.clone()
    prop.update(slot=slot, accepted=cands[5][1], improvement=0.3)
    assert prop.accepted == 1 and not torch.equal(basis0, prop.basis)
    prop.update(slot=slot, accepted=None, improvement=0.0)
    p2 = RE.CpuRefreshProposalModel(k=8, rank=3)
    p2.load_state_dict(prop.state_dict())
    assert torch.equal(p2.basis, prop.basis)


@pytest.mark.parametrize("policy", ["rule", "learned"])
def test_tick_loop_scores_acts_and_traces(tmp_path, policy):
    m = _model(n_slots=6)
    outer = m.outer_model
    trace = tmp_path / "arm" / "trace.ndjson"
    loop = RE.ReplayEvictionLoop(commit_policy=policy, min_slot_age_steps=0, slot_work_chunk_size=4,
                                 action_agreement_count=1, max_slots=4, trace_path=str(trace), trace_flush_rows=1,
                                 max_seconds_per_tick=0.0, oracle_confirm_top_k=8)
    assert not loop.has_probe() and loop.tick(model=m, step=1).slot_commits == []
    ids, valid = _probe()
    touched = set()
    for step in range(2, 12):
        loop.cache_probe(input_ids=ids, valid_mask=valid, cue=None, cache_read_cutoff=None, step=step, stream_id=step)
        r = loop.tick(model=m, step=step)
        touched |= set(r.evicted) | set(r.decayed) | set(r.refreshed) | set(r.quarantined) | set(r.distilled)
        for c in r.slot_commits:
            assert c.new_generation >= c.base_generation
    d = loop.diagnostics()
    assert d["slots_scored"] >= 6 and d["frames_ingested"] == 10 and sum(d["action_counts"].values()) > 0
    recs = outer.table.active_records()
    assert all(rec.score_count > 0 for rec in recs)
    rows = [json.loads(l) for l in trace.read_text().splitlines()]
    assert rows and rows[0]["row_type"] == "arm_slot_decision" and {"action", "rule_action", "accepted"} <= set(rows[0])
    assert loop.latest_probe_step() == 11
    clone = RE.ReplayEvictionLoop(commit_policy=policy)
    clone.load_state_dict(loop.state_dict())
    assert clone.diagnostics()["tick"] == d["tick"] and clone.diagnostics()["action_counts"] == d["action_counts"]
    with pytest.raises(ValueError):
        clone.load_state_dict({"version": 9})
    loop.close()


def test_shadow_mode_never_mutates_and_stale_frames_drop():
    m = _model(n_slots=4)
    table = m.outer_model.table
    before = table.slot_matrix().clone()
    loop = RE.ReplayEvictionLoop(action_mode="shadow", commit_policy="rule", min_slot_age_steps=0, max_slots=2,
                                 action_agreement_count=1, frame_ttl_steps=3, max_seconds_per_tick=0.0)
    ids, valid = _probe()
    loop.cache_probe(input_ids=ids, valid_mask=valid, cache_read_cutoff=None, step=1)
    for step in range(1, 4):
        r = loop.tick(model=m, step=step)
        assert not r.slot_commits and not r.evicted
    assert torch.equal(table.slot_matrix(), before) and table.n_active == 4
    loop.tick(model=m, step=50)
    assert loop.diagnostics()["frames_dropped_stale"] == 1 and not loop.has_probe()
    for bad in (dict(action_mode="x"), dict(scoring_mode="x"), dict(commit_policy="x")):
        with pytest.raises(ValueError):
            RE.ReplayEvictionLoop(**bad)
    ids_evict = RE._evict_slots(m.outer_model, [0, 2])
    assert len(ids_evict) == 2 and table.n_active == 2


def test_tick_loop_with_native_scheduler_and_evidence_engine():
    m = _model(n_slots=6)
    loop = RE.ReplayEvictionLoop(commit_policy="rule", min_slot_age_steps=0, slot_work_chunk_size=4,
                                 action_agreement_count=1, max_seconds_per_tick=0.0, arm_runtime_enabled=True,
                                 evidence_engine_enabled=True, evidence_engine_d_model=16, evidence_engine_lanes=2)
    loop.refresh_evidence_weights(m)
    ids, valid = _probe(T=40)
    for step in range(1, 5):
        loop.cache_probe(input_ids=ids, valid_mask=valid, cue=torch.randn(2, 16), cache_read_cutoff=None, step=step,
                         stream_id=step)
        loop.tick(model=m, step=step)
    d = loop.diagnostics()
    assert d["arm_runtime"]["jobs_emitted"] >= 2 and d["arm_runtime"]["results_recorded"] == d["arm_runtime"]["jobs_emitted"]
    assert d["arm_runtime"]["slots_scored_total"] == d["slots_scored"] >= 6
    ev = d["evidence_engine"]
    assert ev["frames_ingested"] == 4 and ev["cue_nll_calls_total"] == 4 and ev["last_cue_nll_mean"] > 0
    loop.close()
