"""Temporal-head mixtures and chunk scoring (cf. tests/test_temporal_heads.py of the reference)."""
import math

import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200.eval_stream.temporal_heads import (
    PreviousChunkPriorityGate, TemporalHeadConfig, make_same_horizon_virtual_depth_config,
    online_exp_weighted_logprob_mixture, score_temporal_heads_chunk, uniform_logprob_mixture,
    update_online_exp_weighted_log_weights, weighted_logprob_mixture)
from chaoscontrol_b200.models.model import CareStudentLM


def _lp(*shape, seed=0):
    g = torch.Generator().manual_seed(seed)
    return F.log_softmax(torch.randn(*shape, generator=g), dim=-1)


def test_uniform_and_weighted_mixtures_are_probability_space():
    a, b = _lp(2, 5, 7, seed=1), _lp(2, 5, 7, seed=2)
    mix = uniform_logprob_mixture([a, b])
    assert torch.allclose(mix.exp(), 0.5 * (a.exp() + b.exp()), atol=1e-6)
    w = weighted_logprob_mixture([a, b], weights=(3.0, 1.0))
    assert torch.allclose(w.exp(), 0.75 * a.exp() + 0.25 * b.exp(), atol=1e-6)
    assert uniform_logprob_mixture([a]) is a
    with pytest.raises(ValueError):
        weighted_logprob_mixture([a, b], weights=(1.0, 0.0))
    with pytest.raises(ValueError):
        weighted_logprob_mixture([a, b], weights=(1.0,))


def test_online_mixture_matches_token_loop_and_is_causal():
    heads = [_lp(3, 9, 11, seed=s) for s in range(3)]
    targets = torch.randint(0, 11, (3, 8), generator=torch.Generator().manual_seed(5))
    mixed = online_exp_weighted_logprob_mixture(heads, targets, eta=0.7, initial_weights=(1.0, 2.0, 1.0))
    lw = torch.tensor([0.25, 0.5, 0.25]).log().expand(3, 3).clone()
    for pos in range(9):
        ref = torch.logsumexp(torch.stack([h[:, pos] for h in heads], 1) + lw.unsqueeze(-1), dim=1)
        assert torch.allclose(mixed[:, pos], ref, atol=1e-5), pos
        if pos < 8:
            lw = update_online_exp_weighted_log_weights(lw, [h[:, pos] for h in heads], targets[:, pos], eta=0.7)
    # causality: changing a later target cannot change earlier mixed positions
    t2 = targets.clone()
    t2[:, 5] = (t2[:, 5] + 1) % 11
    mixed2 = online_exp_weighted_logprob_mixture(heads, t2, eta=0.7, initial_weights=(1.0, 2.0, 1.0))
    assert torch.equal(mixed[:, :6], mixed2[:, :6])
    assert not torch.allclose(mixed[:, 6:], mixed2[:, 6:])
    with pytest.raises(ValueError):
        online_exp_weighted_logprob_mixture(heads, targets[:, :-1], eta=0.7)
    with pytest.raises(ValueError):
        online_exp_weighted_logprob_mixture(heads, targets, eta=-1.0)


def test_priority_gate():
    gate = PreviousChunkPriorityGate(threshold=1.0, use_disagreement_ema=True, disagreement_weight=2.0,
                                     disagreement_decay=0.5)
    assert not gate.should_run(extra_cost_seconds=0.1, slack_remaining_seconds=10.0)
    gate.update_after_chunk(entropy=0.2, loss_spike=0.1, state_delta_norm=0.1, head_disagreement=1.0,
                            temporal_heads_ran=True)
    assert math.isclose(gate._priority, 0.4 + 2.0 * 0.5)
    assert gate.should_run(extra_cost_seconds=0.1, slack_remaining_seconds=10.0)
    assert not gate.should_run(extra_cost_seconds=11.0, slack_remaining_seconds=10.0)
    gate.update_after_chunk(entropy=0.2, loss_spike=0.1, state_delta_norm=0.1)
    assert math.isclose(gate._priority, 0.4 + 2.0 * 0.25)


def _model():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=64, dim=16, num_layers=2, ff_mult=2, a_mode="diag")


@pytest.mark.parametrize("mixer", ["uniform_logprob", "base_prior_logprob", "online_exp_weights_logprob"])
def test_score_chunk(mixer):
    model = _model()
    before = [c.log_a.detach().clone() for c in (blk.core for blk in model.layers)]
    chunk = torch.randint(0, 64, (2, 12))
    cfg = TemporalHeadConfig(mixer=mixer, online_eta=0.5)
    res = score_temporal_heads_chunk(model, chunk, states_by_shift={}, cfg=cfg)
    assert res.tokens_scored == 22 and math.isfinite(res.loss_nats)
    assert set(res.per_head_loss_nats) == {-0.5, 0.0, 0.5}
    assert sum(res.winner_counts_by_shift.values()) == 22
    # mixture is never worse than the worst head, never better than the per-token oracle
    assert res.loss_nats <= max(res.per_head_loss_nats.values()) + 1e-4
    for blk, b in zip(model.layers, before):
        assert torch.equal(blk.core.log_a, b)
    hl = res.half_life_stats_by_shift
    assert hl[0.5][0]["median"] < hl[0.0][0]["median"] < hl[-0.5][0]["median"]
    assert set(res.state_divergence_by_shift) == {-0.5, 0.5}
    assert (res.online_final_log_weights is not None) == (mixer == "online_exp_weights_logprob")
    # carrying state + online weights into the next chunk
    res2 = score_temporal_heads_chunk(model, chunk, states_by_shift=res.final_states_by_shift, cfg=cfg,
                                      online_initial_log_weights=res.online_final_log_weights,
                                      capture_half_lives=False)
    assert res2.half_life_stats_by_shift[0.0][0]["median"] is None
    assert math.isfinite(res2.loss_nats)


def test_head_ids_and_virtual_depth_config():
    model = _model()
    chunk = torch.randint(0, 64, (1, 6))
    with pytest.raises(ValueError):
        score_temporal_heads_chunk(model, chunk, states_by_shift={}, cfg=TemporalHeadConfig(horizon_shifts=(0.0, 0.0)))
    cfg = TemporalHeadConfig(horizon_shifts=(0.0, 0.0), head_ids=("a", "b"))
    res = score_temporal_heads_chunk(model, chunk, states_by_shift={}, cfg=cfg)
    assert math.isclose(res.per_head_loss_nats["a"], res.per_head_loss_nats["b"], rel_tol=1e-6)
    assert math.isclose(res.loss_nats, res.per_head_loss_nats["a"], rel_tol=1e-5)
    out = make_same_horizon_virtual_depth_config({"num_layers": 3}, depth_recurrence_count=3)
    assert out["depth_recurrence_shared_layers"] == [0, 1, 2] and out["depth_recurrence_count"] == 3
    with pytest.raises(ValueError):
        make_same_horizon_virtual_depth_config({"num_layers": 3}, depth_recurrence_count=0)
